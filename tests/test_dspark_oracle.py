"""DSpark draft stages in the CPU oracle (reference semantics: docs/architecture/05-dspark.md sections 2-7)."""
import copy

import torch

from sparkflash_b200.config import tiny_config
from sparkflash_b200.models.deepseek_v41 import oracle as O, weights as W


def test_draft_block_semantics():
    cfg = tiny_config()
    w = W.dequantize_checkpoint(W.synthetic_checkpoint(cfg, 0), cfg)
    orc = O.Oracle(cfg, w)
    st = orc.new_state()
    prompt = list(range(40, 40 + 14))
    logits = orc.prefill(st, prompt)
    # every backbone position seeded one window key per stage, bounded by the window
    for s in range(cfg.n_mtp_stages):
        assert sorted(st.layers[cfg.n_layers + s].window) == list(range(max(0, 14 - cfg.window), 14))
    anchor = int(logits.argmax())
    before = copy.deepcopy(st)
    toks, conf, lg = orc.draft(st, anchor)
    assert len(toks) == cfg.dspark_block == len(conf) and lg.shape == (cfg.dspark_block, cfg.vocab_size)
    assert all(0 <= t < cfg.vocab_size for t in toks) and all(abs(c) < 50 for c in conf)
    # drafting leaves the sequence state untouched and is deterministic
    assert st.pos == before.pos and st.tokens == before.tokens
    for a, b in zip(st.layers, before.layers):
        assert a.window.keys() == b.window.keys() and len(a.comp_kv) == len(b.comp_kv)
    assert orc.draft(st, anchor)[0] == toks
    # the block is not causal: changing the anchor changes every position's logits, not just the first
    lg2 = orc.draft(st, (anchor + 1) % cfg.vocab_size)[2]
    assert all(not torch.equal(lg[i], lg2[i]) for i in range(cfg.dspark_block))
    # sampling is coupled to the verifier's noise by position: greedy equals temperature -> 0
    assert orc.draft(st, anchor, temperature=1e-6, seed=5)[0] == toks
    # verification by the backbone: accepted drafts are exactly the prefix that matches what the backbone samples
    cur, accepted = anchor, 0
    for t in toks:
        nxt = int(orc.step(st, cur).argmax())
        if nxt != t:
            break
        accepted, cur = accepted + 1, t
    assert 0 <= accepted <= cfg.dspark_block

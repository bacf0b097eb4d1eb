"""Whole-model checks of the other families: each has a full-sequence fp32 oracle and an incremental (cached / recurrent /
ring / device) forward over the same weights, and the two must agree."""
import multiprocessing as mp
import os

import pytest
import torch


def test_glm_sparse_mla_cached_decode_matches_full_recompute():
    from sparkflash_b200.models import glm as G
    c = G.GlmConfig()
    w = G.init_weights(c, 1)
    toks = torch.randint(0, c.vocab, (20,), generator=torch.Generator().manual_seed(2)).tolist()
    want = G.reference_logits(c, w, toks)
    eng = G.CachedEngine(c, w)
    got = torch.cat([eng.step(toks[:7]), eng.step(toks[7:15])] + [eng.step([t]) for t in toks[15:]])
    assert (got - want).abs().max() < 2e-4 * (1 + want.abs().max())
    assert all(len(s) == c.index_topk for s in eng.selected)          # 20 positions > top-8: attention really is sparse
    # with the selection wide open the model is plain MLA: the sparse and the dense logits differ, both are self-consistent
    dense = G.GlmConfig(index_topk=1000)
    assert (G.reference_logits(dense, w, toks) - want).abs().max() > 1e-3
    e2 = G.CachedEngine(dense, w)
    assert (e2.step(toks) - G.reference_logits(dense, w, toks)).abs().max() < 2e-4 * (1 + want.abs().max())


def test_glm_selection_ties_go_to_the_lower_position():
    from sparkflash_b200.models.glm import index_select
    s = torch.tensor([1.0, 3.0, 3.0, 0.5, 3.0])
    assert index_select(s, 5, 2).tolist() == [1, 2] and index_select(s, 3, 8).tolist() == [0, 1, 2]


@pytest.mark.parametrize("kda", [False, True])
def test_qwen_hybrid_oracle_is_causal_and_chunking_free(kda):
    from sparkflash_b200.models import qwen as Q
    c = Q.HybridConfig(kda=kda)
    w = Q.init_weights(c, 3)
    toks = torch.randint(0, c.vocab, (12,), generator=torch.Generator().manual_seed(4)).tolist()
    full = Q.reference_logits(c, w, toks)
    assert full.shape == (12, c.vocab) and torch.isfinite(full).all()
    # a prefix gives the same logits for its positions (recurrent layers, convolution history and attention are causal)
    assert (Q.reference_logits(c, w, toks[:7]) - full[:7]).abs().max() < 1e-4
    other = toks[:7] + [(t + 1) % c.vocab for t in toks[7:]]
    assert (Q.reference_logits(c, w, other)[:7] - full[:7]).abs().max() < 1e-4


@pytest.mark.parametrize("mode", ["experts", "intermediate", "rows"])
def test_inkling_expert_splits_agree_with_the_unsplit_layer(mode):
    from sparkflash_b200.models import inkling as I
    c = I.InklingConfig()
    w = I.init_weights(c, 5)
    x = torch.randn(6, c.d, generator=torch.Generator().manual_seed(6))
    want = I.moe(c, w, "l0.", x)
    for world in (2, 4):
        got, parts = I.moe_split(c, w, "l0.", x, world, mode)
        assert len(parts) == world and (got - want).abs().max() < 1e-4 * (1 + want.abs().max())
        if mode == "rows":
            assert parts[0].shape == (6, c.d // world)
        if mode == "experts":       # a rank that owns none of a token's experts contributes exactly zero for it
            assert any((p.abs().sum(-1) == 0).any() for p in parts)
    toks = list(range(3, 17))
    assert (I.reference_logits(c, w, toks, world=2, split=mode) - I.reference_logits(c, w, toks)).abs().max() < 1e-3
    assert I.reference_logits(c, w, toks).abs().max() <= c.logit_cap


def test_inkling_window_limits_what_a_position_sees():
    from sparkflash_b200.models import inkling as I
    c = I.InklingConfig(layers=1, window=4, conv_width=2)
    w = I.init_weights(c, 7)
    a = list(range(10, 22))
    b = [99] + a[1:]                          # differs only at position 0
    la, lb = I.reference_logits(c, w, a), I.reference_logits(c, w, b)
    assert (la[3] - lb[3]).abs().max() > 1e-4          # inside the window (+ convolution reach) of position 0
    assert (la[8:] - lb[8:]).abs().max() < 1e-5         # one layer: nothing beyond window + convolution reach


def test_dory_steps_match_the_full_sequence_and_loops_split_anywhere():
    from sparkflash_b200.models import dory as D
    c = D.DoryConfig()
    w = D.init_weights(c, 8)
    toks = torch.randint(0, c.vocab, (9,), generator=torch.Generator().manual_seed(9)).tolist()
    want = D.reference_logits(c, w, toks)
    st = D.LoopStage(c, w)
    got = torch.cat([st.logits(0, 0, st.stage(0, 0, st.embed(toks[:5])))] +
                    [st.logits(0, 5 + i, st.stage(0, 5 + i, st.embed([t]))) for i, t in enumerate(toks[5:])])
    assert (got - want).abs().max() < 1e-4 * (1 + want.abs().max())
    # three stages chained by hand = what the ring does: same logits
    stages = [D.LoopStage(c, w, r, 3) for r in range(3)]
    assert [list(s.loops) for s in stages] == [[0, 1], [2, 3], [4, 5]]
    f = stages[0].embed(toks)
    for s in stages:
        f = s.stage(0, 0, f)
    assert (stages[2].logits(0, 0, f) - want).abs().max() < 1e-4 * (1 + want.abs().max())


def _dory_ring(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from sparkflash_b200.models import dory as D
    dist.init_process_group("gloo", rank=rank, world_size=world)
    c = D.DoryConfig()
    w = D.init_weights(c, 8)
    out = D.ring_generate(c, w, {0: [5, 6, 7, 8], 1: [9, 10], 2: [11, 12, 13]}, 5)
    if rank == 0:
        q.put(out)
    dist.barrier()
    dist.destroy_process_group()


def test_dory_ring_generation_matches_one_process():
    from sparkflash_b200.models import dory as D
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_dory_ring, args=(r, 3, 29747, q)) for r in range(3)]
    [p.start() for p in ps]
    got = q.get(timeout=90)
    [p.join(20) for p in ps]
    c = D.DoryConfig()
    w = D.init_weights(c, 8)
    for lane, prompt in {0: [5, 6, 7, 8], 1: [9, 10], 2: [11, 12, 13]}.items():
        assert got[lane] == D.generate(c, w, prompt, 5), lane


class _ToyTarget:
    """A deterministic 'model': next token = (3 * token + position) % vocab; feature = one-hot-ish code of (token, position)."""

    def __init__(self, c):
        self.c, self.calls = c, []

    def step(self, tokens, pos):
        self.calls.append((pos, len(tokens)))
        nxt = [(3 * t + pos + i) % self.c.vocab for i, t in enumerate(tokens)]
        feats = torch.stack([torch.sin(torch.arange(self.c.feat) * (0.1 + t) + pos + i) for i, t in enumerate(tokens)])
        return nxt, feats


def test_dflash_block_drafter_ring_and_acceptance():
    from sparkflash_b200.models import dflash as F
    c = F.DFlashConfig()
    w = F.init_weights(c, 10)
    d = F.BlockDrafter(c, w)
    ring = F.FeatureRing(c)
    feats = torch.randn(40, c.feat, generator=torch.Generator().manual_seed(11))
    ring.write(0, 0, feats)
    assert torch.equal(ring.window(0), feats[-c.ring:])                 # wrapped: the last `ring` positions, oldest first
    ring.rewind(0, 38)                                                   # two rejected positions: the window slides back
    assert torch.equal(ring.window(0)[2:], feats[24:38]) and ring.window(0).shape[0] == c.ring
    p = d.propose(7, feats[-c.ring:])
    assert len(p) == c.block - 1 and p == d.propose(7, feats[-c.ring:])
    assert (d.logits(7, feats[:c.ring]) - d.logits(7, feats[-c.ring:])).abs().max() > 1e-3     # it reads the features
    assert F.accept([4, 5, 6, 7], [4, 5, 9, 1, 2]) == (2, [4, 5, 9])
    assert F.accept([4, 5, 6, 7], [4, 5, 6, 7, 8]) == (4, [4, 5, 6, 7, 8])
    assert F.accept([4, 5], [1, 2, 3]) == (0, [1])
    # the loop emits exactly what the target alone would, whatever the drafter proposes
    tgt = _ToyTarget(c)
    out, forwards = F.speculate(tgt, d, F.FeatureRing(c), 0, 5, 0, 12)
    want, tok = [], 5
    for pos in range(12):
        tok = (3 * tok + pos) % c.vocab
        want.append(tok)
    assert out == want and forwards <= 12


@pytest.mark.gpu
def test_qwen_hybrid_device_rows_match_the_oracle():
    from sparkflash_b200.models import qwen as Q
    for kda in (False, True):
        c = Q.HybridConfig(kda=kda)
        w = Q.init_weights(c, 3)
        g = torch.Generator().manual_seed(12)
        seqs = {0: torch.randint(0, c.vocab, (11,), generator=g).tolist(), 1: torch.randint(0, c.vocab, (8,), generator=g).tolist()}
        want = {l: Q.reference_logits(c, w, s) for l, s in seqs.items()}
        eng = Q.HybridEngine(c, w, lanes=2, max_context=32)
        # step 1: a prefill chunk of lane 0 and one of lane 1 in the same launch; then decode rows of both lanes together
        got = {0: [], 1: []}
        out = eng.step(seqs[0][:6] + seqs[1][:4], [0] * 6 + [1] * 4, list(range(6)) + list(range(4))).cpu()
        got[0].append(out[:6]); got[1].append(out[6:])
        for i in range(4):
            out = eng.step([seqs[0][6 + i], seqs[1][4 + i]], [0, 1], [6 + i, 4 + i]).cpu()
            got[0].append(out[:1]); got[1].append(out[1:])
        for l in (0, 1):
            have = torch.cat(got[l])
            ref = want[l][:have.shape[0]]
            assert (have - ref).abs().max() < 0.03 * (1 + ref.abs().max()), (kda, l, (have - ref).abs().max())
        # rejected speculative rows: snapshot, run two rows, restore, and the next real row is unchanged
        eng.snapshot(0)
        eng.step([1, 2], [0, 0], [10, 11])
        eng.restore(0)
        again = eng.step([seqs[0][10]], [0], [10]).cpu()
        assert (again - want[0][10:11]).abs().max() < 0.03 * (1 + want[0].abs().max())


@pytest.mark.gpu
def test_inkling_device_rows_match_the_oracle():
    from sparkflash_b200.models import inkling as I
    c = I.InklingConfig()
    w = I.init_weights(c, 5)
    toks = torch.randint(0, c.vocab, (14,), generator=torch.Generator().manual_seed(13)).tolist()
    want = I.reference_logits(c, w, toks)
    eng = I.DeviceEngine(c, w, lanes=1)
    got = torch.cat([eng.step([t], [0], [i]).cpu() for i, t in enumerate(toks)])
    assert (got - want).abs().max() < 0.05 * (1 + want.abs().max()), (got - want).abs().max()

"""Engram: layout, hashing, packing, lookup and gate (reference tests: crates/sparkflash-engram/tests/
engram_hash.rs, engram_store_golden.rs; golden numbers from docs/architecture/04-engram.md sections 3-4)."""
import numpy as np
import pytest
import torch

from sparkflash_b200.engram import layout as EL, store as ES


def test_released_layout_reproduces_the_checkpoint_row_counts():
    lay = EL.EngramLayout.build([1, 14], 4, 8, 16_000_000, 99092, expect_rows=[384006168, 384016682])
    assert lay.primes[0, 0].tolist() == [16000057, 16000079, 16000081, 16000097, 16000121, 16000129, 16000133, 16000183]
    assert lay.primes[1, 2].tolist() == [16000781, 16000799, 16000813, 16000819, 16000841, 16000877, 16000879, 16000889]
    assert lay.offsets[0, :, 0].tolist() == [0, 128000880, 256002934] and lay.offsets[1, :, 0].tolist() == [0, 128004290, 256009984]
    assert len(set(lay.primes.reshape(-1).tolist())) == 48
    with pytest.raises(ValueError):
        EL.EngramLayout.build([1, 14], 4, 8, 16_000_000, 99092, expect_rows=[1, 2])
    # the hard-coded multipliers are numpy's PCG64 stream
    bound = ((2 ** 63 - 1) // 99092) // 2
    assert bound == 46539438283891
    for lid in (1, 14):
        vals = np.random.default_rng(10007 * lid).integers(0, bound, size=(4,), dtype=np.int64)
        assert [int(v) * 2 + 1 for v in vals] == EL.RELEASED_MULTIPLIERS[(lid, 99092)]


def test_hash_matches_the_reference_program_and_blocks_at_dead_positions():
    lay = EL.EngramLayout.build([1, 14], 4, 8, 16_000_000, 99092)
    rng = np.random.default_rng(0)
    cache = rng.integers(0, 99092, size=64).astype(np.int64)
    cache[10] = EL.DEAD
    pos = list(range(0, 64))
    for li in (0, 1):
        a = lay.hash_ids(li, cache, pos, pad_id=7)
        b = EL.hash_ids_reference(lay, li, cache, pos, 7)
        assert np.array_equal(a, b)
        assert (a >= 0).all() and (a < lay.rows[li]).all()
        # bucket ranges: column c lies in [offset, offset + prime)
        off, pr = lay.offsets[li].reshape(-1), lay.primes[li].reshape(-1)
        assert ((a >= off) & (a < off + pr)).all()
    # positions 11..13 look back over the dead position: their longer n-grams equal those of a sequence that starts at 11
    tail = cache[11:].copy()
    a = lay.hash_ids(0, cache, [11, 12, 13], 7)
    b = lay.hash_ids(0, tail, [0, 1, 2], 7)
    assert np.array_equal(a, b)


def test_compressed_token_map_normalises():
    toks = [" The", "the", "THE", "é", "e", " ", "", "\t\n", "ﬁ", "fi", "�"]
    lookup, n = EL.build_compressed_token_map(toks, raw=[f"<{i}>" for i in range(len(toks))])
    assert lookup[0] == lookup[1] == lookup[2] and lookup[3] == lookup[4] and lookup[8] == lookup[9]
    assert lookup[5] == lookup[7] != lookup[6] and n == len(set(lookup.tolist()))


def _table(rows, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randint(0, 256, (rows, 256), generator=g, dtype=torch.uint8)
    w[(w & 0x7F) == 0x7F] = 0x3C                 # no NaN codes
    s = torch.randint(120, 130, (rows, 8), generator=g, dtype=torch.uint8)
    return w, s


def test_pack_shards_and_partial_lookups_sum_to_the_full_lookup(tmp_path):
    rows = 1003
    w, s = _table(rows, 1)
    ids = torch.randint(0, rows, (5, 24), generator=torch.Generator().manual_seed(2))
    full = ES.gather_reference(ES.pack_table(w, s, 0, 1), 0, ids)
    parts = 0
    for r in range(4):
        packed = ES.pack_table(w, s, r, 4)
        first, per = ES.shard_range(rows, r, 4)
        assert packed.shape == (per, ES.STRIDE)
        parts = parts + ES.gather_reference(packed, first, ids)
    assert torch.equal(parts, full)
    tail = ES.pack_table(w, s, 3, 4)                # rows past the table: weight 0, scale 1.0
    assert tail[-1, :256].sum() == 0 and (tail[-1, 256:264] == 127).all()
    # the CLI path: checkpoint shards in, per-rank files and manifest out
    from sparkflash_b200.weights.files import write_safetensors
    src = tmp_path / "ck"; src.mkdir()
    write_safetensors(str(src / "m.safetensors"), {"engram.1.embed.weight": w, "engram.1.embed.scale": s})
    rep = ES.pack(str(src), str(tmp_path / "out"), world=2)
    assert len(rep["files"]) == 2 and rep["rows"] == {"1": rows}
    sh = ES.EngramShard.from_file(str(tmp_path / "out" / rep["files"][1]), rows, 1, 2, device="cpu")
    assert torch.equal(sh.gather(ids).float(), ES.gather_reference(ES.pack_table(w, s, 1, 2), sh.first, ids).to(torch.bfloat16).float())


@pytest.mark.gpu
def test_device_gather_and_gate_match_the_reference():
    rows = 5000
    w, s = _table(rows, 3)
    ids = torch.randint(0, rows, (7, 24), generator=torch.Generator().manual_seed(4))
    for resident in (True, False):
        for rank, world in ((0, 1), (1, 2)):
            packed = ES.pack_table(w, s, rank, world)
            sh = ES.EngramShard(packed, rows, rank, world, "cuda", resident=resident)
            got = sh.gather(ids.cuda()).float().cpu()
            want = ES.gather_reference(packed, sh.first, ids).to(torch.bfloat16).float()
            assert torch.equal(got, want)
    n, hc, d = 6, 4, 512
    g = torch.Generator().manual_seed(5)
    h = torch.randn(n, hc, d, generator=g)
    kv = (torch.randn(n, (hc + 1) * d, generator=g) * 0.5).to(torch.bfloat16)
    wq = torch.randn(hc, d, generator=g)
    mask = torch.tensor([1, 1, 0, 1, 1, 1], dtype=torch.uint8)
    want = ES.gate_reference(h, kv, wq, mask, 1e-20)
    hd = h.cuda()
    ES.gate(hd, kv.cuda(), wq.cuda(), mask.cuda(), 1e-20)
    torch.cuda.synchronize()
    assert torch.equal(hd[2].cpu(), h[2])                       # a masked token keeps h exactly
    assert (hd.cpu() - want).abs().max() < 2e-3


@pytest.mark.gpu
def test_engine_with_engram_matches_the_oracle():
    """The serving engine with the n-gram memory wired in before the Engram layers' blocks, against the CPU oracle:
    the first positions to rounding, later ones statistically (cached low-precision values drift apart)."""
    from sparkflash_b200.config import tiny_config
    from sparkflash_b200.engram.runtime import EngramRuntime
    from sparkflash_b200.models.deepseek_v41 import engine as E, oracle as O, prepare as P, weights as W
    cfg = tiny_config(engram=True)
    ck = W.synthetic_checkpoint(cfg, 0)
    orc = O.Oracle(cfg, W.dequantize_checkpoint(ck, cfg))
    base = O.Oracle(cfg, {k: v for k, v in W.dequantize_checkpoint(ck, cfg).items() if not k.startswith("engram.")})
    eng = E.Engine(P.prepare_from_checkpoint(ck, cfg, 0, 1), max_lanes=2, max_context=256, max_rows=16, arm="tc", keep_logits=True,
                   engram=EngramRuntime.from_checkpoint(ck, cfg))
    prompt = torch.randint(0, cfg.vocab_size, (14,), generator=torch.Generator().manual_seed(8)).tolist()
    st, st0 = orc.new_state(), base.new_state()
    errs, agree, moved = [], 0, 0.0
    for pos, tok in enumerate(prompt):
        want = orc.step(st, tok)
        plain = base.step(st0, tok)
        out = eng.step([tok], [1], [pos])
        got = eng.logits[0].float().cpu()
        scale = want.abs().max().item()
        if pos == 0:
            assert (got - want).abs().max().item() < 0.03 * scale
        errs.append((got - want).abs().mean().item() / scale)
        moved = max(moved, (want - plain).abs().max().item() / scale)
        agree += int(out[0]) == int(want.argmax())
    eng.check_status()
    assert moved > 0.05                       # the memory really changes the model's output ...
    assert sum(errs) / len(errs) < 0.06       # ... and the engine follows the oracle with it
    assert agree >= 0.6 * len(prompt)
    # a multi-row chunk on another lane gives the rows the single-row steps gave (n-grams come from the lane's own history)
    eng.step(prompt[:7], [0] * 7, list(range(7)))
    eng.step(prompt[7:], [0] * 7, list(range(7, 14)))
    assert torch.equal(eng.logits[6].float().cpu(), got) or (eng.logits[6].float().cpu() - got).abs().max() < 1e-3 * scale


def test_paged_table_reads_rows_from_the_file_with_cache_and_read_ahead(tmp_path):
    """The table stays on disk: rows come back byte-identical to the packed file, repeated pages hit the cache, pages
    asked for ahead of time are resident when the demand read comes, and a small cache evicts."""
    import numpy as np
    from sparkflash_b200.engram import paged as PG, store as ST
    rows, width = 1000, 256
    g = torch.Generator().manual_seed(2)
    w = torch.randint(0, 120, (rows, width), dtype=torch.uint8, generator=g)          # finite E4M3 codes
    s = torch.randint(110, 130, (rows, width // 32), dtype=torch.uint8, generator=g)
    packed = ST.pack_table(w, s, 0, 1)
    path = tmp_path / "table.bin"
    packed.numpy().tofile(path)
    t = PG.PagedTable(str(path), rows, page_rows=16, cache_pages=8)
    ids = torch.tensor([[0, 5, 999], [17, 16, 400], [-1, 1000, 33]])
    got = t.gather(ids).clone()
    want = torch.zeros((9, ST.STRIDE), dtype=torch.uint8)
    for i, r in enumerate(ids.reshape(-1).tolist()):
        if 0 <= r < rows:
            want[i] = packed[r]
    assert torch.equal(got, want)
    st = t.stats()
    assert st["misses"] == 5 and st["hits"] == 2          # pages 0, 62, 1, 25, 2 loaded once; rows 5 and 16 hit pages 0 and 1
    # read-ahead: pages of rows 600..700 are pulled in by the background thread, the demand read then only hits
    ahead = torch.arange(600, 700)
    assert t.prefetch(ahead) == 7                          # rows 600..699 span pages 37..43
    t.drain()
    before = t.stats()
    t.gather(ahead)
    after = t.stats()
    assert after["misses"] == before["misses"] and after["hits"] - before["hits"] == 100 and after["prefetched_pages"] == 7
    assert after["evictions"] > 0 and after["resident_pages"] <= 8
    # same numbers as the resident shard
    shard = PG.PagedShard(t, device="cpu")
    full = ST.EngramShard(packed, rows, 0, 1, device="cpu")
    q = torch.randint(0, rows, (4, 6), generator=g)
    assert torch.equal(shard.gather(q), full.gather(q))
    t.close()
    with pytest.raises(OSError):
        PG.PagedTable(str(path), rows * 2)                 # the file is too short for that many rows

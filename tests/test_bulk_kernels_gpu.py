"""Many-row tensor-core kernels against plain fp32 references: the bf16 GEMM (kind::f16), the two-term block layout of
the grouped output projection, and the tcgen05 rows attention.  Reference tests: crates/sparkflash-kernels/tests
(decode_mma_device.rs), kernels/opt_mma_sm121.cu bulk paths."""
import pytest
import torch

from sparkflash_b200 import codecs as C

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N_,K,n,splits", [(128, 64, 1, 1), (256, 512, 5, 1), (384, 1024, 40, 4), (256, 320, 300, 1),
                                            (128, 2048, 130, 2), (200, 256, 16, 1)])
def test_umma_bf16_matches_fp32_reference(N_, K, n, splits):
    from sparkflash_b200.ops import native as N
    g = torch.Generator().manual_seed(N_ + K + n)
    w = (torch.randn(N_, K, generator=g) * 0.1).to(torch.bfloat16)
    x = torch.randn(n, K, generator=g).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    dev = "cuda"
    NP = 128 if n > 128 else N.umma_np(n)
    rows_b = (n + NP - 1) // NP * NP
    wd = w.to(dev).contiguous()
    xd = torch.zeros(rows_b, K, dtype=torch.bfloat16, device=dev)
    xd[:n] = x.to(dev)
    ta = N.bf16_map(wd, N_, K, 128)
    tb = N.bf16_map(xd, rows_b, K, NP)
    tiles = (N_ + 127) // 128 * ((n + NP - 1) // NP)
    scratch = torch.zeros(max(1, tiles * splits * 128 * NP), dtype=torch.float32, device=dev)
    tickets = torch.zeros(max(1, tiles), dtype=torch.int32, device=dev)
    out = torch.full((n, N_), float("nan"), dtype=torch.float32, device=dev)
    out_b = torch.zeros((n, N_), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    for _ in range(2):
        N.umma_bf16(ta, tb, n, N_, K, splits=splits, scratch=scratch, tickets=tickets, out_f=out, status=status, NP=NP)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0, status.tolist()
        err = (out.cpu() - ref).abs().max().item()
        assert err <= 1e-4 * ref.abs().max().item() + 1e-5, (err, ref.abs().max().item())   # exact products, fp32 sums
    if N_ % 128 == 0:
        N.umma_bf16(ta, tb, n, N_, K, splits=splits, scratch=scratch, tickets=tickets, out_b=out_b, status=status, NP=NP)
        torch.cuda.synchronize()
        assert (out_b.cpu().float() - ref).abs().max() <= 2 ** -7 * ref.abs().max() + 1e-5


def test_two_term_block_layout_matches_per_block_launches():
    """150 rows through the grouped projection in one launch (blocks of 64 hi + 64 lo rows) give the bits of one launch per
    block of 64 rows, and both stay within FP8 two-term precision of the fp32 product."""
    from sparkflash_b200.ops import native as N
    dev = "cuda"
    groups, N_, K, n = 2, 128, 256, 150
    g = torch.Generator().manual_seed(5)
    w = torch.randn(groups * N_, K, generator=g) * 0.05
    q, s = C.weight_quant_fp8_block32(w)
    wd = C.weight_dequant_fp8_block32(q, s)
    sfa = C.scales_to_prepared(s, groups * N_, 32).to(dev)
    x = torch.randn(n, groups * K, generator=g).to(torch.bfloat16)
    ref = torch.cat([x.float()[:, gi * K:(gi + 1) * K] @ wd[gi * N_:(gi + 1) * N_].t() for gi in range(groups)], 1)
    nblk = (n + 63) // 64
    KB = groups * K // 32
    xq = torch.zeros(nblk * 128, groups * K, dtype=torch.uint8, device=dev)
    atom = torch.full((C.sf_bytes(nblk * 128, KB),), 127, dtype=torch.uint8, device=dev)
    block_bytes = C.sf_bytes(128, KB)
    xdev = x.to(dev)
    for b in range(nblk):
        m = min(64, n - 64 * b)
        N.quant_rows(xdev[64 * b:], xq[128 * b:], None, atom[b * block_bytes:], m, groups * K, split=True, split_off=64)
    qd = q.to(dev).contiguous()
    ta = N.TensorMap(qd, groups * N_, K, K, 128)
    tb = N.TensorMap(xq, nblk * 128, groups * K, groups * K, 128)
    tiles = (N_ // 128) * groups * nblk
    scratch = torch.zeros(tiles * 128 * 128, dtype=torch.float32, device=dev)
    tickets = torch.zeros(tiles, dtype=torch.int32, device=dev)
    out = torch.full((n, groups * N_), float("nan"), dtype=torch.float32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    oq = torch.zeros(nblk * 64, groups * N_, dtype=torch.uint8, device=dev)
    oq_atom = torch.full((C.sf_bytes(nblk * 64, groups * N_ // 32),), 127, dtype=torch.uint8, device=dev)
    N.umma_pair_bulk(ta, tb, sfa, atom, n, N_, K, groups=groups, scratch=scratch, tickets=tickets, out_f=out, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    assert (out.cpu() - ref).abs().max() <= 4e-3 * ref.abs().max()
    # per-block launches of the few-row entry point on the same buffers
    for b in range(nblk):
        m = min(64, n - 64 * b)
        one = torch.zeros(64, groups * N_, dtype=torch.float32, device=dev)      # the few-row entry point writes all 64 rows
        tb1 = N.TensorMap(xq[128 * b:], 128, groups * K, groups * K, 128)
        N.umma_dense_pair(ta, tb1, sfa, atom[b * block_bytes:], 64, N_, K, groups=groups, scratch=scratch, tickets=tickets,
                          out_f=one, status=status, NP=128)
        torch.cuda.synchronize()
        assert torch.equal(one[:m], out[64 * b:64 * b + m]), b
    # re-quantised output for the next projection: codes and atoms decode to the bf16-rounded output
    out_b = torch.zeros(n, groups * N_, dtype=torch.bfloat16, device=dev)
    N.umma_pair_bulk(ta, tb, sfa, atom, n, N_, K, groups=groups, scratch=scratch, tickets=tickets, out_b=out_b, out_q=oq,
                     out_q_atom=oq_atom, status=status)
    torch.cuda.synchronize()
    rq, rs = C.act_quant_fp8(out_b.cpu().float())
    assert torch.equal(oq[:n].cpu(), rq)
    assert torch.equal(C.prepared_to_scales(oq_atom.cpu(), n, groups * N_ // 32), rs)


def _attention_case(heads, rows, with_compressed, seed):
    from sparkflash_b200.models.deepseek_v41 import oracle as O
    from sparkflash_b200.config import full_config
    cfg = full_config()
    hd, rd, window, ring, K = 512, 64, 128, 512, 512
    g = torch.Generator().manual_seed(seed)
    lanes = 2
    pos = torch.tensor(rows, dtype=torch.int32)
    n = len(rows)
    lane = torch.tensor([i % lanes for i in range(n)], dtype=torch.int32)
    invf = O.rope_inv_freq(cfg, True)
    win = torch.randn(lanes, ring, hd, generator=g) * 0.7
    wq, ws = C.act_quant_fp8(win)
    entries = 900
    ckv = torch.randn(lanes, entries, hd, generator=g) * 0.7
    cq, cs = C.kv_quant_fp4(ckv)
    sel = torch.full((n, K), -1, dtype=torch.int32)
    cnt = torch.zeros(n, dtype=torch.int32)
    if with_compressed:
        for r in range(n):
            clen = min(entries, int(pos[r]) + 1)
            k = min(K, clen)
            ids = torch.randperm(clen, generator=g)[:k].sort().values
            sel[r, :k] = ids.int(); cnt[r] = k
    q = (torch.randn(n, heads * hd, generator=g) * 0.5).to(torch.bfloat16)
    sink = torch.randn(heads, generator=g)
    return dict(cfg=cfg, hd=hd, rd=rd, window=window, ring=ring, K=K, pos=pos, lane=lane, invf=invf, wq=wq, ws=ws, cq=cq, cs=cs,
                sel=sel, cnt=cnt, q=q, sink=sink, n=n, heads=heads)


@pytest.mark.parametrize("heads,with_compressed", [(8, True), (40, True), (16, False), (64, True)])
def test_attention_tc_matches_fp32_reference(heads, with_compressed):
    from sparkflash_b200.models.deepseek_v41 import oracle as O
    from sparkflash_b200.ops import native as N
    rows = [700, 5, 131, 0, 127, 128, 400, 899, 64] if heads <= 16 else [700, 5, 131, 899]
    c = _attention_case(heads, rows, with_compressed, seed=11 + heads)
    dev = "cuda"
    n, hd, rd = c["n"], c["hd"], c["rd"]
    out = torch.zeros(n, heads * hd, dtype=torch.bfloat16, device=dev)
    nblk = (n + 63) // 64
    out_q = torch.zeros(nblk * 128, heads * hd, dtype=torch.uint8, device=dev)
    KB = heads * hd // 32
    out_atom = torch.full((C.sf_bytes(nblk * 128, KB),), 127, dtype=torch.uint8, device=dev)
    rope = torch.zeros(n, 1, rd // 2, 2, dtype=torch.float32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    N.rope_table([c["invf"].to(dev)], [1], c["pos"].to(dev), rope, n)
    ckq = C.pack_nibbles(c["cq"]).to(dev) if with_compressed else None
    cks = c["cs"].to(dev) if with_compressed else None
    N.attn_tc(c["q"].to(dev), heads * hd, rope[:, 0], c["lane"].to(dev), c["pos"].to(dev), c["wq"].to(dev), c["ws"].to(dev),
              ckq, cks, c["sel"].to(dev) if with_compressed else None, c["cnt"].to(dev) if with_compressed else None, c["K"],
              c["sink"].to(dev), out, n, heads, hd, rd, c["window"], c["ring"], hd ** -0.5, out_q=out_q, out_atom=out_atom,
              pair_block=64, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    wd = C.act_dequant_fp8(c["wq"], c["ws"])
    cd = C.kv_dequant_fp4(c["cq"], c["cs"])
    invf = c["invf"]
    for r in range(n):
        p, L = int(c["pos"][r]), int(c["lane"][r])
        keys = [wd[L, t % c["ring"]] for t in range(max(0, p - c["window"] + 1), p + 1)]
        keys += [cd[L, j] for j in c["sel"][r, :int(c["cnt"][r])].tolist()]
        Kmat = torch.stack(keys)
        qq = O.apply_rope(c["q"][r].float().view(heads, hd), p, invf)
        s = (qq @ Kmat.t()) * hd ** -0.5
        m = s.max(-1, keepdim=True).values
        e = torch.exp(s - m)
        o = O.bf((e @ Kmat) / (e.sum(-1, keepdim=True) + torch.exp(c["sink"].view(heads, 1) - m)))
        o = O.apply_rope(o, p, invf, inverse=True)
        got = out[r].cpu().float().view(heads, hd)
        assert (got - o).abs().max() <= 0.02 * o.abs().max() + 1e-4, (r, (got - o).abs().max(), o.abs().max())
    # the two-term FP8 copy decodes back to the bf16 output (hi + lo / 16 under the hi scale)
    oq = out_q.cpu()
    for r in range(n):
        hi_row, lo_row = (r // 64) * 128 + r % 64, (r // 64) * 128 + r % 64 + 64
        _, sc = C.act_quant_fp8(out[r].cpu().float().view(1, -1))
        scale = C.ue8m0_decode(sc).repeat_interleave(32, -1).view(-1)
        val = (C.e4m3_decode(oq[hi_row]) + C.e4m3_decode(oq[lo_row]) / 16.0) * scale
        ref = out[r].cpu().float()
        assert (val - ref).abs().max() <= 2 ** -6 * ref.abs().max() + 1e-6, r


def test_attention_tc_agrees_with_rows_kernel():
    """Same inputs through the CUDA-core rows kernel (the exact arm) and the tcgen05 kernel."""
    from sparkflash_b200.ops import native as N
    heads = 32
    c = _attention_case(heads, [300, 899, 17], True, seed=3)
    dev = "cuda"
    n, hd, rd = c["n"], c["hd"], c["rd"]
    rope = torch.zeros(n, 1, rd // 2, 2, dtype=torch.float32, device=dev)
    N.rope_table([c["invf"].to(dev)], [1], c["pos"].to(dev), rope, n)
    args = (c["q"].to(dev), heads * hd, rope[:, 0], c["lane"].to(dev), c["pos"].to(dev), c["wq"].to(dev), c["ws"].to(dev),
            C.pack_nibbles(c["cq"]).to(dev), c["cs"].to(dev), c["sel"].to(dev), c["cnt"].to(dev), c["K"], c["sink"].to(dev))
    a = torch.zeros(n, heads * hd, dtype=torch.bfloat16, device=dev)
    b = torch.zeros_like(a)
    N.attn_rows(*args, a, n, heads, hd, rd, c["window"], c["ring"], hd ** -0.5)
    N.attn_tc(*args, b, n, heads, hd, rd, c["window"], c["ring"], hd ** -0.5)
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().max() <= 0.02 * a.float().abs().max()


def _index_case(n, entries, lanes, seed):
    g = torch.Generator().manual_seed(seed)
    inh, idh, rd = 32, 128, 64
    keys = torch.randn(lanes, entries, idh, generator=g)
    kq, ks = C.act_quant_fp4(keys)                       # MXFP4: codes + one UE8M0 scale per 32
    qraw = (torch.randn(n, inh * idh, generator=g) * 0.8).to(torch.bfloat16)
    wraw = torch.randn(n, inh, generator=g)
    return dict(inh=inh, idh=idh, rd=rd, kq=kq, ks=ks, qraw=qraw, wraw=wraw)


@pytest.mark.parametrize("n,rpg,same_lane", [(3, 1, False), (9, 4, True), (1, 1, True)])
def test_index_scores_on_tensor_cores_match_cuda_core_kernel(n, rpg, same_lane):
    """Same quantised queries and keys through the CUDA-core scores kernel and the tcgen05 one; the candidate-block
    filter and the per-row compressed length mask the same entries."""
    from sparkflash_b200.models.deepseek_v41 import oracle as O
    from sparkflash_b200.config import full_config
    from sparkflash_b200.ops import native as N
    dev = "cuda"
    lanes, entries, ratio = 2, 1000, 2
    c = _index_case(n, entries, lanes, seed=21 + n)
    inh, idh, rd = c["inh"], c["idh"], c["rd"]
    pos = torch.tensor([1999, 300, 777, 5, 1200, 64, 1, 1500, 900][:n], dtype=torch.int32)
    lane = torch.zeros(n, dtype=torch.int32) if same_lane else torch.tensor([i % lanes for i in range(n)], dtype=torch.int32)
    invf = O.rope_inv_freq(full_config(), True)
    rope = torch.zeros(n, 1, rd // 2, 2, dtype=torch.float32, device=dev)
    N.rope_table([invf.to(dev)], [1], pos.to(dev), rope, n)
    ik_q = C.pack_nibbles(c["kq"]).to(dev).contiguous()      # [lanes, entries, 64]
    ik_s = c["ks"].to(dev).contiguous()                       # [lanes, entries, 4]
    qraw, wraw = c["qraw"].to(dev), c["wraw"].to(dev)
    wscale = idh ** -0.5 * inh ** -0.5
    bs = 8
    cand = (torch.rand(n, (entries + bs - 1) // bs, generator=torch.Generator().manual_seed(1)) > 0.3).to(torch.uint8).to(dev)
    # CUDA-core arm
    qi = torch.zeros(n, idh, inh, dtype=torch.float32, device=dev)
    wt = torch.zeros(n, inh, dtype=torch.float32, device=dev)
    ref = torch.full((n, entries), float("nan"), dtype=torch.float32, device=dev)
    N.index_q(qraw, inh * idh, 0, wraw, inh, 0, rope[:, 0], pos.to(dev), qi, wt, n, inh, idh, rd, wscale)
    N.index_scores(qi, wt, ik_q, ik_s, lane.to(dev), pos.to(dev), cand, bs, ref, n, inh, idh, ratio, entries)
    # tensor-core arm
    q4 = torch.zeros(n * inh, idh // 2, dtype=torch.uint8, device=dev)
    q_atoms = torch.full((n * 512,), 127, dtype=torch.uint8, device=dev)
    wt2 = torch.zeros(n, inh, dtype=torch.float32, device=dev)
    out = torch.full((n, entries), float("nan"), dtype=torch.float32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    N.index_q4(qraw, inh * idh, 0, wraw, inh, 0, rope[:, 0], q4, q_atoms, wt2, n, inh, idh, rd, rpg, wscale)
    tk = N.TensorMap(ik_q.view(lanes * entries, idh // 2), lanes * entries, idh, idh // 2, 128, fp4=True)
    tq = N.TensorMap(q4, n * inh, idh, idh // 2, 32 * rpg, fp4=True)
    N.index_scores_tc(tk, tq, ik_s, entries, q_atoms, wt2, lane.to(dev), pos.to(dev), cand, bs, out, n, ratio, entries, rpg, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    assert torch.equal(wt, wt2)
    for r in range(n):
        clen = (int(pos[r]) + 1) // ratio
        a, b = ref[r, :clen].cpu(), out[r, :clen].cpu()
        assert torch.equal(torch.isinf(a), torch.isinf(b)), r
        fin = ~torch.isinf(a)
        if fin.any():
            # the two query kernels may round a rotated element to neighbouring bf16 values (fused vs separate multiply-add),
            # which moves one FP4 code: nearly every score agrees to fp32 summation order, none is far off
            err, scale = (a[fin] - b[fin]).abs(), a[fin].abs().max() + 1e-6
            assert (err <= 1e-4 * scale).float().mean() >= 0.98 and err.max() <= 5e-2 * scale, (r, err.max(), scale)
        assert torch.isinf(out[r, clen:]).all()


def test_select_long_rows_matches_single_block_select():
    """The chunked select (several blocks per row, then a merge) returns exactly the ids of the one-block select, ties
    included (a quantised score column makes many ties; the lowest indices must win)."""
    from sparkflash_b200.ops import native as N
    dev = "cuda"
    n, L, K, chunk = 3, 70000, 512, 16384
    g = torch.Generator().manual_seed(4)
    sc = torch.randn(n, L, generator=g)
    sc[1] = (sc[1] * 4).round() / 4                 # heavy ties
    sc[2, 1000:] = float("-inf")                    # fewer finite entries than a chunk, more than K
    sc[0, ::7] = float("-inf")
    pos = torch.tensor([L - 1, L - 1, 50000], dtype=torch.int32)
    scd = sc.to(dev)
    ids1 = torch.zeros(n, K, dtype=torch.int32, device=dev); cnt1 = torch.zeros(n, dtype=torch.int32, device=dev)
    ids2 = torch.zeros(n, K, dtype=torch.int32, device=dev); cnt2 = torch.zeros(n, dtype=torch.int32, device=dev)
    nch = (L + chunk - 1) // chunk
    tmp_ids = torch.zeros(n, nch, K, dtype=torch.int32, device=dev)
    tmp_cnt = torch.zeros(n, nch, dtype=torch.int32, device=dev)
    tmp_list = torch.zeros(n, nch * K, dtype=torch.int32, device=dev)
    N.select_topk(scd, pos.to(dev), 1, 1, L, K, ids1, cnt1, n)
    N.select_topk_long(scd, pos.to(dev), 1, 1, L, K, ids2, cnt2, n, chunk, tmp_ids, tmp_cnt, tmp_list)
    torch.cuda.synchronize()
    assert torch.equal(cnt1, cnt2) and torch.equal(ids1, ids2)
    # and both follow the rule: value descending, index ascending among equals
    for r in range(n):
        ln = int(pos[r]) + 1
        order = sorted(range(ln), key=lambda i: (-sc[r, i].item(), i))
        want = sorted(i for i in order[:K] if sc[r, i] > float("-inf"))
        assert ids1[r, :int(cnt1[r])].tolist() == want


@pytest.mark.parametrize("W,with_post", [(1, True), (2, True), (1, False)])
def test_many_row_seam_through_bulk_copies_gives_the_bits_of_the_register_kernel(W, with_post):
    """The many-row fold moves a row through shared memory with bulk copies (residual copies and partial outputs in, new
    residual, folded output, normalised row, codes and scale bytes out): every output matches the kernel that loads and
    stores from registers bit for bit, scale atoms included."""
    from sparkflash_b200 import codecs as CC
    from sparkflash_b200.ops import native as N
    dev = "cuda"
    d, hc, n = 5120, 4, 300
    g = torch.Generator().manual_seed(31 + W)
    h = (torch.randn(n, hc, d, generator=g) * 0.5).to(torch.bfloat16)
    ys = [(torch.randn(n, d, generator=g) * 0.3).to(torch.bfloat16).to(dev) for _ in range(W)]
    norm_w = (1 + 0.05 * torch.randn(d, generator=g)).to(dev)
    prev = torch.rand(n, N.coef_stride(hc), generator=g).to(dev)
    outs = []
    try:
        for arm in (1, 0):
            N.seam_tune(arm)
            hh = h.clone().to(dev)
            xn = torch.zeros(n, d, dtype=torch.bfloat16, device=dev)
            xq = torch.zeros(n, d, dtype=torch.uint8, device=dev)
            xs = torch.zeros(n, d // 32, dtype=torch.uint8, device=dev)
            atom = torch.zeros(CC.sf_bytes(n, d // 32), dtype=torch.uint8, device=dev)
            ysum = torch.zeros(n, d, dtype=torch.bfloat16, device=dev)
            hss = torch.zeros(n, dtype=torch.float32, device=dev)
            N.seam_fold(hh, ys if with_post else None, prev, prev, prev.stride(0), norm_w, xn, xq, xs, n, hc, d, 1e-20,
                        ysum=ysum if with_post else None, hss=hss, xs_atom=atom)
            torch.cuda.synchronize()
            outs.append((hh, xn, xq, xs, atom, ysum, hss))
    finally:
        N.seam_tune(0)
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert outs[0][1].float().abs().sum() > 0 and outs[0][2].any()


def test_many_row_seam_matches_the_cluster_kernel_and_bf16_coefficients():
    """Steps of 129+ rows fold with one block per row and take the predictor dots from the bf16 tensor-core GEMM: residual
    copies, normalised rows and FP8 codes agree with the few-row kernels, coefficients to the two-term precision."""
    from sparkflash_b200.ops import native as N
    dev = "cuda"
    d, hc, mix, W, n = 5120, 4, 24, 2, 150
    g = torch.Generator().manual_seed(17)
    h = (torch.randn(n, hc, d, generator=g) * 0.5).to(torch.bfloat16)
    ys = [(torch.randn(n, d, generator=g) * 0.3).to(torch.bfloat16).to(dev) for _ in range(W)]
    fn = (torch.randn(mix, hc * d, generator=g) * 0.05).to(dev)
    base = (torch.randn(mix, generator=g) * 0.1).to(dev)
    scale = torch.tensor([1.0, 0.9, 1.1]).to(dev)
    norm_w = (1 + 0.05 * torch.randn(d, generator=g)).to(dev)
    cs = N.coef_stride(hc)
    prev = torch.rand(n, cs, generator=g).to(dev)

    def run(rows: slice, hss=None):
        m = rows.stop - rows.start
        hh = h[rows].clone().to(dev)
        xn = torch.zeros(m, d, dtype=torch.bfloat16, device=dev)
        xq = torch.zeros(m, d, dtype=torch.uint8, device=dev)
        xs = torch.zeros(m, d // 32, dtype=torch.uint8, device=dev)
        pv = prev[rows].contiguous()
        N.seam_fold(hh, [y[rows].contiguous() for y in ys], pv, pv, pv.stride(0), norm_w, xn, xq, xs, m, hc, d, 1e-20, hss=hss)
        return hh, xn, xq, xs
    hss = torch.zeros(n, dtype=torch.float32, device=dev)
    big = run(slice(0, n), hss)                       # one block per row
    parts = [run(slice(0, 75)), run(slice(75, n))]    # cluster kernel
    torch.cuda.synchronize()
    hh = torch.cat([p[0] for p in parts]); xn = torch.cat([p[1] for p in parts]); xq = torch.cat([p[2] for p in parts])
    assert torch.equal(big[0], hh)                                      # residual copies: same arithmetic per element
    assert (big[1].float() - xn.float()).abs().max() <= 2 ** -7 * xn.float().abs().max()
    assert (big[2] != xq).float().mean() < 0.01                          # codes may move where the row sum's order differs
    assert torch.allclose(hss.cpu(), hh.float().pow(2).sum((1, 2)).cpu(), rtol=1e-4)
    # coefficients: few-row kernel vs bf16 GEMM + finish
    nblk = N.seam_nblk(d)
    partials = torch.zeros(n, nblk, 1 + mix, device=dev)
    tickets = torch.zeros(n, dtype=torch.int32, device=dev)
    ref = torch.zeros(n, cs, device=dev)
    N.seam_coef(hh, fn, scale, base, partials, tickets, ref, n, hc, d, 20, 1e-20, 1e-6)
    hi = fn.to(torch.bfloat16); lo = (fn - hi.float()).to(torch.bfloat16)
    fn2 = torch.cat([hi, lo], 0).contiguous()
    R = 256
    hpad = torch.zeros(R, hc, d, dtype=torch.bfloat16, device=dev); hpad[:n] = hh
    ta, tb = N.bf16_map(fn2, 2 * mix, hc * d, 128), N.bf16_map(hpad, R, hc * d, 128)
    splits, tt = 16, R // 128
    scratch = torch.zeros(splits * tt * 128 * 128, dtype=torch.float32, device=dev)
    tk = torch.zeros(tt, dtype=torch.int32, device=dev)
    acc = torch.zeros(R, 64, dtype=torch.float32, device=dev)
    out = torch.zeros(n, cs, device=dev)
    N.umma_bf16(ta, tb, n, 2 * mix, hc * d, splits=splits, scratch=scratch, tickets=tk, out_f=acc, out_stride=64)
    N.seam_coef_finish(acc, hss, scale, base, out, n, hc, d, 20, 1e-20, 1e-6)
    torch.cuda.synchronize()
    assert torch.allclose(out.cpu(), ref.cpu(), rtol=2e-3, atol=2e-4), (out.cpu() - ref.cpu()).abs().max()


@pytest.mark.parametrize("N_,K,n", [(512, 256, 300), (2048, 512, 1024), (4096, 256, 2500)])
def test_persistent_bulk_gemm_gives_the_bits_of_the_tile_per_cta_kernel(N_, K, n):
    """The persistent many-row kernel (one CTA per SM walking over tiles, epilogue under the next main loop) against the
    one-tile-per-CTA kernel: same bf16 bits, and both within FP8 precision of the fp32 product.  The last shape gives
    every CTA several tiles (both accumulator sets and every barrier phase are used) and a partial last token tile."""
    from sparkflash_b200.ops import native as N
    dev = "cuda"
    g = torch.Generator().manual_seed(N_ + n)
    w = torch.randn(N_, K, generator=g) * 0.05
    x = torch.randn(n, K, generator=g)
    q, s = C.weight_quant_fp8_block32(w)
    wd = C.weight_dequant_fp8_block32(q, s)
    sfa = C.scales_to_prepared(s, N_, 32).to(dev)
    xq, xs = C.act_quant_fp8(x)
    ref = C.act_dequant_fp8(xq, xs) @ wd.t()
    rows = (n + 127) // 128 * 128
    xpad = torch.zeros(rows, K, dtype=torch.uint8, device=dev)
    xpad[:n] = xq.to(dev)
    sfb = C.scales_to_prepared(xs, n, 1).to(dev)
    qd = q.to(dev).contiguous()
    ta = N.TensorMap(qd, N_, K, K, 128)
    tb = N.TensorMap(xpad, rows, K, K, 128)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    outs = []
    try:
        for arm in (1, 2):            # 1: never persistent, 2: persistent whenever the shape allows
            N.umma_tune(5, arm)
            out = torch.zeros(n, N_, dtype=torch.bfloat16, device=dev)
            for _ in range(2):
                N.umma_bulk(ta, tb, sfa, sfb, n, N_, K, out_b=out, status=status)
            torch.cuda.synchronize()
            assert status.tolist()[0] == 0, status.tolist()
            outs.append(out.float().cpu())
    finally:
        N.umma_tune(5, 0)
    assert torch.equal(outs[0], outs[1])
    assert (outs[1] - ref).abs().max() <= 1e-2 * ref.abs().max()

"""GPU tests: every rows-step kernel against a plain PyTorch fp32 reference of the same op, and the
whole tiny model against the CPU oracle (reference test strategy: CPU twins vs device kernels,
batch_exactness.rs / verify_rows.rs style invariance checks)."""
import pytest
import torch

from sparkflash_b200 import codecs as C
from sparkflash_b200.config import tiny_config

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny():
    from sparkflash_b200.models.deepseek_v41 import oracle as O, prepare as P, weights as W
    cfg = tiny_config()
    ck = W.synthetic_checkpoint(cfg, 0)
    w = W.dequantize_checkpoint(ck, cfg)
    return cfg, ck, w, O.Oracle(cfg, w), P.prepare_from_checkpoint(ck, cfg)


def _prompt(cfg, n, seed=1):
    return torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ---- kernels -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("wfmt,N_,K,n", [(0, 96, 256, 1), (0, 40, 128, 5), (1, 64, 256, 3), (1, 130, 512, 9),
                                         (2, 48, 256, 2), (2, 1000, 64, 7)])
def test_gemv_matches_fp32_reference(wfmt, N_, K, n):
    from sparkflash_b200.ops import native as N
    g = torch.Generator().manual_seed(wfmt * 100 + N_)
    w = torch.randn(N_, K, generator=g) * 0.05
    x = torch.randn(n, K, generator=g)
    dev = "cuda"
    out = torch.zeros(n, N_, dtype=torch.float32, device=dev)
    if wfmt == 0:
        q, s = C.weight_quant_fp8_block32(w)
        wd = C.weight_dequant_fp8_block32(q, s)
        sf = s.repeat_interleave(32, 0)[:N_].contiguous()
        xq, xs = C.act_quant_fp8(x)
        ref = C.act_dequant_fp8(xq, xs) @ wd.t()
        N.gemv(0, q.to(dev), sf.to(dev), K, N_, K, n, xq=xq.to(dev), xs=xs.to(dev), out_f=out)
    elif wfmt == 1:
        q, s = C.weight_quant_fp4_row32(w)
        wd = C.weight_dequant_fp4_row32(q, s)
        sf = s.contiguous()
        xb = x.to(torch.bfloat16)
        ref = C.act_roundtrip_fp8(xb.float()) @ wd.t()
        N.gemv(1, q.to(dev), sf.to(dev), K // 2, N_, K, n, xb=xb.to(dev), x_quant=True, out_f=out)
    else:
        wb = w.to(torch.bfloat16)
        xb = x.to(torch.bfloat16)
        ref = xb.float() @ wb.float().t()
        N.gemv(2, wb.to(dev), None, 2 * K, N_, K, n, xb=xb.to(dev), out_f=out)
    torch.cuda.synchronize()
    err = (out.cpu() - ref).abs().max().item()
    assert err <= 2e-4 * ref.abs().max().item() + 1e-6, err


def test_gemv_grouped_and_batch_invariant():
    from sparkflash_b200.ops import native as N
    g = torch.Generator().manual_seed(5)
    groups, N_, K, n = 2, 64, 128, 6
    w = torch.randn(groups * N_, K, generator=g) * 0.05
    q, s = C.weight_quant_fp8_block32(w)
    wd = C.weight_dequant_fp8_block32(q, s)
    sf = s.repeat_interleave(32, 0)[:groups * N_].contiguous().cuda()
    xb = torch.randn(n, groups * K, generator=g).to(torch.bfloat16)
    out = torch.zeros(n, groups * N_, dtype=torch.float32, device="cuda")
    N.gemv(0, q.cuda(), sf, K, N_, K, n, groups=groups, xb=xb.cuda(), out_f=out)
    ref = torch.cat([xb.float()[:, gi * K:(gi + 1) * K] @ wd[gi * N_:(gi + 1) * N_].t() for gi in range(groups)], 1)
    assert (out.cpu() - ref).abs().max() <= 2e-4 * ref.abs().max()
    one = torch.zeros(1, groups * N_, dtype=torch.float32, device="cuda")
    for r in range(n):
        N.gemv(0, q.cuda(), sf, K, N_, K, 1, groups=groups, xb=xb[r:r + 1].cuda(), out_f=one)
        assert torch.equal(one[0], out[r]), "row bits depend on the batch"


def test_select_topk_rules():
    from sparkflash_b200.ops import native as N
    n, L, K = 5, 300, 16
    g = torch.Generator().manual_seed(3)
    sc = torch.randn(n, 512, generator=g)
    sc[1, :L] = 1.0                      # all ties: lowest indices win
    sc[2, 10:290] = float("-inf")        # fewer finite entries than K
    sc[3, 5] = sc[3, 200] = sc[3, 100] = 9.0
    pos = torch.full((n,), L - 1, dtype=torch.int32)
    pos[4] = 7                            # short row
    ids = torch.zeros(n, K, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(n, dtype=torch.int32, device="cuda")
    N.select_topk(sc.cuda(), pos.cuda(), 1, 1, 512, K, ids, cnt, n)
    torch.cuda.synchronize()
    for r in range(n):
        ln = int(pos[r]) + 1
        vals = sc[r, :ln].tolist()
        order = sorted(range(ln), key=lambda i: (-vals[i], i))
        want = sorted(i for i in order[:K] if vals[i] > float("-inf"))
        got = ids[r, :int(cnt[r])].tolist()
        assert got == want, (r, got, want)
        assert all(v == -1 for v in ids[r, int(cnt[r]):].tolist())


def test_router_matches_oracle(tiny):
    from sparkflash_b200.ops import native as N
    cfg, ck, w, orc, dw = tiny
    g = torch.Generator().manual_seed(7)
    n, E, k = 6, 24, 4
    dots = torch.randn(n, E, generator=g) * 2
    bias = torch.randn(E, generator=g) * 0.1
    ids = torch.zeros(n, k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n, k, dtype=torch.float32, device="cuda")
    N.router_topk(dots.cuda(), bias.cuda(), None, None, ids, wts, n, E, k, 1.5)
    s = torch.sqrt(torch.nn.functional.softplus(dots))
    for r in range(n):
        pick = sorted(torch.topk(s[r] + bias, k).indices.tolist())
        assert ids[r].tolist() == pick
        ww = s[r][pick]
        ww = ww / (ww.sum() + 1e-20) * 1.5
        assert torch.allclose(wts[r].cpu(), ww, rtol=1e-5, atol=1e-6)


def test_sampler_matches_oracle():
    from sparkflash_b200.models.deepseek_v41 import oracle as O
    from sparkflash_b200.ops import native as N
    g = torch.Generator().manual_seed(9)
    n, V = 3, 500
    logits = torch.randn(n, V, generator=g)
    pos = torch.tensor([4, 17, 900], dtype=torch.int32)
    temp = torch.tensor([0.0, 1.0, 0.7], dtype=torch.float32)
    seed = torch.tensor([1, 2, 3], dtype=torch.int64)
    bv = torch.zeros(n, device="cuda"); bi = torch.zeros(n, dtype=torch.int32, device="cuda")
    N.sample(logits.cuda(), pos.cuda(), temp.cuda(), seed.cuda(), None, bv, bi, n, V, 0)
    for r in range(n):
        assert int(bi[r]) == O.sample_token(logits[r], float(temp[r]), int(seed[r]), int(pos[r]) + 1)


# ---- whole model ---------------------------------------------------------------------------------------------
def test_engine_matches_oracle_token_by_token(tiny):
    """Positions whose whole history stays within one warp's accumulation order are bit-close; later
    ones differ by reassociation plus bf16 re-rounding of the residual stream, so the bar is the kind
    the reference uses for its served gate (mean error, top-1 agreement), not equality."""
    from sparkflash_b200.models.deepseek_v41 import engine as E
    cfg, ck, w, orc, dw = tiny
    eng = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16, use_graphs=False)
    prompt = _prompt(cfg, 40)
    st = orc.new_state()
    agree, mean_err, worst = 0, [], 0.0
    for pos, tok in enumerate(prompt):
        ol = orc.step(st, tok)
        eng.step([tok], [0], [pos])
        el = eng.logits[0].cpu()
        scale = ol.abs().max().item()
        err = (el - ol).abs()
        if pos < 4:
            assert err.max().item() < 1e-3 * scale, (pos, err.max().item())
        mean_err.append(err.mean().item() / scale)
        worst = max(worst, err.max().item() / scale)
        agree += int(el.argmax()) == int(ol.argmax())
    eng.check_status()
    assert sum(mean_err) / len(mean_err) < 0.03, sum(mean_err) / len(mean_err)
    assert worst < 0.6, worst
    assert agree >= 0.7 * len(prompt), agree


def test_seam_matches_oracle_math():
    from sparkflash_b200.config import ModelConfig
    from sparkflash_b200.models.deepseek_v41 import oracle as O
    from sparkflash_b200.ops import native as N
    for d, n, W in ((256, 3, 1), (5120, 2, 2)):
        cfg = ModelConfig(hidden_size=d)
        hc, mix = 4, 24
        g = torch.Generator().manual_seed(d)
        h = (torch.randn(n, hc, d, generator=g) * 0.5).to(torch.bfloat16)
        ys = [(torch.randn(n, d, generator=g) * 0.3).to(torch.bfloat16) for _ in range(W)]
        fn = torch.randn(mix, hc * d, generator=g) * 0.05
        base = torch.randn(mix, generator=g) * 0.1
        scale = torch.tensor([1.0, 0.9, 1.1])
        norm_w = 1 + 0.05 * torch.randn(d, generator=g)
        prev = torch.zeros(n, N.coef_stride(hc))
        ref_h, ref_xn, ref_coef = [], [], []
        for r in range(n):
            pre, post, comb = O.hc_coeffs(h[r].float() * 0.7, fn, scale, base, cfg)  # any valid coefficients
            prev[r] = torch.cat([pre, post, comb.flatten()])
            y = O.bf(sum(y_[r].float() for y_ in ys))
            hn = O.hc_post(y, h[r].float(), post, comb)
            p2, q2, c2 = O.hc_coeffs(hn, fn, scale, base, cfg)
            ref_h.append(hn); ref_coef.append(torch.cat([p2, q2, c2.flatten()]))
            ref_xn.append(O.rmsnorm(O.hc_pre(hn, pre), norm_w, cfg.norm_eps))
        dev = "cuda"
        hd_ = h.clone().to(dev)
        nblk = N.seam_nblk(d)
        partials = torch.zeros(n, nblk, 1 + mix, device=dev)
        coef = torch.zeros(n, N.coef_stride(hc), device=dev)
        xn = torch.zeros(n, d, dtype=torch.bfloat16, device=dev)
        xq = torch.zeros(n, d, dtype=torch.uint8, device=dev)
        xs = torch.zeros(n, d // 32, dtype=torch.uint8, device=dev)
        prev_d = prev.to(dev)
        tickets = torch.zeros(n, dtype=torch.int32, device=dev)
        N.seam_fold(hd_, [y_.to(dev) for y_ in ys], prev_d, prev_d, prev_d.stride(0), norm_w.to(dev), xn, xq, xs, n,
                    hc, d, cfg.norm_eps)
        N.seam_coef(hd_, fn.to(dev), scale.to(dev), base.to(dev), partials, tickets, coef, n, hc, d,
                    cfg.hc_sinkhorn_iters, cfg.norm_eps, cfg.hc_eps)
        torch.cuda.synchronize()
        rh = torch.stack(ref_h)
        assert (hd_.cpu().float() - rh).abs().max() <= 2 ** -7 * rh.abs().max(), "residual copies"
        assert torch.allclose(coef.cpu(), torch.stack(ref_coef), rtol=2e-4, atol=2e-5)
        ref = torch.stack(ref_xn)
        got = xn.cpu().float()
        assert (got - ref).abs().max() <= 2 ** -7 * ref.abs().max()  # one bf16 ulp at most
        rq, rs = C.act_quant_fp8(got)
        assert torch.equal(xq.cpu(), rq) and torch.equal(xs.cpu(), rs)


def test_attention_rows_matches_fp32_reference():
    from sparkflash_b200.models.deepseek_v41 import oracle as O
    from sparkflash_b200.config import full_config
    from sparkflash_b200.ops import native as N
    cfg = full_config()
    hd, rd, heads, window, ring, K = 512, 64, 4, 128, 256, 512
    g = torch.Generator().manual_seed(11)
    lanes, n = 2, 3
    pos = torch.tensor([700, 5, 131], dtype=torch.int32)
    lane = torch.tensor([0, 1, 1], dtype=torch.int32)
    invf = O.rope_inv_freq(cfg, True)
    win = torch.randn(lanes, ring, hd, generator=g) * 0.7
    wq, ws = C.act_quant_fp8(win)
    entries = 400
    ckv = torch.randn(lanes, entries, hd, generator=g) * 0.7
    cq, cs = C.kv_quant_fp4(ckv)
    sel = torch.full((n, K), -1, dtype=torch.int32)
    cnt = torch.zeros(n, dtype=torch.int32)
    for r in range(n):
        clen = min(entries, int(pos[r]) + 1)
        k = min(K, clen, 300)
        ids = torch.randperm(clen, generator=g)[:k].sort().values
        sel[r, :k] = ids.int(); cnt[r] = k
    q = (torch.randn(n, heads * hd, generator=g) * 0.5).to(torch.bfloat16)
    sink = torch.randn(heads, generator=g)
    dev = "cuda"
    out = torch.zeros(n, heads * hd, dtype=torch.bfloat16, device=dev)
    rope = torch.zeros(n, 1, rd // 2, 2, dtype=torch.float32, device=dev)
    N.rope_table([invf.to(dev)], [1], pos.to(dev), rope, n)
    N.attn_rows(q.to(dev), heads * hd, rope[:, 0], lane.to(dev), pos.to(dev), wq.to(dev), ws.to(dev),
                C.pack_nibbles(cq).to(dev), cs.to(dev), sel.to(dev), cnt.to(dev), K, sink.to(dev), out, n, heads,
                hd, rd, window, ring, hd ** -0.5)
    torch.cuda.synchronize()
    wd = C.act_dequant_fp8(wq, ws)
    cd = C.kv_dequant_fp4(cq, cs)
    for r in range(n):
        p, L = int(pos[r]), int(lane[r])
        keys = [wd[L, t % ring] for t in range(max(0, p - window + 1), p + 1)]
        keys += [cd[L, j] for j in sel[r, :int(cnt[r])].tolist()]
        Kmat = torch.stack(keys)
        qq = O.apply_rope(q[r].float().view(heads, hd), p, invf)
        s = (qq @ Kmat.t()) * hd ** -0.5
        m = s.max(-1, keepdim=True).values
        e = torch.exp(s - m)
        o = O.bf((e @ Kmat) / (e.sum(-1, keepdim=True) + torch.exp(sink.view(heads, 1) - m)))
        o = O.apply_rope(o, p, invf, inverse=True)
        got = out[r].cpu().float().view(heads, hd)
        assert (got - o).abs().max() <= 0.02 * o.abs().max() + 1e-4, (r, (got - o).abs().max(), o.abs().max())


def test_rows_step_is_batch_invariant_and_graph_replay_is_exact(tiny):
    from sparkflash_b200.models.deepseek_v41 import engine as E
    cfg, ck, w, orc, dw = tiny
    prompt = _prompt(cfg, 37, seed=4)
    a = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16, use_graphs=False)
    b = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16, use_graphs=True)
    single = []
    for pos, tok in enumerate(prompt):
        a.step([tok], [0], [pos])
        single.append(a.logits[0].clone())
    pos = 0
    chunked = []
    for c in (16, 5, 16):
        b.step(prompt[pos:pos + c], [1] * c, list(range(pos, pos + c)))
        chunked += [b.logits[i].clone() for i in range(c)]
        pos += c
    for i, (x, y) in enumerate(zip(single, chunked)):
        assert torch.equal(x, y), f"row {i} differs between 1-row steps and chunked rows steps"
    a.check_status(); b.check_status()


def test_generate_greedy_matches_oracle_prefix(tiny):
    from sparkflash_b200.models.deepseek_v41 import engine as E
    cfg, ck, w, orc, dw = tiny
    eng = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16)
    prompt = _prompt(cfg, 32)
    toks, logits = eng.generate(prompt, 16, collect_logits=True)
    ref, ref_logits = orc.generate(prompt, 16)
    # free-running generations stay comparable only while the tokens agree
    same = 0
    for a, b in zip(toks, ref):
        if a != b:
            break
        same += 1
    assert same >= 1
    for i in range(same):
        scale = ref_logits[i].abs().max().item()
        err = (logits[i].cpu() - ref_logits[i]).abs()
        assert err.mean().item() < 0.03 * scale and err.max().item() < 0.5 * scale


def test_tensor_core_arm_matches_cuda_core_arm_and_oracle(tiny):
    """Same model through the tcgen05 arm: per-position logits stay within the reassociation tolerance
    of the CUDA-core arm, and the first positions (no reduction-order freedom yet) agree closely with
    the oracle."""
    from sparkflash_b200.models.deepseek_v41 import engine as E
    cfg, ck, w, orc, dw = tiny
    a = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16, use_graphs=False, arm="cuda")
    b = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16, use_graphs=False, arm="tc")
    assert b.tcl[0].wqkv_a is not None and b.tcl[0].w13 is not None
    prompt = _prompt(cfg, 24, seed=8)
    st = orc.new_state()
    errs, agree = [], 0
    for pos, tok in enumerate(prompt):
        ol = orc.step(st, tok)
        a.step([tok], [0], [pos]); b.step([tok], [0], [pos])
        la, lb = a.logits[0].cpu(), b.logits[0].cpu()
        scale = ol.abs().max().item()
        if pos < 3:
            assert (lb - ol).abs().max().item() < 0.02 * scale, (pos, (lb - ol).abs().max().item())
        errs.append((la - lb).abs().mean().item() / scale)
        agree += int(la.argmax()) == int(lb.argmax())
    a.check_status(); b.check_status()
    assert sum(errs) / len(errs) < 0.03 and agree >= 0.7 * len(prompt), (sum(errs) / len(errs), agree)
    # rows step on the tensor-core arm: chunked rows reproduce the single-row logits bit for bit
    c = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16, use_graphs=True, arm="tc")
    single = []
    d_ = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16, use_graphs=False, arm="tc")
    for pos, tok in enumerate(prompt[:20]):
        d_.step([tok], [0], [pos]); single.append(d_.logits[0].clone())
    pos = 0
    for n_ in (7, 13):
        c.step(prompt[pos:pos + n_], [1] * n_, list(range(pos, pos + n_)))
        for i in range(n_):
            assert torch.equal(c.logits[i], single[pos + i]), f"row {pos + i} depends on the batch (tc arm)"
        pos += n_
    c.check_status()


@pytest.mark.parametrize("arm", ["cuda", "tc"])
def test_virtual_tensor_parallel_ranks_match_oracle_seams(tiny, arm):
    """Two tensor-parallel ranks emulated on one GPU: both ranks' engines live in this process, share one
    'symmetric' allocation and run their stages in lockstep (a rank's consumer is only launched after every
    rank's producer, so no kernel ever waits on a kernel that has not been launched).  This exercises the
    fused push / flag / rank-order-fold protocol, the TP weight slicing and the vocabulary-parallel sampler,
    against the oracle's TP-seam simulation."""
    from sparkflash_b200.models.deepseek_v41 import engine as E, oracle as O, prepare as P
    from sparkflash_b200.parallel.fused import FusedComm
    cfg, ck, w, orc, dw = tiny
    W = 2
    comms = FusedComm.local_group(W, 16, cfg.hidden_size)
    engs = []
    for r in range(W):
        e = E.Engine(P.prepare_from_checkpoint(ck, cfg, r, W), max_lanes=2, max_context=256, max_rows=16,
                     comm=comms[r], use_graphs=False, arm=arm)
        comms[r].attach_local(e)
        engs.append(e)
    orc2 = O.Oracle(cfg, w, world=W)
    st = orc2.new_state()
    prompt = _prompt(cfg, 20, seed=5)
    agree, errs = 0, []
    for pos, tok in enumerate(prompt):
        ol = orc2.step(st, tok)
        for e in engs:
            e.tokens[:1] = tok; e.row_lane[:1] = 0; e.row_pos[:1] = pos; e.temp[:1] = 0.0; e.seed[:1] = 0
        gens = [e._forward_gen(1, 1024) for e in engs]
        live = True
        while live:
            live = False
            for g in gens:
                try:
                    next(g); live = True
                except StopIteration:
                    pass
        torch.cuda.synchronize()
        for e in engs:
            e.check_status()
        logits = torch.cat([e.logits[0].cpu() for e in engs])
        scale = ol.abs().max().item()
        if pos == 0:
            assert (logits - ol).abs().max().item() < 0.02 * scale, (pos, (logits - ol).abs().max().item())
        # later positions: FP8 / FP4 rounding-boundary flips of cached values make the trajectories drift apart
        # (the same happens between two correct implementations), so the bar is statistical
        errs.append((logits - ol).abs().mean().item() / scale)
        toks = [int(e.tokens_out[0]) for e in engs]
        assert toks[0] == toks[1] == int(logits.argmax()), (toks, int(logits.argmax()))
        agree += toks[0] == int(ol.argmax())
    assert sum(errs) / len(errs) < 0.06, sum(errs) / len(errs)
    assert agree >= 0.6 * len(prompt), agree


def test_virtual_expert_parallel_ranks_match_the_single_rank_engine(tiny):
    """Expert parallelism (whole experts per rank, shared expert run by one rank per layer) on two virtual ranks in
    lockstep: same tokens on both ranks, first position within rounding of the oracle's expert-parallel seams, later ones
    statistically (a different summation grouping than tensor parallelism, same arithmetic otherwise)."""
    from sparkflash_b200.models.deepseek_v41 import engine as E, oracle as O, prepare as P
    from sparkflash_b200.parallel.fused import FusedComm
    cfg, ck, w, orc, dw = tiny
    W = 2
    comms = FusedComm.local_group(W, 16, cfg.hidden_size)
    engs = []
    for r in range(W):
        pw = P.prepare_from_checkpoint(ck, cfg, r, W, moe_mode="ep")
        assert pw.experts_local == cfg.n_routed_experts // W and pw.layers[0].w13.shape[0] == pw.experts_local
        e = E.Engine(pw, max_lanes=2, max_context=256, max_rows=16, comm=comms[r], use_graphs=False, arm="tc")
        comms[r].attach_local(e)
        engs.append(e)
    orc_ep = O.Oracle(cfg, w, world=W, moe_mode="ep")
    st = orc_ep.new_state()
    prompt = _prompt(cfg, 16, seed=7)
    agree, errs = 0, []
    for pos, tok in enumerate(prompt):
        ref = orc_ep.step(st, tok)
        for e in engs:
            e.tokens[:1] = tok; e.row_lane[:1] = 0; e.row_pos[:1] = pos; e.temp[:1] = 0.0; e.seed[:1] = 0
        gens = [e._forward_gen(1, 1024) for e in engs]
        live = True
        while live:
            live = False
            for g in gens:
                try:
                    next(g); live = True
                except StopIteration:
                    pass
        torch.cuda.synchronize()
        for e in engs:
            e.check_status()
        logits = torch.cat([e.logits[0].cpu() for e in engs])
        scale = ref.abs().max().item()
        if pos == 0:
            assert (logits - ref).abs().max().item() < 0.02 * scale, (logits - ref).abs().max().item() / scale
        errs.append((logits - ref).abs().mean().item() / scale)
        toks = [int(e.tokens_out[0]) for e in engs]
        assert toks[0] == toks[1] == int(logits.argmax())
        agree += toks[0] == int(ref.argmax())
    assert sum(errs) / len(errs) < 0.06 and agree >= 0.6 * len(prompt)


def test_grouped_moe_gives_the_bits_of_the_ungrouped_kernels(tiny):
    """Rows steps of 4+ rows sort their (token, expert) pairs by expert so that an expert is read once per segment; the per-pair
    arithmetic and the slot-order sum per token are unchanged, so the logits are bit-identical."""
    from sparkflash_b200.models.deepseek_v41 import engine as E
    cfg, ck, w, orc, dw = tiny
    prompt = _prompt(cfg, 48, seed=11)
    outs = []
    for grouped in (False, True):
        e = E.Engine(dw, max_lanes=3, max_context=256, max_rows=16, arm="tc", use_graphs=False, keep_logits=True)
        e.group_moe = grouped
        e.step(prompt[:16], [0] * 16, list(range(16)))
        e.step(prompt[16:21], [1] * 5, list(range(5)))                      # 5 rows: one short segment per expert
        e.step(prompt[21:37], [0] * 5 + [1] * 5 + [2] * 6, list(range(16, 21)) + list(range(5, 10)) + list(range(6)))   # three lanes in one step
        e.check_status()
        outs.append(e.logits[:16].clone())
    assert torch.equal(outs[0], outs[1])


def test_steps_of_more_than_64_rows_give_the_bits_of_small_steps(tiny):
    """A 128-row step runs its attention and output projections per block of 64 rows (the two-term activation copy fills a
    128-row tile with 64 rows) and everything else over all rows at once: same logits, bit for bit, as 16-row steps."""
    from sparkflash_b200.models.deepseek_v41 import engine as E
    cfg, ck, w, orc, dw = tiny
    prompt = _prompt(cfg, 200, seed=11)
    small = E.Engine(dw, max_lanes=1, max_context=256, max_rows=16, use_graphs=False, arm="tc", keep_logits=True)
    big = E.Engine(dw, max_lanes=1, max_context=256, max_rows=128, use_graphs=True, arm="tc", keep_logits=True)
    want, got = [], []
    for pos in range(0, 200, 16):
        c = prompt[pos:pos + 16]
        small.step(c, [0] * len(c), list(range(pos, pos + len(c))))
        want += [small.logits[i].clone() for i in range(len(c))]
    pos = 0
    for c_len in (128, 72):
        c = prompt[pos:pos + c_len]
        big.step(c, [0] * c_len, list(range(pos, pos + c_len)))
        got += [big.logits[i].clone() for i in range(c_len)]
        pos += c_len
    small.check_status(); big.check_status()
    for i, (x, y) in enumerate(zip(want, got)):
        assert torch.equal(x, y), f"row {i} differs"


def test_virtual_tensor_parallel_ranks_take_a_128_row_step(tiny):
    """Two lockstep tensor-parallel ranks on the tensor-core arm: a 128-row prompt step (two 64-row blocks, partial outputs
    exchanged by the generic push after the blocks) leaves the same caches as sixteen-row steps - the next decode rows sample
    the same tokens on both ranks and in both runs."""
    from sparkflash_b200.models.deepseek_v41 import engine as E, prepare as P
    from sparkflash_b200.parallel.fused import FusedComm
    cfg, ck, w, orc, dw = tiny
    W = 2
    prompt = _prompt(cfg, 128, seed=13)

    def run(max_rows, chunks):
        comms = FusedComm.local_group(W, max_rows, cfg.hidden_size)
        engs = []
        for r in range(W):
            e = E.Engine(P.prepare_from_checkpoint(ck, cfg, r, W), max_lanes=1, max_context=256, max_rows=max_rows,
                         comm=comms[r], use_graphs=False, arm="tc")
            comms[r].attach_local(e)
            engs.append(e)

        def step(tokens, positions):
            n = len(tokens)
            for e in engs:
                e.tokens[:n] = torch.tensor(tokens, dtype=torch.int32, device=e.dev)
                e.row_lane[:n] = 0
                e.row_pos[:n] = torch.tensor(positions, dtype=torch.int32, device=e.dev)
                e.temp[:n] = 0.0; e.seed[:n] = 0
            gens = [e._forward_gen(n, 1024) for e in engs]
            live = True
            while live:
                live = False
                for g in gens:
                    try:
                        next(g); live = True
                    except StopIteration:
                        pass
            torch.cuda.synchronize()
            for e in engs:
                e.check_status()
            outs = [e.tokens_out[:n].tolist() for e in engs]
            assert outs[0] == outs[1]
            return outs[0]
        pos, last = 0, None
        for c in chunks:
            last = step(prompt[pos:pos + c], list(range(pos, pos + c)))
            pos += c
        toks, tok = [], last[-1]
        for i in range(6):
            tok = step([tok], [pos + i])[0]
            toks.append(tok)
        return last, toks

    big_last, big_toks = run(128, [128])
    small_last, small_toks = run(16, [16] * 8)
    assert big_last[-16:] == small_last and big_toks == small_toks


def test_two_shot_exchange_kernels_sum_in_rank_order():
    """Reduce-scatter push, fold on the owner and all-gather push over four lockstep ranks: every rank ends up with, for
    row t, the bf16 rounding of the fp32 sum of the four partials in rank order, in slot t / rs at row rs + t % rs."""
    from sparkflash_b200.parallel.fused import FusedComm
    W, R, d, n = 4, 256, 512, 203
    comms = FusedComm.local_group(W, R, d)
    g = torch.Generator().manual_seed(5)
    parts = [(torch.randn(R, d, generator=g) * 0.7).to(torch.bfloat16).cuda() for _ in range(W)]
    status = torch.zeros(8, dtype=torch.int32, device="cuda")

    class _E:       # what FusedComm reads of an engine
        class w:
            layers = [0, 0]
    for c in comms:
        c.attach_local(_E)
        c.begin_step()
    for r, c in enumerate(comms):
        c.push_rs(parts[r], n, 1, 3)
    for c in comms:
        c.fold_push_rs(n, 1, 3, 4, status=status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    acc = torch.zeros(n, d)
    for r in range(W):
        acc += parts[r][:n].float().cpu()
    want = acc.to(torch.bfloat16)
    rs = FusedComm.rs_rows(n, W)

    class _Raw:      # a device address as a byte tensor
        def __init__(self, ptr, nbytes):
            self.__cuda_array_interface__ = {"shape": (nbytes,), "strides": None, "typestr": "|u1", "data": (ptr, False), "version": 3}

    def raw(ptr, nbytes, dtype):
        return torch.as_tensor(_Raw(ptr, nbytes), device="cuda").view(dtype)
    for c in comms:
        lay = c.layout
        got = torch.empty(n, d, dtype=torch.bfloat16)
        for j in range(W):
            lo, hi = j * rs, min(n, (j + 1) * rs)
            if hi > lo:
                slot = raw(lay.y(c.base, 1, j), R * d * 2, torch.bfloat16).view(R, d)
                got[lo:hi] = slot[rs:rs + hi - lo].cpu()
        assert torch.equal(got, want)
        flags = raw(lay.flag(c.base, 1, 0), 4 * W, torch.int32).cpu()
        epoch = int(raw(c.epoch_ptr, 4, torch.int32).cpu()[0])
        assert flags.tolist() == [epoch + 4] * W
    for c in comms:
        c.close()


def test_two_shot_seams_give_the_bits_of_the_one_shot_push(tiny):
    """A many-row step whose partial outputs cross in two shots (reduce-scatter, fold on the owner, all-gather) leaves the same
    residual stream, caches and sampled tokens as the one-shot push: the owner's sum is the sum every rank formed before."""
    from sparkflash_b200.models.deepseek_v41 import engine as E, prepare as P
    from sparkflash_b200.parallel.fused import FusedComm
    cfg, ck, w, orc, dw = tiny
    W, n = 2, 160
    prompt = _prompt(cfg, n, seed=29)
    saved = (E.Engine.TWO_SHOT_ROWS, E.Engine.TWO_SHOT_WORLD)

    def run(two_shot: bool):
        E.Engine.TWO_SHOT_ROWS, E.Engine.TWO_SHOT_WORLD = (129 if two_shot else 10 ** 9), 2
        comms = FusedComm.local_group(W, n, cfg.hidden_size)
        engs = []
        for r in range(W):
            e = E.Engine(P.prepare_from_checkpoint(ck, cfg, r, W), max_lanes=1, max_context=256, max_rows=n,
                         comm=comms[r], use_graphs=False, arm="tc")
            comms[r].attach_local(e)
            engs.append(e)
        assert engs[0]._two_shot(n) == two_shot and not engs[0]._two_shot(1)

        def step(tokens, positions):
            m = len(tokens)
            for e in engs:
                e.tokens[:m] = torch.tensor(tokens, dtype=torch.int32, device=e.dev)
                e.row_lane[:m] = 0
                e.row_pos[:m] = torch.tensor(positions, dtype=torch.int32, device=e.dev)
                e.temp[:m] = 0.0; e.seed[:m] = 0
            gens = [e._forward_gen(m, 1024) for e in engs]
            live = True
            while live:
                live = False
                for gg in gens:
                    try:
                        next(gg); live = True
                    except StopIteration:
                        pass
            torch.cuda.synchronize()
            for e in engs:
                e.check_status()
            return [e.tokens_out[:m].clone() for e in engs], [e.h[:m].clone() for e in engs]
        toks, hs = step(prompt, list(range(n)))
        tail = []
        tok = int(toks[0][-1])
        for i in range(4):
            t2, _ = step([tok], [n + i])
            tok = int(t2[0][0]); tail.append(tok)
        return toks, hs, tail
    try:
        one = run(False)
        two = run(True)
    finally:
        E.Engine.TWO_SHOT_ROWS, E.Engine.TWO_SHOT_WORLD = saved
    for r in range(W):
        assert torch.equal(one[1][r], two[1][r])        # residual copies after the last seam
        assert torch.equal(one[0][r], two[0][r])        # sampled tokens of every row
    assert one[2] == two[2]


def test_step_ledger_and_segment_identity(tiny):
    """The engine counts launches, collectives and host<->device crossings per step against a budget, and a captured
    graph is tied to the launch list it was recorded from."""
    from sparkflash_b200.models.deepseek_v41 import engine as E
    from sparkflash_b200.runtime.ledger import Budget, LedgerError, StepLedger
    cfg, ck, w, orc, dw = tiny
    eng = E.Engine(dw, max_lanes=2, max_context=256, max_rows=16, use_graphs=True, arm="tc")
    eng.ledger = StepLedger(Budget.for_rows_step(cfg.n_layers, 1, False))
    prompt = _prompt(cfg, 12, seed=3)
    eng.step(prompt[:8], [0] * 8, list(range(8)))              # captures
    eng.step(prompt[:8], [0] * 8, list(range(8)))              # replays
    got = eng.last_ledger
    assert got["problems"] == [] and got["collective"] == 0 and got["h2d"] == 5 and got["d2h"] == 1 and got["host_sync"] == 1
    assert got["launch"] == eng.launches_per_step > 0
    # the launch list of the captured 8-row step is what an eager run of the same step issues now
    eng.verify_segment(8, eng._bucket(7))
    eng.group_moe = False                                       # the experts would now run ungrouped: another launch list
    with pytest.raises(RuntimeError, match="changed since capture"):
        eng.verify_segment(8, eng._bucket(7))
    eng.group_moe = True
    # a budget that allows no result copy refuses the sampled step
    eng.ledger = StepLedger(Budget(max_d2h=0))
    with pytest.raises(LedgerError):
        eng.step(prompt[:8], [0] * 8, list(range(8)))
    eng.check_status()


def test_wide_moe_segments_and_the_persistent_kernels_give_the_bits_of_16_pair_segments(tiny):
    """Many-row steps cut the sorted (token, expert) pairs into segments of 64 instead of 16, and large launches run the
    persistent gate/up and down kernels: per-pair arithmetic and the per-token slot-order sum are unchanged, so the logits
    of a step are bit-identical under all three forms."""
    from sparkflash_b200.models.deepseek_v41 import engine as E
    from sparkflash_b200.ops import native as N
    cfg, ck, w, orc, dw = tiny
    prompt = _prompt(cfg, 60, seed=23)
    outs = []
    try:
        for wide_rows, persistent in ((10 ** 6, 1), (4, 1), (4, 2), (4, 3)):     # 3: the down kernel with one column tile per work item
            N.umma_tune(6, min(persistent, 2))
            N.umma_tune(7, persistent)
            e = E.Engine(dw, max_lanes=2, max_context=256, max_rows=64, arm="tc", use_graphs=False, keep_logits=True)
            e.GROUP_WIDE_ROWS = wide_rows
            e.step(prompt[:40], [0] * 40, list(range(40)))
            e.step(prompt[40:60], [0] * 12 + [1] * 8, list(range(40, 52)) + list(range(8)))
            e.check_status()
            outs.append(e.logits[:20].clone())
    finally:
        N.umma_tune(6, 0)
        N.umma_tune(7, 0)
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[1], outs[2])
    assert torch.equal(outs[2], outs[3])


def test_guard_bands_stay_intact_over_decode_and_chunk_steps_and_report_a_changed_band(tiny):
    """Every device buffer of a guarded engine sits between two 256-byte bands of a fixed pattern: steps of every kind leave
    them intact (no kernel writes outside its buffers), and a band changed from the host is reported with the allocation's
    source line."""
    from sparkflash_b200.models.deepseek_v41 import engine as E
    cfg, ck, w, orc, dw = tiny
    prompt = _prompt(cfg, 150, seed=5)
    plain = E.Engine(dw, max_lanes=2, max_context=256, max_rows=128, arm="tc", use_graphs=False, keep_logits=True)
    eng = E.Engine.with_guards(dw, max_lanes=2, max_context=256, max_rows=128, arm="tc", use_graphs=False, keep_logits=True)
    assert len(eng.guard_arena.records) > 20
    with eng.guard_arena.active():
        for e in (plain, eng):
            e.step(prompt[:128], [0] * 128, list(range(128)))
            e.step(prompt[128:140], [0] * 12, list(range(128, 140)))
            e.step(prompt[140:145], [1] * 5, list(range(5)))
            e.step(prompt[145:146], [0], [140])
    eng.check_status()
    assert torch.equal(plain.logits[:1], eng.logits[:1])              # the bands change nothing in the results
    rec = eng.guard_arena.records[3]
    rec.raw[-1] = 0
    with pytest.raises(RuntimeError, match="written after its bounds"):
        eng.check_status()
    rec.raw[-1] = 0xA5
    rec.raw[0] = 1
    assert "before" in eng.guard_arena.check()[0] and ".py:" in eng.guard_arena.check()[0]


def test_guard_bands_stay_intact_over_a_many_row_step_at_full_per_token_shapes():
    """The many-row path (tcgen05 attention with its staged epilogue, persistent GEMMs, 64-pair expert segments, bulk stores)
    under guard bands: a 600-row chunk whose last token tile is partial, then a decode step on the cache it filled."""
    from sparkflash_b200.config import reduced_config
    from sparkflash_b200.models.deepseek_v41 import engine as E, prepare as P
    cfg = reduced_config(8, 3)
    eng = E.Engine.with_guards(P.prepare_synthetic(cfg, 0, 1), max_lanes=2, max_context=2048, max_rows=640, arm="tc", synthetic_scales=True,
                               use_graphs=False)
    ids = torch.randint(0, cfg.vocab_size, (1300,), generator=torch.Generator().manual_seed(9)).tolist()
    with eng.guard_arena.active():
        eng.step(ids[:600], [0] * 600, list(range(600)), head="last")
        eng.step(ids[600:1200], [0] * 600, list(range(600, 1200)), head="last")
        tok = eng.step(ids[1200:1201], [0], [1200])
    eng.check_status()
    assert 0 <= int(tok[0]) < cfg.vocab_size and len(eng.guard_arena.records) > 40

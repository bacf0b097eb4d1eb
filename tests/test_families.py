"""Other model families: linear-attention / convolution state layers (reference semantics and invariances) and the
latent-recurrence ring over CPU ranks.  Reference tests: crates/sparkflash-model-qwen4-exp/tests/{batch_exactness,
verify_rows,checkpoint_roundtrip}.rs, crates/sparkflash-model-dory ring tests."""
import os

import pytest
import torch
import torch.multiprocessing as mp

from sparkflash_b200.models import linear_attn as LA


def _delta_inputs(T, H, dk, dv, per_channel, seed):
    g = torch.Generator().manual_seed(seed)
    q, k = torch.randn(T, H, dk, generator=g), torch.nn.functional.normalize(torch.randn(T, H, dk, generator=g), dim=-1)
    v = torch.randn(T, H, dv, generator=g)
    a = torch.sigmoid(torch.randn(T, H, dk if per_channel else 1, generator=g) + 2).squeeze(-1) if not per_channel else torch.sigmoid(torch.randn(T, H, dk, generator=g) + 2)
    b = torch.sigmoid(torch.randn(T, H, generator=g))
    return q, k, v, a, b


@pytest.mark.parametrize("per_channel", [False, True])
def test_delta_rule_chunk_equals_steps_and_rejected_rows_are_undone(per_channel):
    T, H, dk, dv = 9, 2, 8, 6
    q, k, v, a, b = _delta_inputs(T, H, dk, dv, per_channel, 0)
    S1, S2 = torch.zeros(H, dk, dv), torch.zeros(H, dk, dv)
    whole = LA.delta_rule_reference(q, k, v, a, b, S1)
    parts = torch.cat([LA.delta_rule_reference(q[i:j], k[i:j], v[i:j], a[i:j], b[i:j], S2) for i, j in ((0, 1), (1, 5), (5, 9))])
    assert torch.equal(whole, parts) and torch.equal(S1, S2)                  # chunk width does not change the bits
    # the memory answers what it was told: after writing (k, v) with b = 1 and no decay, reading k returns v
    S = torch.zeros(1, 4, 3); kk = torch.nn.functional.normalize(torch.randn(1, 1, 4), dim=-1); vv = torch.randn(1, 1, 3)
    o = LA.delta_rule_reference(kk, kk, vv, torch.ones(1, 1), torch.ones(1, 1), S)
    assert torch.allclose(o, vv, atol=1e-6)
    # speculative rows: snapshot, run 3 rows, reject them -> the state is exactly what it was
    snap = S1.clone()
    LA.delta_rule_reference(q[:3], k[:3], v[:3], a[:3], b[:3], S1)
    S1.copy_(snap)
    assert torch.equal(S1, S2)


def test_short_conv_history_and_softcap():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(10, 5, generator=g).to(torch.bfloat16)
    w = torch.randn(5, 4, generator=g)
    h1, h2 = torch.zeros(5, 3), torch.zeros(5, 3)
    whole = LA.short_conv_reference(x, w, h1)
    parts = torch.cat([LA.short_conv_reference(x[i:j], w, h2) for i, j in ((0, 3), (3, 4), (4, 10))])
    assert torch.equal(whole, parts) and torch.equal(h1, h2)
    # causal: output t depends on rows <= t only
    x2 = x.clone(); x2[7:] = 0
    assert torch.equal(LA.short_conv_reference(x2, w, torch.zeros(5, 3))[:7], whole[:7])
    y = LA.softcap_reference(torch.tensor([-1000.0, 0.0, 1.0, 1000.0]), 30.0)
    assert y[0] > -30.0001 and y[3] < 30.0001 and abs(float(y[2]) - 1.0) < 1e-3


@pytest.mark.gpu
def test_device_state_layers_match_references_across_lanes():
    T, H, dk, dv = 7, 3, 64, 48
    for per_channel in (False, True):
        st = LA.DeltaState(3, H, dk, dv, per_channel)
        refS = [torch.zeros(H, dk, dv) for _ in range(3)]
        for step in range(3):
            q, k, v, a, b = _delta_inputs(T, H, dk, dv, per_channel, 10 + step)
            row_lane = [2, 2, 2, 0, 0, 1, 1]                       # a prefill chunk, a verify block and a pair, one launch
            got = st.step(q.cuda(), k.cuda(), v.cuda(), a.cuda(), b.cuda(), row_lane).cpu()
            for lane in (0, 1, 2):
                idx = [i for i, l in enumerate(row_lane) if l == lane]
                want = LA.delta_rule_reference(q[idx], k[idx], v[idx], a[idx], b[idx], refS[lane])
                assert (got[idx] - want).abs().max() < 1e-4 * (1 + want.abs().max())
                assert (st.S[lane].cpu() - refS[lane]).abs().max() < 1e-4
        st.snapshot(1)
        q, k, v, a, b = _delta_inputs(2, H, dk, dv, per_channel, 99)
        before = st.S[1].clone()
        st.step(q.cuda(), k.cuda(), v.cuda(), a.cuda(), b.cuda(), [1, 1])
        assert not torch.equal(st.S[1], before)
        st.restore(1)
        assert torch.equal(st.S[1], before)
    g = torch.Generator().manual_seed(3)
    cs = LA.ConvState(2, 96, 4)
    w = torch.randn(96, 4, generator=g)
    hist = [torch.zeros(96, 3), torch.zeros(96, 3)]
    for step in range(3):
        x = torch.randn(6, 96, generator=g).to(torch.bfloat16)
        row_lane = [1, 1, 1, 1, 0, 0]
        got = cs.step(x.cuda(), w.cuda(), row_lane).float().cpu()
        for lane in (0, 1):
            idx = [i for i, l in enumerate(row_lane) if l == lane]
            want = LA.short_conv_reference(x[idx], w, hist[lane]).float()
            assert (got[idx] - want).abs().max() <= 2 ** -6 * (1 + want.abs().max())
    lg = torch.randn(4, 1000, generator=g) * 100
    assert torch.allclose(LA.softcap_(lg.clone().cuda(), 30.0).cpu(), LA.softcap_reference(lg, 30.0), atol=1e-4)
    gg, uu = torch.randn(64, 32, generator=g).to(torch.bfloat16), torch.randn(64, 32, generator=g).to(torch.bfloat16)
    want = (lambda c: (c * torch.sigmoid(c) * uu.float()))(LA.softcap_reference(gg.float(), 10.0))
    assert (LA.softcapped_swiglu(gg.cuda(), uu.cuda(), 10.0).float().cpu() - want).abs().max() < 0.05


def _ring_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from sparkflash_b200.parallel.ring import RingStage
    dist.init_process_group("gloo", rank=rank, world_size=world)
    d, loops_per_rank = 16, 2
    g = torch.Generator().manual_seed(5)
    Wm = torch.randn(d, d, generator=g) * 0.3            # the shared block: every rank holds the same weights
    head = torch.randn(50, d, generator=g)
    seen = []

    def stage(lane, pos, x):
        seen.append((lane, pos))
        for _ in range(loops_per_rank):
            x = torch.tanh(x @ Wm) + 0.1 * pos
        return x

    st = RingStage(stage, lambda lane, pos, x: (x @ head.t()).argmax(-1), d)
    if rank == 0:
        steps = [(l, p, torch.randn(1 + (l % 2), d, generator=torch.Generator().manual_seed(100 * l + p))) for p in range(3) for l in range(4)]
        out = st.drive(steps)
        st.shutdown()
        q.put(("answers", [o.tolist() for o in out]))
    else:
        q.put((f"ran{rank}", st.serve()))
    dist.barrier()
    dist.destroy_process_group()


def test_recurrence_ring_matches_one_process():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 3
    ps = [ctx.Process(target=_ring_worker, args=(r, world, 29741, q)) for r in range(world)]
    [p.start() for p in ps]
    got = dict(q.get(timeout=60) for _ in range(world))
    [p.join(20) for p in ps]
    assert got["ran1"] == 12 and got["ran2"] == 12
    # the same steps in one process: all 6 loops in a row
    d = 16
    g = torch.Generator().manual_seed(5)
    Wm = torch.randn(d, d, generator=g) * 0.3
    head = torch.randn(50, d, generator=g)
    want = []
    for p in range(3):
        for l in range(4):
            x = torch.randn(1 + (l % 2), d, generator=torch.Generator().manual_seed(100 * l + p))
            for _ in range(6):
                x = torch.tanh(x @ Wm) + 0.1 * p
            want.append((x @ head.t()).argmax(-1).tolist())
    assert got["answers"] == want

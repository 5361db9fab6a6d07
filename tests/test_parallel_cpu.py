"""Host-side logic of the multi-GPU modes on CPU: the carry chains over gloo (world size 2
and 3) and the head partition."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    from retention_integration_b200 import parallel

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)  # same data on every rank
        b, h, E, n_local = 2, 3, 40, 4
        n = n_local * world
        X = torch.randn(b, n, h, E, generator=g)
        A = -torch.rand(b, n, h, generator=g)
        dY = torch.randn(b, n, h, E, generator=g)
        # global recurrences in float64
        Y = torch.zeros(b, n + 1, h, E, dtype=torch.float64)
        for m in range(n):
            Y[:, m + 1] = Y[:, m] * torch.exp(A[:, m].double()).unsqueeze(-1) + X[:, m].double()
        Gm = torch.zeros(b, n + 1, h, E, dtype=torch.float64)
        for m in reversed(range(n)):
            Gm[:, m] = dY[:, m].double() + torch.exp(A[:, m].double()).unsqueeze(-1) * Gm[:, m + 1]
        lo, hi = rank * n_local, (rank + 1) * n_local
        # local block reductions (what the carry-only kernel passes compute)
        F = torch.zeros(b, h, E)
        for m in range(lo, hi):
            F = F * torch.exp(A[:, m]).unsqueeze(-1) + X[:, m]
        Gl = torch.zeros(b, h, E)
        for m in reversed(range(lo, hi)):
            Gl = dY[:, m] + torch.exp(A[:, m]).unsqueeze(-1) * Gl
        L = A[:, lo:hi].sum(1)
        comm = parallel.DistComm()
        C = parallel.forward_chain(comm, F, L)
        inc = parallel.backward_chain(comm, Gl, L)
        # the rank-to-rank chain gives the same carries as the single gather
        chain = parallel.ChainComm(comm)
        C2 = parallel.forward_chain(chain, F, L)
        inc2 = parallel.backward_chain(chain, Gl, L)
        ok = True
        ok &= (C is None) == (C2 is None) and (C is None or torch.allclose(C, C2, atol=1e-5))
        ok &= (inc is None) == (inc2 is None) and (inc is None or torch.allclose(inc, inc2, atol=1e-5))
        if rank == 0:
            ok &= C is None
        else:
            ok &= torch.allclose(C.double(), Y[:, lo], atol=1e-4)
        if rank == world - 1:
            ok &= inc is None
        else:
            ok &= torch.allclose(inc.double(), Gm[:, hi], atol=1e-4)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_carry_chains_over_gloo(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)


def _absent_peer_worker(rank, world, port, ret, mode):
    import datetime
    import time

    import torch.distributed as dist

    from retention_integration_b200 import parallel

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    F, L = torch.ones(1, 1, 8), torch.zeros(1, 1)
    comm = parallel.DistComm()
    if mode == "chain":
        comm = parallel.ChainComm(comm)
    if rank == 0:
        # this rank joins the group and then never takes part in the exchange (a hung or lost peer)
        time.sleep(10)
        ret[rank] = "absent"
        return
    t0 = time.time()
    try:
        parallel.forward_chain(comm, F, L)
        ret[rank] = "returned"
    except parallel.ExchangeTimeout:
        ret[rank] = f"timeout after {time.time() - t0:.1f}s"


@pytest.mark.parametrize("mode", ["gather", "chain"])
def test_exchange_with_an_absent_peer_times_out(mode):
    """A peer that never sends: the waiting rank gets ExchangeTimeout after the group's deadline (4 s here)
    instead of blocking.  Host-side fault injection only - no GPU is involved."""
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_absent_peer_worker, args=(r, 2, port, ret, mode)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    for p in procs:
        if p.is_alive():
            p.kill()
    assert str(ret.get(1, "")).startswith("timeout"), dict(ret)
    assert float(ret[1].split()[2][:-1]) < 9.0, dict(ret)


def test_mailbox_chain_matches_dist_semantics():
    from retention_integration_b200 import parallel

    world, box = 4, {}
    F = [torch.full((1, 1, 2), float(r + 1)) for r in range(world)]
    L = [torch.full((1, 1), -0.5 * (r + 1)) for r in range(world)]
    C = [parallel.forward_chain(parallel.MailboxComm(r, world, box), F[r], L[r]) for r in range(world)]
    assert C[0] is None and not box
    expect = torch.zeros(1, 1, 2)
    for r in range(1, world):
        expect = expect * torch.exp(L[r - 1]).unsqueeze(-1) + F[r - 1]
        assert torch.allclose(C[r], expect)


def test_head_slice_keeps_groups_together():
    from retention_integration_b200 import PRError, parallel

    kv, q = parallel.head_slice(8, 3, 2, 4)
    assert (kv.start, kv.stop, q.start, q.stop) == (4, 6, 12, 18)
    with pytest.raises(PRError):
        parallel.head_slice(6, 1, 0, 4)

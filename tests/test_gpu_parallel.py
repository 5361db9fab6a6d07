"""Sequence-parallel retention on one GPU: the ranks are emulated one after another with an
in-process mailbox, and the stitched result must equal the single-device call."""
import pytest
import torch
import torch.nn.functional as F

from tests._golden import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,gated", [(2, True), (4, True), (2, False)])
def test_sequence_parallel_equals_single_device(cuda_device, world, gated):
    import retention_integration_b200 as prb
    from retention_integration_b200 import _lib, parallel

    g = torch.Generator().manual_seed(world)
    b, t, h, r, d, c = 1, 2048, 2, 2, 64, 256
    Q = torch.randn(b, t, h * r, d, generator=g).bfloat16().to(cuda_device)
    K = torch.randn(b, t, h, d, generator=g).bfloat16().to(cuda_device)
    V = torch.randn(b, t, h, d, generator=g).bfloat16().to(cuda_device)
    lg = F.logsigmoid(torch.randn(b, t, h, generator=g) + 4.0).to(cuda_device) if gated else None  # slow decay
    dO = torch.randn(b, t, h * r, d, generator=g).bfloat16().to(cuda_device)

    ref_in = [x.clone().requires_grad_(True) for x in (Q, K, V)] + ([lg.clone().requires_grad_(True)] if gated else [None])
    O_ref = prb.power_retention(*ref_in, deg=2, chunk_size=c)
    O_ref.backward(dO)

    box, tl = {}, t // world
    locs, outs = [], []
    for rk in range(world):
        sl = slice(rk * tl, (rk + 1) * tl)
        ins = [x[:, sl].clone().requires_grad_(True) for x in (Q, K, V)]
        ins.append(lg[:, sl].clone().requires_grad_(True) if gated else None)
        locs.append(ins)
        outs.append(parallel.power_retention_sequence_parallel(*ins, deg=2, chunk_size=c,
                                                               comm=parallel.MailboxComm(rk, world, box)))
    assert not box
    for rk in reversed(range(world)):
        outs[rk].backward(dO[:, rk * tl:(rk + 1) * tl])
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0 and not box
    assert rel_l2(torch.cat(outs, 1).float(), O_ref.float()) < 2e-3
    for i, name in enumerate(["dQ", "dK", "dV", "dlog_G"]):
        if ref_in[i] is None:
            continue
        got = torch.cat([locs[rk][i].grad for rk in range(world)], 1).float()
        assert rel_l2(got, ref_in[i].grad.float()) < 5e-3, name


def _nccl_worker(rank, world, port, t, c, ret):
    import os

    import torch.distributed as dist

    import retention_integration_b200 as prb
    from retention_integration_b200 import parallel

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        g = torch.Generator().manual_seed(11)
        b, h, d = 1, 2, 64
        Q, K, V, dO = (torch.randn(b, t, h, d, generator=g).bfloat16().to(dev) for _ in range(4))
        lg = F.logsigmoid(torch.randn(b, t, h, generator=g) + 4.0).to(dev)
        tl = t // world
        sl = slice(rank * tl, (rank + 1) * tl)
        ins = [x[:, sl].clone().requires_grad_(True) for x in (Q, K, V, lg)]
        O = parallel.power_retention_sequence_parallel(*ins, deg=2, chunk_size=c)
        O.backward(dO[:, sl])
        full = [x.clone().requires_grad_(True) for x in (Q, K, V, lg)]
        O_ref = prb.power_retention(*full, deg=2, chunk_size=c)
        O_ref.backward(dO)
        errs = [rel_l2(O.float(), O_ref[:, sl].float())]
        errs += [rel_l2(a.grad.float(), f.grad[:, sl].float()) for a, f in zip(ins, full)]
        torch.cuda.synchronize()
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_over_nccl():
    """Real ranks, one per GPU, boundary states exchanged with NCCL send/recv."""
    import socket

    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, 4096, 256, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for r in range(world):
        assert max(ret[r]) < 5e-3, (r, ret[r])


@pytest.mark.parametrize("slices", [None, [1, 1, 2], [2, 1, 1]])
def test_host_pipeline_matches_direct_call(cuda_device, slices):
    """Pinned host tensors in, pinned host results out, head slices (equal or uneven) pipelined over three streams."""
    import retention_integration_b200 as prb
    from retention_integration_b200.host import HostPipeline

    g = torch.Generator().manual_seed(31)
    b, t, h, d, c = 1, 1024, 4, 64, 256
    Qh, Kh, Vh, dOh = (torch.randn(b, t, h, d, generator=g).bfloat16().pin_memory() for _ in range(4))
    Gh = F.logsigmoid(torch.randn(b, t, h, generator=g) + 2.0).pin_memory()
    out = {k: torch.empty(b, t, h, d, dtype=torch.bfloat16).pin_memory() for k in ("O", "dQ", "dK", "dV")}
    out["dlog_G"] = torch.empty(b, t, h).pin_memory()
    pipe = HostPipeline(b, t, h, d, torch.bfloat16, cuda_device, c, n_slices=4, slices=slices)
    for _ in range(2):  # the second round reuses every buffer
        pipe.fwd_bwd(Qh, Kh, Vh, Gh, dOh, out)
        torch.cuda.synchronize()
    ins = [x.to(cuda_device).requires_grad_(True) for x in (Qh, Kh, Vh, Gh)]
    O = prb.power_retention(*ins, deg=2, chunk_size=c)
    O.backward(dOh.to(cuda_device))
    torch.cuda.synchronize()
    assert torch.equal(out["O"], O.detach().cpu())
    for name, x in zip(("dQ", "dK", "dV", "dlog_G"), ins):
        assert torch.equal(out[name], x.grad.cpu()), name

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

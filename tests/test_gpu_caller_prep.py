"""pr_caller_prep_fwd / _bwd (split of the projection output, gate logsigmoid, rotary, layout write) against the
fixture made with the reference's own helpers and against the CPU oracle."""
import pytest
import torch

from oracle import caller_prep_oracle as cpo
from tests._golden import load as load_golden, rel_l2

pytestmark = pytest.mark.gpu


def test_against_reference_golden(cuda_device):
    """The 16-bit outputs are the reference's bit for bit; the gradient is rounded once where autograd rounds
    each of its two terms (model.py:159-164 under autograd), so it agrees to a bf16 unit."""
    import retention_integration_b200 as prb

    g = load_golden("caller_prep_nanogpt")
    B, T, h, r, d = (int(x) for x in g["meta"])
    hq = h * r
    qkvg = g["qkvg"].to(torch.bfloat16).to(cuda_device).requires_grad_(True)   # 514 columns: padded inside to 520
    sin, cos = prb.rotary_tables(T, d, cuda_device)
    assert torch.allclose(sin.cpu(), g["sin"], atol=2e-6) and torch.allclose(cos.cpu(), g["cos"], atol=2e-6)
    sin, cos = g["sin"].to(cuda_device), g["cos"].to(cuda_device)  # the fixture's own tables for the bit-exact part
    Q, K, V, log_g = prb.prepare_qkvg(qkvg, sin, cos, h, hq, d)
    for name, got in (("Q", Q), ("K", K), ("V", V)):
        assert got.is_contiguous() and torch.equal(got.float().cpu(), g[name]), name
    assert log_g.dtype == torch.float32 and torch.allclose(log_g.cpu(), g["log_g"], rtol=0, atol=2e-7)
    to = lambda k, dt: g[k].to(dt).to(cuda_device)
    torch.autograd.backward([Q, K, V, log_g], [to("dQ", torch.bfloat16), to("dK", torch.bfloat16),
                                                to("dV", torch.bfloat16), to("dlog_g", torch.float32)])
    got = qkvg.grad.float().cpu()
    assert got.shape == g["dqkvg"].shape
    assert rel_l2(got, g["dqkvg"]) < 3e-3
    assert (got - g["dqkvg"]).abs().max() <= 2.0 ** -7 * g["dqkvg"].abs().max()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,t,h,r,d,gated,half", [(2, 100, 8, 1, 64, True, False), (1, 77, 2, 4, 64, True, True),
                                                   (3, 33, 4, 2, 32, False, True), (1, 64, 8, 1, 128, True, False)])
def test_against_oracle(cuda_device, dtype, b, t, h, r, d, gated, half):
    import retention_integration_b200 as prb

    gen = torch.Generator().manual_seed(b * 100 + t)
    hq = h * r
    W = (hq + 2 * h) * d + (h if gated else 0)
    x = torch.randn(b, t, W, generator=gen).to(dtype)
    sin, cos = cpo.sinusoidal_tables(t, d)
    xr = x.clone().requires_grad_(True)
    ref = cpo.caller_prep(xr, sin, cos, h, hq, d, gated=gated, gate_bias=1.5, half_split=half)
    xd = x.to(cuda_device).requires_grad_(True)
    got = prb.prepare_qkvg(xd, sin.to(cuda_device), cos.to(cuda_device), h, hq, d, gated=gated, gate_bias=1.5,
                           half_split=half)
    grads = []
    for a, c in zip(got[:3], ref[:3]):
        assert torch.equal(a.float().cpu(), c.float())
        grads.append(torch.randn(c.shape, generator=gen).to(dtype))
    if gated:
        assert torch.allclose(got[3].cpu(), ref[3], rtol=1e-6, atol=2e-7)
        grads.append(torch.randn(b, t, h, generator=gen))
    else:
        assert got[3] is None
    n = 4 if gated else 3
    torch.autograd.backward(list(ref[:n]), grads)
    torch.autograd.backward(list(got[:n]), [gr.to(cuda_device) for gr in grads])
    assert rel_l2(xd.grad.float().cpu(), xr.grad.float()) < 3e-3


def test_large_input_properties(cuda_device):
    """b1 t65536 h8 d64 (the benchmark's shape, 202 MB of projection output): rotation keeps every pair's norm,
    values pass through untouched, and the gradient kernel applied to the forward's own outputs undoes the rotation."""
    import retention_integration_b200 as prb
    from retention_integration_b200 import ops

    b, t, h, d = 1, 65536, 8, 64
    W = 3 * h * d + h
    gen = torch.Generator(device=cuda_device).manual_seed(1)
    x = torch.randn(b, t, W, generator=gen, device=cuda_device).bfloat16()
    sin, cos = prb.rotary_tables(t, d, cuda_device)
    Q, K, V, log_g = prb.prepare_qkvg(x, sin, cos, h, h, d)
    assert torch.equal(V.view(b, t, h * d), x[..., 2 * h * d:3 * h * d])
    q_in = x[..., : h * d].view(b, t, h, d).float()
    n_in = (q_in[..., ::2] ** 2 + q_in[..., 1::2] ** 2).sqrt()
    n_out = (Q.float()[..., ::2] ** 2 + Q.float()[..., 1::2] ** 2).sqrt()
    assert (n_out - n_in).abs().max() <= 2.0 ** -7 * n_in.max()
    assert (log_g <= 0).all() and torch.isfinite(log_g).all()
    back = ops.caller_prep_bwd(x, cos, sin, h, h, d, True, prb.caller.GATE_BIAS, False, Q, K, V, torch.zeros_like(log_g))
    assert rel_l2(back[..., : 2 * h * d].float(), x[..., : 2 * h * d].float()) < 4e-3
    assert torch.equal(back[..., 2 * h * d:3 * h * d], x[..., 2 * h * d:3 * h * d])


def test_refusals(cuda_device):
    import retention_integration_b200 as prb

    sin, cos = prb.rotary_tables(16, 64, cuda_device)
    x = torch.randn(1, 16, 3 * 64 + 1, device=cuda_device).bfloat16()
    with pytest.raises(prb.PRError):
        prb.prepare_qkvg(x.float(), sin, cos, 1, 1, 64)
    with pytest.raises(prb.PRError):
        prb.prepare_qkvg(x[..., :100], sin, cos, 1, 1, 64)
    with pytest.raises(prb.PRError):
        prb.prepare_qkvg(x, sin[:8], cos[:8], 1, 1, 64)

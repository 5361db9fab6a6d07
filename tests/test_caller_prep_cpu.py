"""The caller-glue oracle against the fixture made with the reference's own rotary helpers
(deploy/nanoGPT/model.py:66-84, :143-164)."""
import torch

from oracle import caller_prep_oracle as cpo
from tests._golden import load as load_golden


def test_oracle_reproduces_the_reference_glue():
    g = load_golden("caller_prep_nanogpt")
    B, T, h, r, d = (int(x) for x in g["meta"])
    hq = h * r
    qkvg = g["qkvg"].to(torch.bfloat16).requires_grad_(True)
    sin, cos = cpo.sinusoidal_tables(T, d)
    assert torch.equal(sin, g["sin"]) and torch.equal(cos, g["cos"])
    Q, K, V, log_g = cpo.caller_prep(qkvg, sin, cos, h, hq, d)
    for name, got in (("Q", Q), ("K", K), ("V", V)):
        assert torch.equal(got.float(), g[name]), name          # 16-bit results: bit for bit
    assert torch.allclose(log_g, g["log_g"], rtol=0, atol=1e-7)
    torch.autograd.backward([Q, K, V, log_g], [g["dQ"].to(torch.bfloat16), g["dK"].to(torch.bfloat16),
                                                g["dV"].to(torch.bfloat16), g["dlog_g"]])
    assert torch.equal(qkvg.grad.float(), g["dqkvg"])


def test_rotary_is_a_rotation_in_both_pairings():
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(2, 40, 3, 32, generator=gen)
    sin, cos = cpo.sinusoidal_tables(40, 32)
    for half in (False, True):
        y = cpo.rotary(x, sin, cos, half)
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
        back = cpo.rotary(y, -sin, cos, half)  # rotating by the opposite angle undoes it
        assert torch.allclose(back, x, atol=1e-5)


def test_product_path_refuses_host_tensors():
    """No CPU fallback: the package's prepare_qkvg raises on anything but CUDA 16-bit tensors."""
    import pytest

    import retention_integration_b200 as prb

    x = torch.randn(1, 8, 3 * 64 + 8).bfloat16()
    sin, cos = cpo.sinusoidal_tables(8, 64)
    with pytest.raises(prb.PRError):
        prb.prepare_qkvg(x, sin, cos, 1, 1, 64)
    s2, c2 = prb.rotary_tables(8, 64, "cpu")  # the table helper itself is plain torch
    assert torch.allclose(s2, sin) and torch.allclose(c2, cos)

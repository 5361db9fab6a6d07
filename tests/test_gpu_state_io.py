"""initial_state / return_final_state of power_retention (retention/power_retention_maker.py:131-140,158-172,
left unfinished in the reference): a sequence processed in two segments, the second continuing from the
state the first one returns, must reproduce the one-pass result - outputs, the gradients of the second
segment's inputs, and the state itself against its definition evaluated token by token in float64."""
import pytest
import torch
import torch.nn.functional as F

from oracle import power_retention_oracle as oracle
from tests._golden import rel_l2

pytestmark = pytest.mark.gpu


def _inputs(b, t, h, r, gated, seed):
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn(b, t, h * r, 64, generator=g).bfloat16()
    K = torch.randn(b, t, h, 64, generator=g).bfloat16()
    V = torch.randn(b, t, h, 64, generator=g).bfloat16()
    lg = F.logsigmoid(torch.randn(b, t, h, generator=g) + 2.0) if gated else None
    dO = torch.randn(b, t, h * r, 64, generator=g).bfloat16()
    return Q, K, V, lg, dO


def _exact_state_f64(K, V, lg):
    """S = sum_j e^{a_T - a_j} w phi(k_j) v_j^T and its normaliser, exact layout, float64."""
    b, t, h, d = K.shape
    K, V = K.double(), V.double()
    decay = torch.ones(b, t, h, dtype=torch.float64)
    if lg is not None:
        a = lg.double().cumsum(1)
        decay = torch.exp(a[:, -1:] - a)
    ia, ib = torch.triu_indices(d, d)
    w = torch.where(ia == ib, 1.0, 2.0).double()
    phi = K[..., ia] * K[..., ib] * w * decay.unsqueeze(-1)          # [b,t,h,D]
    S = torch.einsum("bthD,bthe->bhDe", phi, V)
    return S, phi.sum(1)


@pytest.mark.parametrize("t1,t2,chunk,gated,r", [(512, 512, 128, True, 1), (384, 640, 128, False, 2),
                                                 (300, 724, 256, True, 1), (256, 100, None, True, 1)])
def test_two_segments_equal_one_pass(cuda_device, t1, t2, chunk, gated, r):
    import retention_integration_b200 as prb

    b, h = 2, 2
    t = t1 + t2
    Q, K, V, lg, dO = _inputs(b, t, h, r, gated, seed=t1 + t2)
    dev = cuda_device
    seg = lambda x, lo, hi: None if x is None else x[:, lo:hi].to(dev)
    # segment 1 -> state
    _, st = prb.power_retention(seg(Q, 0, t1), seg(K, 0, t1), seg(V, 0, t1), seg(lg, 0, t1), return_final_state=True,
                                chunk_size=chunk)
    state, sok = st
    assert state.shape == (b, h, 2080, 64) and sok.shape == (b, h, 2080) and sok.dtype == torch.float32
    S_ref, s_ref = _exact_state_f64(K[:, :t1], V[:, :t1], None if lg is None else lg[:, :t1])
    assert rel_l2(state.float().cpu(), S_ref) < 1e-2
    assert rel_l2(sok.cpu(), s_ref) < 5e-3
    # segment 2 continues from it
    leaves = [seg(x, t1, t).requires_grad_(True) for x in (Q, K, V)]
    g2 = seg(lg, t1, t).requires_grad_(True) if gated else None
    O2, st2 = prb.power_retention(*leaves, g2, initial_state=(state, sok), return_final_state=True, chunk_size=chunk)
    O2.backward(seg(dO, t1, t))
    torch.cuda.synchronize()
    # one pass over the whole sequence in fp32 on the CPU oracle, upstream gradient on segment 2 only
    ref_leaves = [x.float().requires_grad_(True) for x in (Q, K, V)]
    ref_g = lg.clone().requires_grad_(True) if gated else None
    O_ref = oracle.power_retention(*ref_leaves, ref_g, deg=2, chunk_size=128)
    dO_full = dO.float().clone()
    dO_full[:, :t1] = 0
    O_ref.backward(dO_full)
    assert rel_l2(O2.float().cpu(), O_ref[:, t1:]) < 2e-2
    for name, ours, ref in zip(("dQ", "dK", "dV"), leaves, ref_leaves):
        assert rel_l2(ours.grad.float().cpu(), ref.grad[:, t1:]) < 2e-2, name
    if gated:
        assert rel_l2(g2.grad.cpu(), ref_g.grad[:, t1:]) < 2e-2
    # and the state after both segments is the state of the whole sequence
    S_all, s_all = _exact_state_f64(K, V, lg)
    assert rel_l2(st2[0].float().cpu(), S_all) < 1e-2
    assert rel_l2(st2[1].cpu(), s_all) < 5e-3


def test_final_state_feeds_the_inference_operator(cuda_device):
    """Chunked prefill -> state -> decode: equals the quadratic form over the whole sequence."""
    import retention_integration_b200 as prb

    b, h, t0, steps = 2, 2, 640, 4
    Q, K, V, lg, _ = _inputs(b, t0 + steps, h, 1, True, seed=9)
    ref = oracle.power_retention_quadratic(Q, K, V, lg)
    dev = cuda_device
    Qd, Kd, Vd, ld = (x.to(dev) for x in (Q, K, V, lg))
    Y0, (state, sok) = prb.power_retention(Qd[:, :t0], Kd[:, :t0], Vd[:, :t0], ld[:, :t0], return_final_state=True,
                                           chunk_size=128)
    assert rel_l2(Y0.float().cpu(), ref[:, :t0].float()) < 2e-2
    for i in range(steps):
        lo, hi = t0, t0 + i + 1
        Y, _, _ = prb.power_retention_inference(Qd[:, hi - 1:hi], Kd[:, lo:hi], Vd[:, lo:hi], ld[:, lo:hi], state, sok,
                                                switch_over_seq_len=1024)
        assert rel_l2(Y.float().cpu(), ref[:, hi - 1:hi].float()) < 1e-2, i

"""power_retention_inference on a B200: the reference's golden outputs (decode with a state,
switch-over, state-only query, several query tokens) and the recurrence's own invariants."""
import pytest
import torch
import torch.nn.functional as F

from oracle import power_retention_oracle as oracle
from tests._golden import load, make_state, rel_l2

pytestmark = pytest.mark.gpu


def _dev(x, dev, dtype=None):
    if x is None:
        return None
    return x.to(dev) if dtype is None else x.to(dtype).to(dev)


@pytest.mark.parametrize("name", ["infer_decode_state", "infer_switch_over", "infer_no_state_switch",
                                  "infer_state_only", "infer_prefill_with_state"])
def test_against_reference_golden(cuda_device, name):
    import retention_integration_b200 as prb
    from retention_integration_b200 import _lib, layout

    g = load(name)
    b, tq, tk, h, r, d, with_state, sw = g["meta"]
    bf = torch.bfloat16
    state = sk = None
    if with_state:  # fixtures hold the reference's padded layout
        state = _dev(layout.from_reference_layout(g["state"], d), cuda_device, bf)
        sk = _dev(layout.from_reference_layout(g["sum_of_keys"], d, dim=-1), cuda_device)
    Y, ns, nk = prb.power_retention_inference(_dev(g["Q"], cuda_device, bf), _dev(g.get("K"), cuda_device, bf),
                                              _dev(g.get("V"), cuda_device, bf), _dev(g.get("log_G"), cuda_device),
                                              state, sk, deg=2, switch_over_seq_len=sw)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    assert rel_l2(Y.float().cpu(), g["Y"]) < 1e-2
    if tk >= sw:
        assert ns.shape == (b, h, layout.exact_dim(d), d) and nk.shape == (b, h, layout.exact_dim(d))
        assert rel_l2(ns.float().cpu(), layout.from_reference_layout(g["new_state"], d)) < 1e-2
        assert rel_l2(nk.cpu(), layout.from_reference_layout(g["new_sum_of_keys"], d, dim=-1)) < 5e-3  # keys are discounted in 16-bit here, in fp32 in the fixture
        # and back: the reference's own layout
        assert rel_l2(layout.to_reference_layout(layout.from_reference_layout(g["new_state"], d), d).sum(-2),
                      g["new_state"].sum(-2)) < 1e-5
    else:
        assert ns is state and nk is sk  # same objects, like the reference


def test_state_feedback_reproduces_output(cuda_device):
    """After a switch-over, querying the new state alone gives the same output
    (the reference's inference_tests.py:39-51; atol 1e-2, rtol 1e-3 there)."""
    import retention_integration_b200 as prb

    g = torch.Generator().manual_seed(3)
    b, tk, h, r, d = 2, 128, 2, 2, 64
    Q = (torch.randn(b, 1, h * r, d, generator=g) / 8).bfloat16().to(cuda_device)
    K = (torch.randn(b, tk, h, d, generator=g) / 8).bfloat16().to(cuda_device)
    V = (torch.randn(b, tk, h, d, generator=g) / 8).bfloat16().to(cuda_device)
    lg = F.logsigmoid(6.9 + torch.randn(b, tk, h, generator=g)).to(cuda_device)
    Y1, s1, k1 = prb.power_retention_inference(Q, K, V, lg, switch_over_seq_len=128)
    Y2, s2, k2 = prb.power_retention_inference(Q, None, None, None, s1, k1, switch_over_seq_len=128)
    assert s2 is s1 and k2 is k1
    assert torch.allclose(Y1.float(), Y2.float(), atol=1e-2, rtol=1e-2)


def test_prefill_then_decode_matches_full_sequence(cuda_device):
    """Compress a prefix into a state, then decode token by token with a growing cache: every
    output equals the quadratic form over the whole sequence."""
    import retention_integration_b200 as prb

    g = torch.Generator().manual_seed(4)
    b, t0, steps, h, d = 2, 256, 6, 2, 64
    t = t0 + steps
    Q, K, V = (torch.randn(b, t, h, d, generator=g).bfloat16() for _ in range(3))
    lg = F.logsigmoid(torch.randn(b, t, h, generator=g) + 3.0)
    ref = oracle.power_retention_quadratic(Q, K, V, lg)
    Qd, Kd, Vd, ld = (x.to(cuda_device) for x in (Q, K, V, lg))
    # the first call sees the whole prefix as its cache and compresses it (tk >= switch_over)
    Y, state, sk = prb.power_retention_inference(Qd[:, t0 - 1:t0], Kd[:, :t0], Vd[:, :t0], ld[:, :t0],
                                                 switch_over_seq_len=t0)
    assert rel_l2(Y.float().cpu(), ref[:, t0 - 1:t0].float()) < 1e-2
    assert state.shape == (b, h, 2080, d) and sk.shape == (b, h, 2080)
    for i in range(steps):
        lo, hi = t0, t0 + i + 1
        Y, s2, k2 = prb.power_retention_inference(Qd[:, hi - 1:hi], Kd[:, lo:hi], Vd[:, lo:hi], ld[:, lo:hi], state,
                                                  sk, switch_over_seq_len=1024)
        assert s2 is state and k2 is sk
        assert rel_l2(Y.float().cpu(), ref[:, hi - 1:hi].float()) < 1e-2, i


@pytest.mark.parametrize("ratio", [1, 4])
def test_decode_reads_cache_slices_in_place(cuda_device, ratio):
    """A query and a cache that are slices [:, :tk] of longer preallocated tensors (a serving loop's KV and gate
    cache) give bit-identical results to dense copies, with and without GQA, while the cache grows."""
    import retention_integration_b200 as prb

    g = torch.Generator().manual_seed(41)
    b, h, d, cap = 3, 2, 64, 40
    hq = h * ratio
    mk = lambda *s: torch.randn(*s, generator=g).bfloat16().to(cuda_device)
    Kc, Vc, Qs = mk(b, cap, h, d), mk(b, cap, h, d), mk(b, cap, hq, d)
    lgc = F.logsigmoid(torch.randn(b, cap, h, generator=g) + 1.0).to(cuda_device)
    K0, V0 = mk(b, 256, h, d), mk(b, 256, h, d)
    lg0 = F.logsigmoid(torch.randn(b, 256, h, generator=g) + 1.0).to(cuda_device)
    _, state, sk = prb.power_retention_inference(mk(b, 1, hq, d), K0, V0, lg0, switch_over_seq_len=256)
    for tk in (1, 7, 33, cap):
        q, k, v, lg = Qs[:, tk - 1:tk], Kc[:, :tk], Vc[:, :tk], lgc[:, :tk]
        assert not k.is_contiguous() or tk == cap
        y_view, _, _ = prb.power_retention_inference(q, k, v, lg, state, sk, switch_over_seq_len=1024)
        y_copy, _, _ = prb.power_retention_inference(q.contiguous(), k.contiguous(), v.contiguous(),
                                                     lg.contiguous(), state, sk, switch_over_seq_len=1024)
        torch.cuda.synchronize()
        assert torch.equal(y_view, y_copy), tk
        assert torch.isfinite(y_view).all()


def _decode_vs_oracle(dev, b, h, r, tk, seed, check_rows, dtype=torch.bfloat16, gate_shift=0.0):
    """One decode step (tq = 1, state given) against oracle.power_retention_inference, compared on the
    (batch, kv head) pairs in `check_rows` (the oracle expands every query, so a few pairs keep it quick)."""
    import retention_integration_b200 as prb
    from retention_integration_b200 import layout

    g = torch.Generator().manual_seed(seed)
    d, D = 64, 2080
    hq = h * r
    Q = torch.randn(b, 1, hq, d, generator=g).to(dtype)
    state, sok = make_state(b, h, d, 24, g)
    state = state.to(dtype)
    K = V = lg = None
    if tk > 0:
        K = torch.randn(b, tk, h, d, generator=g).to(dtype)
        V = torch.randn(b, tk, h, d, generator=g).to(dtype)
        lg = F.logsigmoid(torch.randn(b, tk, h, generator=g) + gate_shift)
    to = lambda x: None if x is None else x.to(dev)
    Y, s2, k2 = prb.power_retention_inference(to(Q), to(K), to(V), to(lg), to(state), to(sok),
                                              switch_over_seq_len=1024)
    torch.cuda.synchronize()
    assert torch.isfinite(Y.float()).all()
    for bi, hi in check_rows:
        sl_q = slice(hi * r, (hi + 1) * r)
        cut = lambda x: None if x is None else x[bi:bi + 1, :, hi:hi + 1]
        st_ref = layout.to_reference_layout(state[bi:bi + 1, hi:hi + 1].float(), d)
        sk_ref = layout.to_reference_layout(sok[bi:bi + 1, hi:hi + 1], d, dim=-1)
        Kc, Vc = cut(K), cut(V)
        Y_ref, _, _ = oracle.power_retention_inference(
            Q[bi:bi + 1, :, sl_q].float(), None if Kc is None else Kc.float(), None if Vc is None else Vc.float(),
            cut(lg), st_ref, sk_ref, deg=2, switch_over_seq_len=1024)
        assert rel_l2(Y[bi:bi + 1, :, sl_q].float().cpu(), Y_ref) < 1e-2, (bi, hi, tk)


@pytest.mark.parametrize("tk", [0, 1, 300])
def test_decode_at_benchmark_shape_unsplit_state_read(cuda_device, tk):
    """b16 h32: 512 (batch, head) pairs, so every CTA of the state read walks all 2080 rows of its state
    (no split of the expanded dimension) - the path the decode benchmark runs."""
    _decode_vs_oracle(cuda_device, 16, 32, 1, tk, seed=100 + tk,
                      check_rows=[(0, 0), (7, 13), (15, 31), (3, 30)])


@pytest.mark.parametrize("b,h,r,tk", [(8, 24, 1, 65), (6, 32, 1, 0), (10, 20, 4, 17), (2, 3, 1, 9)])
def test_decode_state_read_split_in_two_and_five(cuda_device, b, h, r, tk):
    """192-200 (batch, head) pairs: the expanded dimension is read in two halves; 6 pairs: in five parts."""
    _decode_vs_oracle(cuda_device, b, h, r, tk, seed=b * h + tk, check_rows=[(0, 0), (b - 1, h - 1), (b // 2, h // 2)])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,h,r,tk", [(16, 32, 1, 1500), (4, 8, 2, 700), (2, 2, 8, 1300)])
def test_decode_long_cache_both_dtypes(cuda_device, dtype, b, h, r, tk):
    """Caches longer than one gate block of the attention warps (640 tokens: the suffix sums carry over from block
    to block), query-head groups of two and of eight (two CTAs per kv head), fp16 as well as bf16 states.  Slow
    gates keep the oldest cached tokens' weights alive, so a lost carry would show."""
    _decode_vs_oracle(cuda_device, b, h, r, tk, seed=3 * b + tk, check_rows=[(0, 0), (b - 1, h - 1)], dtype=dtype,
                      gate_shift=5.0)

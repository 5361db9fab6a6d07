"""Parity of power_retention (forward and backward) on a B200 against the CPU oracle, the
reference's golden fixtures, and size-independent properties at the benchmark size.

Tolerance (stated by the task): relative L2 <= 2e-2 against an fp32 run of the reference
for bf16/fp16 inputs, and at least as close as the reference's own 16-bit path, which is
measured here by running the oracle in bf16 on the same inputs.
"""
import pytest
import torch
import torch.nn.functional as F

from oracle import power_retention_oracle as oracle
from tests._golden import load, rel_l2

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _run_ours(dev, Q, K, V, lg, dO, chunk, **kw):
    import retention_integration_b200 as prb
    from retention_integration_b200 import _lib

    leaves = [x.to(dev).requires_grad_(True) for x in (Q, K, V)]
    g = lg.to(dev).requires_grad_(True) if lg is not None else None
    O = prb.power_retention(leaves[0], leaves[1], leaves[2], g, deg=2, chunk_size=chunk, **kw)
    O.backward(dO.to(dev))
    torch.cuda.synchronize()
    assert _lib.device_status(dev.index or 0) == 0
    out = {"O": O, "dQ": leaves[0].grad, "dK": leaves[1].grad, "dV": leaves[2].grad}
    if g is not None:
        out["dlog_G"] = g.grad
    return {k: v.detach().float().cpu() for k, v in out.items()}


def _run_oracle(Q, K, V, lg, dO, chunk, dtype):
    leaves = [x.to(dtype).requires_grad_(True) for x in (Q, K, V)]
    g = lg.clone().requires_grad_(True) if lg is not None else None
    O = oracle.power_retention(leaves[0], leaves[1], leaves[2], g, deg=2, chunk_size=chunk)
    O.backward(dO.to(dtype))
    out = {"O": O, "dQ": leaves[0].grad, "dK": leaves[1].grad, "dV": leaves[2].grad}
    if g is not None:
        out["dlog_G"] = g.grad
    return {k: v.detach().float() for k, v in out.items()}


def _case(b, t, h, r, d, gated, shift, seed, dtype=torch.bfloat16, in_scale=1.0):
    g = torch.Generator().manual_seed(seed)
    Q = (torch.randn(b, t, h * r, d, generator=g) * in_scale).to(dtype)
    K = (torch.randn(b, t, h, d, generator=g) * in_scale).to(dtype)
    V = (torch.randn(b, t, h, d, generator=g) * in_scale).to(dtype)
    lg = F.logsigmoid(torch.randn(b, t, h, generator=g) + shift) if gated else None
    dO = torch.randn(b, t, h * r, d, generator=g).to(dtype)
    return Q, K, V, lg, dO


# grid modelled on the reference's own (perf/tests/test_list.py:248-259): t in {31,128,1024,2000},
# chunk in {None,128}, gated or not; plus GQA, a long chunk and slow/fast decay.
CASES = [
    # b, t, h, r, gated, shift, chunk
    (1, 31, 2, 1, True, 0.0, None),
    (1, 128, 2, 1, False, 0.0, None),
    (1, 128, 2, 1, True, 0.0, 128),
    (1, 1024, 2, 1, True, 0.0, 128),
    (1, 1024, 2, 1, False, 0.0, 128),
    (1, 2000, 2, 1, True, 2.0, 128),   # padding
    (2, 512, 2, 2, True, 4.0, 256),    # GQA + slow decay
    (1, 600, 1, 8, False, 0.0, 128),   # GQA ratio 8 + padding
    (1, 2048, 1, 1, True, 0.0, 1024),  # the benchmark's chunk size
    (1, 4096, 1, 1, True, 0.0, 1024),  # four chunks of it: middle chunks carry state terms on both sides
    (1, 5120, 1, 2, False, 0.0, 1024), # five chunks, ungated, GQA
    (1, 300, 2, 1, True, 2.0, None),   # quadratic branch, ragged length
    (1, 768, 2, 1, True, 1.0, 192),    # chunk not a multiple of the 128-row tile (second tile half empty)
    (1, 480, 1, 2, True, 0.0, 96),     # chunk shorter than a tile, ragged 64-key steps, GQA
    (1, 1280, 2, 1, False, 0.0, 320),  # two and a half tiles per chunk, ungated
]


@pytest.mark.parametrize("b,t,h,r,gated,shift,chunk", CASES)
def test_forward_backward_vs_fp32_oracle(cuda_device, b, t, h, r, gated, shift, chunk):
    Q, K, V, lg, dO = _case(b, t, h, r, 64, gated, shift, seed=t + h)
    ours = _run_ours(cuda_device, Q, K, V, lg, dO, chunk)
    gold = _run_oracle(Q, K, V, lg, dO, chunk, torch.float32)
    ref16 = _run_oracle(Q, K, V, lg, dO, chunk, torch.bfloat16)
    for key in gold:
        err, err16 = rel_l2(ours[key], gold[key]), rel_l2(ref16[key], gold[key])
        assert err < TOL, (key, err)
        assert err < 1.5 * err16 + 1e-3, (key, err, err16)  # as close as the 16-bit reference path


@pytest.mark.parametrize("lo,hi", [(-4.0, -2.0), (0.0, 0.2)])
def test_extreme_gates(cuda_device, lo, hi):
    """Very fast decay (pair weights underflow inside a chunk, where the separable gate factors of the
    attention kernels flush to zero) and growing gates (log G > 0, factors above one)."""
    Q, K, V, _, dO = _case(1, 512, 2, 1, 64, False, 0.0, seed=5)
    g = torch.Generator().manual_seed(6)
    lg = lo + (hi - lo) * torch.rand(1, 512, 2, generator=g)
    ours = _run_ours(cuda_device, Q, K, V, lg, dO, 256)
    gold = _run_oracle(Q, K, V, lg, dO, 256, torch.float32)
    ref16 = _run_oracle(Q, K, V, lg, dO, 256, torch.bfloat16)
    for key in gold:
        assert torch.isfinite(ours[key]).all(), key
        err, err16 = rel_l2(ours[key], gold[key]), rel_l2(ref16[key], gold[key])
        # with growing gates the gate gradient of late tokens is a difference of large sums that cancel:
        # the reference's own 16-bit path is at 4.8e-2 there, so the bound is relative to it
        assert err < max(TOL, 1.5 * err16), (key, err, err16)


@pytest.mark.parametrize("t,scale,gated,r", [(128, 1.0, True, 1), (1024, 0.125, False, 1), (300, 0.125, True, 2)])
def test_degree_four_on_the_state_free_branch(cuda_device, t, scale, gated, r):
    """deg = 4 is in the reference's attention grid (perf/tests/test_list.py:55); its state operators stop at
    deg 2, so like there it is available where no state is formed (chunk_size None)."""
    import retention_integration_b200 as prb

    Q, K, V, lg, dO = _case(1, t, 2, r, 64, gated, 2.0, seed=t, in_scale=0.35)
    dev = cuda_device
    leaves = [x.to(dev).requires_grad_(True) for x in (Q, K, V)]
    g = lg.to(dev).requires_grad_(True) if gated else None
    O = prb.power_retention(*leaves, g, deg=4, scale=scale, chunk_size=None)
    O.backward(dO.to(dev))
    ref = [x.float().requires_grad_(True) for x in (Q, K, V)]
    rg = lg.clone().requires_grad_(True) if gated else None
    O_ref = oracle.power_retention(*ref, rg, deg=4, scale=scale, chunk_size=None)
    O_ref.backward(dO.float())
    assert rel_l2(O.float().cpu(), O_ref) < TOL
    for name, a, b in zip(("dQ", "dK", "dV"), leaves, ref):
        assert rel_l2(a.grad.float().cpu(), b.grad) < TOL, name
    if gated:
        assert rel_l2(g.grad.cpu(), rg.grad) < TOL


@pytest.mark.parametrize("d,chunk", [(32, 128), (16, None), (48, 64)])
def test_small_head_dims_run_on_padded_features(cuda_device, d, chunk):
    """d in {16, 32, 48}: zero-padded to the 64-wide kernels, exact (the reference's grids hold d = 32)."""
    Q, K, V, lg, dO = _case(1, 512, 2, 2, d, True, 2.0, seed=d)
    ours = _run_ours(cuda_device, Q, K, V, lg, dO, chunk)
    gold = _run_oracle(Q, K, V, lg, dO, chunk, torch.float32)
    for key in gold:
        assert ours[key].shape == gold[key].shape
        assert rel_l2(ours[key], gold[key]) < TOL, key


def test_fp16_inputs(cuda_device):
    Q, K, V, lg, dO = _case(1, 512, 2, 1, 64, True, 2.0, seed=77, dtype=torch.float16, in_scale=0.5)
    ours = _run_ours(cuda_device, Q, K, V, lg, dO, 128)
    gold = _run_oracle(Q, K, V, lg, dO, 128, torch.float32)
    for key in gold:
        assert rel_l2(ours[key], gold[key]) < TOL, key


@pytest.mark.parametrize("auto_chunk", [False, True])
@pytest.mark.parametrize("name", ["train_gated_fp32", "train_slow_decay_fp32", "train_gated_bf16",
                                  "train_ungated_gqa_pad_fp32", "train_short_quadratic_fp32"])
def test_against_reference_golden_outputs(cuda_device, name, auto_chunk):
    """Same seeded inputs as the reference run that produced the fixture (inputs are bf16-exact); with the chunk
    size the reference ran with, and with the one the package would choose by itself."""
    from retention_integration_b200 import retention

    retention.AUTO_CHUNK = auto_chunk
    g = load(name)
    b, t, h, d, r, gated, chunk, stride = g["meta"]
    ours = _run_ours(cuda_device, g["Q"].bfloat16(), g["K"].bfloat16(), g["V"].bfloat16(),
                     g["log_G"] if gated else None, g["dO"].bfloat16(), chunk or None)
    tol = TOL if name.endswith("fp32") else 2.5e-2  # bf16 fixture: both sides carry 16-bit noise
    for key in ("O", "dQ", "dK", "dV") + (("dlog_G",) if gated else ()):
        assert rel_l2(ours[key][:, ::stride], g[key]) < tol, key


@pytest.mark.parametrize("auto_chunk", [False, True])
def test_cfg1_shape_against_reference_golden(cuda_device, auto_chunk):
    from retention_integration_b200 import retention

    retention.AUTO_CHUNK = auto_chunk
    g = load("train_cfg1_fp32")  # b1 t1024 h4 d64 c128 gated: the reference's CPU-runnable case
    ours = _run_ours(cuda_device, g["Q"].bfloat16(), g["K"].bfloat16(), g["V"].bfloat16(), g["log_G"],
                     g["dO"].bfloat16(), 128)
    for key in ("O", "dQ", "dK", "dV", "dlog_G"):
        assert rel_l2(ours[key][:, ::8], g[key]) < TOL, key


def test_chunk_size_invariance_and_determinism(cuda_device):
    """Chunked == quadratic, as in the reference's chunk-consistency test
    (perf/tests/chunk_consistency_tests.py:22-45); two runs are bitwise identical."""
    Q, K, V, lg, dO = _case(1, 1024, 2, 1, 64, True, 3.0, seed=5)
    a = _run_ours(cuda_device, Q, K, V, lg, dO, 128)
    a2 = _run_ours(cuda_device, Q, K, V, lg, dO, 128)
    bq = _run_ours(cuda_device, Q, K, V, lg, dO, None)
    c = _run_ours(cuda_device, Q, K, V, lg, dO, 256)
    for key in a:
        assert torch.equal(a[key], a2[key]), key
        assert rel_l2(a[key], bq[key]) < 1e-2, key
        assert rel_l2(a[key], c[key]) < 1e-2, key


@pytest.mark.parametrize("gated,r", [(True, 1), (False, 2)])
def test_native_sequencer_equals_python_sequencer(cuda_device, gated, r):
    """pr_retention_fwd / pr_retention_bwd launch the same kernels in the same order as the Python-driven
    sequence: bit-identical outputs and gradients."""
    from retention_integration_b200 import retention

    Q, K, V, lg, dO = _case(2, 768, 2, r, 64, gated, 1.0, seed=12)
    try:
        retention.NATIVE_SEQUENCER = True
        a = _run_ours(cuda_device, Q, K, V, lg, dO, 128)
        retention.NATIVE_SEQUENCER = False
        b = _run_ours(cuda_device, Q, K, V, lg, dO, 128)
    finally:
        retention.NATIVE_SEQUENCER = True
    for key in a:
        assert torch.equal(a[key], b[key]), key


def test_step_captured_in_a_cuda_graph_replays_bit_identically(cuda_device):
    """A forward+backward captured from the caller's stream replays to the same bits as eager launches.  The
    backward forks its query-side branch onto the library's second stream and joins it back with events; the
    capture has to record that fork and join as dependencies of the one graph (a step left outside it, or
    unjoined, would fail the capture or race with the replay)."""
    import retention_integration_b200 as prb

    Q, K, V, lg, dO = (x.to(cuda_device) for x in _case(1, 1024, 2, 2, 64, True, 1.0, seed=21))

    def step():
        q, k, v, g = (x.detach().clone().requires_grad_(True) for x in (Q, K, V, lg))
        O = prb.power_retention(q, k, v, g, deg=2, chunk_size=256)
        O.backward(dO)
        return O, q.grad, k.grad, v.grad, g.grad

    eager = [x.clone() for x in step()]  # also the library's first call: its second stream exists from here on
    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream(cuda_device).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for got, want in zip(captured, eager):
        assert torch.equal(got, want)


def test_gqa_equals_repeated_heads(cuda_device):
    """GQA == MHA with the kv heads repeated (perf/tests/gqa_tests.py:44-66)."""
    Q, K, V, lg, dO = _case(1, 512, 2, 4, 64, True, 2.0, seed=8)
    gq = _run_ours(cuda_device, Q, K, V, lg, dO, 128)
    Kr, Vr, lgr = K.repeat_interleave(4, 2), V.repeat_interleave(4, 2), lg.repeat_interleave(4, 2)
    mha = _run_ours(cuda_device, Q, Kr, Vr, lgr, dO, 128)
    assert rel_l2(gq["O"], mha["O"]) < 1e-3
    assert rel_l2(gq["dQ"], mha["dQ"]) < 5e-3
    assert rel_l2(gq["dK"], mha["dK"].view(1, 512, 2, 4, 64).sum(3)) < 1e-2
    assert rel_l2(gq["dV"], mha["dV"].view(1, 512, 2, 4, 64).sum(3)) < 1e-2


def test_full_benchmark_size_properties(cuda_device):
    """At b1 t65536 h8 d64 c1024 (too large for the oracle): no NaN, output invariant to the
    chunk size, and a 2048-token prefix agrees with the fp32 oracle (causality)."""
    import retention_integration_b200 as prb

    g = torch.Generator().manual_seed(0)
    b, t, h, d = 1, 65536, 8, 64
    Q, K, V = (torch.randn(b, t, h, d, generator=g).bfloat16().to(cuda_device) for _ in range(3))
    lg = F.logsigmoid(torch.randn(b, t, h, generator=g)).to(cuda_device)
    O1 = prb.power_retention(Q, K, V, lg, chunk_size=1024)
    O2 = prb.power_retention(Q, K, V, lg, chunk_size=512)
    torch.cuda.synchronize()
    assert torch.isfinite(O1).all()
    assert rel_l2(O1.float().cpu(), O2.float().cpu()) < 1e-2
    pre = slice(0, 2048)
    O_ref = oracle.power_retention(Q[:, pre, :2].float().cpu(), K[:, pre, :2].float().cpu(),
                                   V[:, pre, :2].float().cpu(), lg[:, pre, :2].cpu(), chunk_size=1024)
    assert rel_l2(O1[:, pre, :2].float().cpu(), O_ref) < TOL


def test_full_benchmark_size_is_bitwise_reproducible(cuda_device):
    """Five forward+backward runs at b1 t65536 h8 d64 give bit-identical results for chunk 1024 and 512.  Races
    between CTAs sharing an SM only show at grids of thousands of CTAs, far beyond the oracle-sized cases."""
    import retention_integration_b200 as prb

    g = torch.Generator().manual_seed(1)
    b, t, h, d = 1, 65536, 8, 64
    Q, K, V, dO = (torch.randn(b, t, h, d, generator=g).bfloat16().to(cuda_device) for _ in range(4))
    lg = F.logsigmoid(torch.randn(b, t, h, generator=g)).to(cuda_device)

    def run(c):
        leaves = [x.detach().requires_grad_(True) for x in (Q, K, V, lg)]
        O = prb.power_retention(*leaves, chunk_size=c)
        O.backward(dO)
        torch.cuda.synchronize()
        return [O.detach()] + [x.grad for x in leaves]

    for c in (1024, 512):
        ref = run(c)
        for _ in range(4):
            for name, x, r in zip(("O", "dQ", "dK", "dV", "dlog_G"), run(c), ref):
                assert torch.equal(x, r), (c, name)


def test_rejects_unsupported_arguments(cuda_device):
    import retention_integration_b200 as prb

    q = torch.zeros(1, 128, 1, 64, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(AssertionError):
        prb.power_retention(q, q, q, None, deg=3)            # odd degree: refused by the reference too
    with pytest.raises(prb.PRError):
        prb.power_retention(q, q, q, None, deg=4, chunk_size=64)  # states exist for deg 2 only, here and there
    with pytest.raises(prb.PRError):
        prb.power_retention(q.float(), q.float(), q.float(), None)  # 16-bit inputs only

"""The allocation-free decode entry point (pr_decode_step_static) against pr_decode_step.

For hosts that cannot allocate device memory while serving (a memory pool frozen after start-up,
an allocator owned by another component of the process) the library keeps the decode scratch in a
fixed device array.  This test calls both entry points through the C ABI on the same inputs, twice
in a row with different cache lengths (the second call finds the first call's leftovers in the
array), and wants the same bits: both run the same kernels, only the scratch differs.  The first
call is also compared with the CPU oracle.  The file is collected last and passes alone as well.
"""
import ctypes

import pytest
import torch
import torch.nn.functional as F

from oracle import power_retention_oracle as oracle
from tests._golden import rel_l2

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_matches_caller_scratch(cuda_device):
    from retention_integration_b200 import _lib
    from retention_integration_b200._lib import ptr, stream_ptr

    L = _lib.lib()
    g = torch.Generator().manual_seed(21)
    b, h, r, d, D = 3, 4, 2, 64, 2080
    hq = h * r
    state = (torch.randn(b, h, D, d, generator=g) * 0.1).bfloat16().to(cuda_device)
    sok = (torch.rand(b, h, D, generator=g) + 0.5).to(cuda_device)
    ns = L.pr_decode_nsplit()
    for tk in (37, 5):  # two calls in a row share the static array
        Q = torch.randn(b, 1, hq, d, generator=g).bfloat16().to(cuda_device)
        K = torch.randn(b, tk, h, d, generator=g).bfloat16().to(cuda_device)
        V = torch.randn(b, tk, h, d, generator=g).bfloat16().to(cuda_device)
        lg = F.logsigmoid(torch.randn(b, tk, h, generator=g) + 2.0).to(cuda_device)
        # existing entry point: the caller brings the scratch
        a = torch.empty(b, tk, h, device=cuda_device)
        py = torch.empty(b, hq, ns, d, device=cuda_device)
        pl = torch.empty(b, hq, ns, device=cuda_device)
        O_ref = torch.empty_like(Q)
        args = [ctypes.c_int(_lib.dtype_code(Q.dtype)), ctypes.c_int(b), ctypes.c_int(tk), ctypes.c_int(h),
                ctypes.c_int(hq), ctypes.c_int(d), ptr(Q), ptr(K), ptr(V), ptr(lg), ptr(state), ptr(sok),
                ctypes.c_float(0.125)]
        tail = [ctypes.c_int(0), stream_ptr(cuda_device)]
        _lib.check(L.pr_decode_step(*args, ptr(a), ptr(py), ptr(pl), ptr(O_ref), *tail), "pr_decode_step")
        # new entry point: no scratch arguments at all
        O = torch.empty_like(Q)
        _lib.check(L.pr_decode_step_static(*args, ptr(O), *tail), "pr_decode_step_static")
        torch.cuda.synchronize()
        assert torch.isfinite(O.float()).all()
        assert torch.equal(O, O_ref), tk  # same kernels, same inputs: only the scratch differs
        if tk == 37:
            from retention_integration_b200 import layout

            Y, _, _ = oracle.power_retention_inference(
                Q.float().cpu(), K.float().cpu(), V.float().cpu(), lg.cpu(),
                layout.to_reference_layout(state.float().cpu(), d),
                layout.to_reference_layout(sok.cpu(), d, dim=-1), deg=2, switch_over_seq_len=1024)
            assert rel_l2(O.float().cpu(), Y) < 1e-2  # the tolerance of the inference tests


def test_static_scratch_limits_are_refused(cuda_device):
    from retention_integration_b200 import _lib

    L = _lib.lib()
    rc = L.pr_decode_step_static(0, 2048, 1, 1, 1, 64, None, None, None, None, None, None, ctypes.c_float(1.0), None,
                                 0, None)
    assert rc == -1 and b"static scratch limit" in L.pr_last_error()
    rc = L.pr_decode_step_static(0, 129, 4, 1, 8, 64, None, None, None, None, None, None, ctypes.c_float(1.0),
                                 None, 0, None)
    assert rc == -1 and b"static scratch limit" in L.pr_last_error()

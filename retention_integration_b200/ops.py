"""Thin Python wrappers over the C ABI of libpr_b200.so.

Each function allocates its outputs with torch (device memory is torch's job here),
passes raw device pointers and the current stream, and raises PRError on a non-zero
status.  No function in this module computes anything itself.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong

import torch

from . import _lib
from ._lib import check, dtype_code, lib, ptr, stream_ptr


class LaunchLog:
    """Counts kernel launches and, when `timing` is on, brackets every launch with CUDA
    events on the launching stream (used by bench.py for the per-kernel breakdown)."""

    def __init__(self):
        self.count = 0
        self.timing = False
        self.events = []  # (name, start, end)

    def reset(self, timing: bool = False):
        self.count = 0
        self.timing = timing
        self.events = []

    def summary(self):
        """name -> (launches, total ms).  Synchronise before calling."""
        out = {}
        for name, s, e in self.events:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + s.elapsed_time(e))
        return out


launch_log = LaunchLog()

# kernels launched per entry point (for the launch count reported by bench.py)
_KERNELS_PER_CALL = {}


def _call(name: str, *args):
    fn = getattr(lib(), name)
    if launch_log.timing:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        rc = fn(*args)
        e.record()
        launch_log.events.append((name, s, e))
    else:
        rc = fn(*args)
    check(rc, name)
    launch_log.count += 1


def state_rows(d: int) -> int:
    """Rows of a chunk state: the reference package's expansion layout (2560 for d = 64)."""
    return 128 * (d // 16) * (d // 16 + 1)


def _dev(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise _lib.PRError("tensors must live on a CUDA device: there is no CPU path")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def selftest_umma(variant: int, a: torch.Tensor, b: torch.Tensor, n: int, k: int) -> torch.Tensor:
    out = torch.empty(128, n, device=a.device, dtype=torch.float32)
    _call("pr_selftest_umma", c_int(variant), c_int(dtype_code(a.dtype)), c_int(n), c_int(k), ptr(a), ptr(b),
                                 ptr(out), c_int(_dev(a)), stream_ptr(a.device))
    return out


def gate_prep(x: torch.Tensor, log_g, c: int, query_side: bool, mult: float = 1.0, want_gates: bool = True,
              row_scale=None, want_xt: bool = True, a_in=None):
    """x [b,t,hx,d], log_g [b,t,h] fp32 or None ->
    (a [b,t,h] fp32 or None, A [b,n,h] fp32, xT [b,n,hx,d,cp]) with cp = c rounded up to 64.
    With row_scale [b,t,hx] fp32 a fourth result is the copy of xT scaled per token."""
    b, t, hx, d = x.shape
    h = log_g.shape[2] if log_g is not None else hx
    n = t // c
    cp = (c + 63) // 64 * 64
    write = want_gates and not query_side
    if not want_xt and c > 16384:
        # one chunk longer than the chunk-local pass holds in shared memory: plain cumulative sum over the sequence
        if log_g is None:
            return None, None, None
        assert n == 1, "long chunks are only supported where the chunk is the whole sequence"
        a = torch.empty(b, t, h, device=x.device, dtype=torch.float32)
        _call("pr_gate_cumsum", c_int(b), c_int(t), c_int(h), ptr(log_g), c_longlong(t * h), ptr(a), c_int(_dev(x)),
              stream_ptr(x.device))
        return a, a[:, -1:, :].contiguous(), None
    a = torch.empty(b, t, h, device=x.device, dtype=torch.float32) if (write and log_g is not None) else None
    A = torch.empty(b, n, h, device=x.device, dtype=torch.float32) if write else None
    xt = torch.empty(b, n, hx, d, cp, device=x.device, dtype=x.dtype) if want_xt else None
    xts = torch.empty_like(xt) if (row_scale is not None and want_xt) else None
    # a_in: cumulative gates an earlier call has made (the backward reuses the forward's): read, not recomputed
    _call("pr_gate_prep", c_int(dtype_code(x.dtype)), c_int(b), c_int(t), c_int(h), c_int(hx), c_int(d), c_int(c),
                             ptr(log_g), ptr(x), ptr(a if a_in is None else a_in), ptr(A), ptr(xt), ptr(row_scale),
                             ptr(xts), c_int(1 if query_side else 0), c_float(mult),
                             c_int(1 if (write and a_in is None) else 0), c_int(_dev(x)), stream_ptr(x.device))
    if row_scale is not None:
        return a, A, xt, xts
    return a, A, xt


def dout_prep(O: torch.Tensor, dO: torch.Tensor, l: torch.Tensor):
    """O, dO [..., d] 16-bit, l [...] fp32 -> (dy = dO / l (16-bit), dl = -<O, dO> / l fp32)."""
    d = O.shape[-1]
    rows = O.numel() // d
    dy = torch.empty_like(O)
    dl = torch.empty_like(l)
    _call("pr_dout_prep", c_int(dtype_code(O.dtype)), c_longlong(rows), c_int(d), ptr(O), ptr(dO), ptr(l), ptr(dy),
                             ptr(dl), c_int(_dev(O)), stream_ptr(O.device))
    return dy, dl


def chunk_state(xt: torch.Tensor, xts, v: torch.Tensor, c: int, nh: int, key_weights: bool, want_gram: bool):
    """xt [b,n,hx,d,cp] (hx = nh*group), v [b,t,hx,d] -> (S [b,n,nh,DR,d], gram [b,n,nh,d,d] fp32 or None)."""
    b, n, hx, d, cp = xt.shape
    t = v.shape[1]
    group = hx // nh
    out = torch.empty(b, n, nh, state_rows(d), d, device=xt.device, dtype=xt.dtype)
    gram = torch.empty(b, n, nh, d, d, device=xt.device, dtype=torch.float32) if want_gram else None
    if want_gram and xts is None:
        xts = xt
    _call("pr_chunk_state", c_int(dtype_code(xt.dtype)), c_int(b), c_int(t), c_int(nh), c_int(group), c_int(d),
                               c_int(c), ptr(xt), ptr(xts), ptr(v), ptr(out), ptr(gram),
                               c_int(1 if key_weights else 0), c_int(_dev(xt)), stream_ptr(xt.device))
    return out, gram


def discumsum_fwd(X: torch.Tensor, A: torch.Tensor, inplace: bool = False, carry_in=None, want_carry: bool = False,
                  carry_only: bool = False):
    """X [b,n,h,...] 16-bit, A [b,n,h] fp32.  inplace: X becomes the states entering each chunk
    (n entries); otherwise returns Y [b,n+1,h,...] like the reference's discumsum.
    carry_only: nothing is written but the fp32 carry leaving the last chunk (returned alone)."""
    b, n, h = X.shape[:3]
    E = X[0, 0, 0].numel()
    n_out = n if (inplace or carry_only) else n + 1
    Y = None if carry_only else (X if inplace else torch.empty(b, n_out, *X.shape[2:], device=X.device, dtype=X.dtype))
    want_carry = want_carry or carry_only
    carry_out = torch.empty(b, h, E, device=X.device, dtype=torch.float32) if want_carry else None
    _call("pr_discumsum_fwd", c_int(dtype_code(X.dtype)), c_int(b), c_int(n), c_int(n_out), c_int(h),
                                 c_longlong(E), ptr(X), ptr(Y), ptr(A), ptr(carry_in), ptr(carry_out),
                                 c_int(_dev(X)), stream_ptr(X.device))
    if carry_only:
        return carry_out
    return (Y, carry_out) if want_carry else Y


def discumsum_bwd_carry(dY: torch.Tensor, A: torch.Tensor, carry_in=None):
    """Reverse scan reduced to its carry: G[0] for G[m] = dY[m] + exp(A[m]) G[m+1], G[n] = carry_in."""
    b, n, h = dY.shape[:3]
    E = dY[0, 0, 0].numel()
    carry_out = torch.empty(b, h, E, device=dY.device, dtype=torch.float32)
    _call("pr_discumsum_bwd", c_int(dtype_code(dY.dtype)), c_int(b), c_int(n), c_int(h), c_longlong(E), ptr(dY),
          ptr(None), ptr(None), ptr(A), ptr(carry_in), ptr(carry_out), ptr(None), c_int(0), c_int(0),
          c_int(_dev(dY)), stream_ptr(dY.device))
    return carry_out


def discumsum_bwd(dY: torch.Tensor, Y: torch.Tensor, A: torch.Tensor, row_len: int = 0, row_weights: bool = False,
                  inplace: bool = True, carry_in=None, want_carry: bool = False):
    """Reverse scan.  dY, Y [b,n,h,...].  Returns (dX, dA_part [b,h,blocks,n] fp32[, carry_out]):
    the chunk-gate gradient is left as per-block partial sums, which gate_grad() adds up."""
    b, n, h = dY.shape[:3]
    E = dY[0, 0, 0].numel()
    blocks = lib().pr_discumsum_bwd_blocks(c_longlong(E))
    dX = dY if inplace else torch.empty_like(dY)
    part = torch.empty(b, h, blocks, n, device=dY.device, dtype=torch.float32)
    carry_out = torch.empty(b, h, E, device=dY.device, dtype=torch.float32) if want_carry else None
    _call("pr_discumsum_bwd", c_int(dtype_code(dY.dtype)), c_int(b), c_int(n), c_int(h), c_longlong(E), ptr(dY),
                                 ptr(Y), ptr(dX), ptr(A), ptr(carry_in), ptr(carry_out), ptr(part), c_int(row_len),
                                 c_int(1 if row_weights else 0), c_int(_dev(dY)), stream_ptr(dY.device))
    return (dX, part, carry_out) if want_carry else (dX, part)


def gram_scan_fwd(G: torch.Tensor, A: torch.Tensor, dtype, want_full: bool, carry_in=None, want_carry=False):
    """G [b,n,h,d,d] fp32 -> (hi, lo [b,n,h,d,d] 16-bit, full fp32 or None): Gram matrices entering each chunk."""
    b, n, h, d, _ = G.shape
    hi = torch.empty(b, n, h, d, d, device=G.device, dtype=dtype)
    lo = torch.empty_like(hi)
    full = torch.empty_like(G) if want_full else None
    carry_out = torch.empty(b, h, d * d, device=G.device, dtype=torch.float32) if want_carry else None
    _call("pr_gram_scan_fwd", c_int(dtype_code(dtype)), c_int(b), c_int(n), c_int(h), c_int(d), ptr(G), ptr(hi),
                                 ptr(lo), ptr(full), ptr(A), ptr(carry_in), ptr(carry_out), c_int(_dev(G)),
                                 stream_ptr(G.device))
    return (hi, lo, full, carry_out) if want_carry else (hi, lo, full)


def gram_scan_bwd(dZg: torch.Tensor, Zg: torch.Tensor, A: torch.Tensor, dtype, carry_in=None, want_carry=False):
    """dZg, Zg [b,n,h,d,d] fp32 -> (hi, lo of the symmetrised d(gram_m), dA partial sums [b,h,blocks,n])."""
    b, n, h, d, _ = dZg.shape
    hi = torch.empty(b, n, h, d, d, device=dZg.device, dtype=dtype)
    lo = torch.empty_like(hi)
    blocks = lib().pr_gram_scan_bwd_blocks(c_int(d))
    part = torch.empty(b, h, blocks, n, device=dZg.device, dtype=torch.float32)
    carry_out = torch.empty(b, h, d * d, device=dZg.device, dtype=torch.float32) if want_carry else None
    _call("pr_gram_scan_bwd", c_int(dtype_code(dtype)), c_int(b), c_int(n), c_int(h), c_int(d), ptr(dZg), ptr(Zg),
                                 ptr(hi), ptr(lo), ptr(A), ptr(carry_in), ptr(carry_out), ptr(part), c_int(_dev(dZg)),
                                 stream_ptr(dZg.device))
    return (hi, lo, part, carry_out) if want_carry else (hi, lo, part)


def state_scan_fwd(S, gram, A, dtype, carry_in=None, gcarry_in=None, want_carry: bool = False):
    """discumsum_fwd (in place) + gram_scan_fwd (with the fp32 copy) in one launch.
    Returns (Z, zhi, zlo, zfull, carry_out or None, gram carry_out or None)."""
    b, n, h = S.shape[:3]
    d = gram.shape[-1]
    E = S[0, 0, 0].numel()
    hi = torch.empty(b, n, h, d, d, device=S.device, dtype=dtype)
    lo = torch.empty_like(hi)
    full = torch.empty_like(gram)
    co = torch.empty(b, h, E, device=S.device, dtype=torch.float32) if want_carry else None
    gco = torch.empty(b, h, d * d, device=S.device, dtype=torch.float32) if want_carry else None
    _call("pr_state_scan_fwd", c_int(dtype_code(S.dtype)), c_int(b), c_int(n), c_int(h), c_int(d), c_longlong(E),
          ptr(S), ptr(A), ptr(carry_in), ptr(co), ptr(gram), ptr(hi), ptr(lo), ptr(full), ptr(gcarry_in), ptr(gco),
          c_int(_dev(S)), stream_ptr(S.device))
    return S, hi, lo, full, co, gco


def state_scan_bwd(dZ, Z, dZg, zfull, A, dtype, carry_in=None, gcarry_in=None):
    """discumsum_bwd (in place, key weights on) + gram_scan_bwd in one launch.
    Returns (wdS, dA_state partial sums, ghi, glo, dA_gram partial sums)."""
    b, n, h = dZ.shape[:3]
    d = dZg.shape[-1]
    E = dZ[0, 0, 0].numel()
    blocks = lib().pr_discumsum_bwd_blocks(c_longlong(E))
    gblocks = lib().pr_gram_scan_bwd_blocks(c_int(d))
    part = torch.empty(b, h, blocks, n, device=dZ.device, dtype=torch.float32)
    gpart = torch.empty(b, h, gblocks, n, device=dZ.device, dtype=torch.float32)
    hi = torch.empty(b, n, h, d, d, device=dZ.device, dtype=dtype)
    lo = torch.empty_like(hi)
    _call("pr_state_scan_bwd", c_int(dtype_code(dZ.dtype)), c_int(b), c_int(n), c_int(h), c_int(d), c_longlong(E),
          ptr(dZ), ptr(Z), ptr(A), ptr(carry_in), ptr(None), ptr(part), ptr(dZg), ptr(zfull), ptr(hi), ptr(lo),
          ptr(gcarry_in), ptr(None), ptr(gpart), c_int(_dev(dZ)), stream_ptr(dZ.device))
    return dZ, part, hi, lo, gpart


def chunk_out(Q, K, V, a, Z, zg_hi, zg_lo, n_chunks: int, cq: int, ck: int, state_from_chunk: int, scale: float,
              normalize: bool = True, q_gate_last: bool = False, want_l: bool = True, deg: int = 2):
    """Fused attention + state read-out.  Q [b,n*cq,hq,d]; K,V [b,n*ck,h,d] or None; a [b,n*ck,h] or None;
    Z [b,n,h,DR,d] or None.  Returns (O [b,n*cq,hq,d], l [b,n*cq,hq] fp32 or None)."""
    b, tq, hq, d = Q.shape
    h = K.shape[2] if K is not None else Z.shape[2]
    O = torch.empty_like(Q)
    l = torch.empty(b, tq, hq, device=Q.device, dtype=torch.float32) if want_l else None
    _call("pr_chunk_out", c_int(dtype_code(Q.dtype)), c_int(b), c_int(n_chunks), c_int(cq), c_int(ck), c_int(hq),
                             c_int(h), c_int(d), ptr(Q), ptr(K), ptr(V), ptr(a), ptr(Z), ptr(zg_hi), ptr(zg_lo),
                             c_int(state_from_chunk), c_int(1 if q_gate_last else 0), c_int(1 if normalize else 0),
                             c_float(scale), c_int(deg), ptr(O), ptr(l), c_int(_dev(Q)), stream_ptr(Q.device))
    return O, l


def expand_grad(W, X, State, g_hi, g_lo, a, A, row_g, c: int, h: int, query_side: bool, scale: float,
                gram_mult: float, chunk_lo: int, chunk_hi: int):
    """Gradient through the expansion.  W, X [b,t,hx,d]; State [b,n,h,DR,d]; g_hi/g_lo [b,n,h,d,d].
    Returns (dX [b,t,hx,d] fp32, gdot [b,t,hx] fp32)."""
    b, t, hx, d = X.shape
    dX = torch.empty(b, t, hx, d, device=X.device, dtype=torch.float32)
    gdot = torch.empty(b, t, hx, device=X.device, dtype=torch.float32)
    _call("pr_expand_grad", c_int(dtype_code(X.dtype)), c_int(b), c_int(t), c_int(h), c_int(hx), c_int(d), c_int(c),
                               ptr(W), ptr(X), ptr(State), ptr(g_hi), ptr(g_lo), ptr(a), ptr(A), ptr(row_g),
                               c_int(1 if query_side else 0), c_float(scale), c_float(gram_mult), c_int(chunk_lo),
                               c_int(chunk_hi), ptr(dX), ptr(gdot), c_int(_dev(X)), stream_ptr(X.device))
    return dX, gdot


def chunk_dq(Q, dO, K, V, a, dl, l, dq_state, c: int, scale: float, deg: int = 2):
    """Returns (dQ [b,t,hq,d], da_q [b,t,hq] fp32)."""
    b, t, hq, d = Q.shape
    h = K.shape[2]
    dQ = torch.empty_like(Q)
    da_q = torch.empty(b, t, hq, device=Q.device, dtype=torch.float32)
    _call("pr_chunk_dq", c_int(dtype_code(Q.dtype)), c_int(b), c_int(t), c_int(hq), c_int(h), c_int(d), c_int(c),
                            ptr(Q), ptr(dO), ptr(K), ptr(V), ptr(a), ptr(dl), ptr(l), ptr(dq_state), c_float(scale),
                            c_int(deg), ptr(dQ), ptr(da_q), c_int(_dev(Q)), stream_ptr(Q.device))
    return dQ, da_q


def chunk_dkv(Q, dO, K, V, wdS, a, A, dl, l, dk_state, c: int, state_chunk_hi: int, scale: float, deg: int = 2):
    """Returns (dK, dV [b,t,h,d], da_k [b,t,h] fp32)."""
    b, t, hq, d = Q.shape
    h = K.shape[2]
    dK, dV = torch.empty_like(K), torch.empty_like(V)
    da_k = torch.empty(b, t, h, device=Q.device, dtype=torch.float32)
    _call("pr_chunk_dkv", c_int(dtype_code(Q.dtype)), c_int(b), c_int(t), c_int(hq), c_int(h), c_int(d), c_int(c),
                             ptr(Q), ptr(dO), ptr(K), ptr(V), ptr(wdS), ptr(a), ptr(A), ptr(dl), ptr(l), ptr(dk_state),
                             c_int(state_chunk_hi), c_float(scale), c_int(deg), ptr(dK), ptr(dV), ptr(da_k),
                             c_int(_dev(Q)), stream_ptr(Q.device))
    return dK, dV, da_k


def gate_grad(da_q, gq, da_k, wk, dA_scan, dA_gram, c: int):
    """Assembles dlog_G [b,t,h] from the per-token terms and the reverse scans' partial sums
    (dA_scan [b,h,blocks,n], dA_gram [b,h,blocks2,n])."""
    b, t, hq = da_q.shape
    h = da_k.shape[2]
    out = torch.empty(b, t, h, device=da_q.device, dtype=torch.float32)
    blocks = dA_scan.shape[2] if dA_scan is not None else 0
    gblocks = dA_gram.shape[2] if dA_gram is not None else 0
    _call("pr_gate_grad", c_int(b), c_int(t), c_int(h), c_int(hq), c_int(c), ptr(da_q), ptr(gq), ptr(da_k),
                             ptr(wk), ptr(dA_scan), c_int(blocks), ptr(dA_gram), c_int(gblocks), ptr(out), c_int(_dev(da_q)),
                             stream_ptr(da_q.device))
    return out


def decode_state(Q, state, sum_of_keys, a_last, scale: float):
    """Q [b,1,hq,d]; state [b,h,D,d]; sum_of_keys [b,h,D]; a_last [b,h] or None -> partial sums."""
    b, _, hq, d = Q.shape
    h = state.shape[1]
    ns = lib().pr_decode_nsplit()
    part_y = torch.empty(b, hq, ns, d, device=Q.device, dtype=torch.float32)
    part_l = torch.empty(b, hq, ns, device=Q.device, dtype=torch.float32)
    _call("pr_decode_state", c_int(dtype_code(Q.dtype)), c_int(b), c_int(h), c_int(hq), c_int(d), ptr(Q), ptr(state),
          ptr(sum_of_keys), ptr(a_last), c_float(scale), ptr(part_y), ptr(part_l), c_int(_dev(Q)),
          stream_ptr(Q.device))
    return part_y, part_l


def decode_finish(Q, K, V, a, scale: float, part_y, part_l, h: int):
    """Attention over the cached tokens + state partials -> O [b,1,hq,d]."""
    b, _, hq, d = Q.shape
    tk = K.shape[1] if K is not None else 0
    O = torch.empty_like(Q)
    _call("pr_decode_finish", c_int(dtype_code(Q.dtype)), c_int(b), c_int(tk), c_int(h), c_int(hq), c_int(d), ptr(Q),
          ptr(K), ptr(V), ptr(a), c_float(scale), ptr(part_y), ptr(part_l), ptr(O), c_int(_dev(Q)),
          stream_ptr(Q.device))
    return O


def state_merge(state, sum_of_keys, S, gram, a_last):
    """new_state = state*exp(a_last) + S (chunk-state -> exact layout); S [b,1,h,DR,d], gram [b,1,h,d,d]."""
    b, _, h, _, d = S.shape
    D = d * (d + 1) // 2
    new_state = torch.empty(b, h, D, d, device=S.device, dtype=S.dtype)
    new_sok = torch.empty(b, h, D, device=S.device, dtype=torch.float32)
    _call("pr_state_merge", c_int(dtype_code(S.dtype)), c_int(b), c_int(h), c_int(d), ptr(state), ptr(sum_of_keys),
          ptr(S), ptr(gram), ptr(a_last), ptr(new_state), ptr(new_sok), c_int(_dev(S)), stream_ptr(S.device))
    return new_state, new_sok


class _Problem(ctypes.Structure):
    _fields_ = [("dtype", c_int), ("b", c_int), ("t", c_int), ("h", c_int), ("hq", c_int), ("d", c_int), ("c", c_int),
                ("scale", c_float)]


def _problem(Q, h: int, c: int, scale: float) -> _Problem:
    b, t, hq, d = Q.shape
    return _Problem(dtype_code(Q.dtype), b, t, h, hq, d, c, scale)


def _workspace(prob: _Problem, what: int, dev) -> torch.Tensor:
    n = ctypes.c_size_t(0)
    check(lib().pr_workspace_bytes(ctypes.byref(prob), c_int(what), ctypes.byref(n)), "pr_workspace_bytes")
    return torch.empty(max(n.value, 16), device=dev, dtype=torch.uint8)


def retention_fwd(Q, K, V, log_G, c: int, scale: float, carry=None, want_final: bool = False):
    """The chunked forward in one library call.  Returns (O, saved workspace, final (state, gram) fp32 carries or
    (None, None))."""
    b, t, hq, d = Q.shape
    h = K.shape[2]
    prob = _problem(Q, h, c, scale)
    saved = _workspace(prob, 0, Q.device)
    scratch = _workspace(prob, 1, Q.device)
    O = torch.empty_like(Q)
    Cs, Cg = carry if carry is not None else (None, None)
    Fs = Fg = None
    if want_final:
        Fs = torch.empty(b, h, state_rows(d) * d, device=Q.device, dtype=torch.float32)
        Fg = torch.empty(b, h, d * d, device=Q.device, dtype=torch.float32)
    _call("pr_retention_fwd", ctypes.byref(prob), ptr(Q), ptr(K), ptr(V), ptr(log_G), ptr(Cs), ptr(Cg), ptr(O),
          ptr(saved), ptr(scratch), ptr(Fs), ptr(Fg), c_int(_dev(Q)), stream_ptr(Q.device))
    launch_log.count += 4  # five kernels behind one call
    return O, saved, Fs, Fg


def retention_bwd(Q, K, V, log_G, O, dO, saved, c: int, scale: float, had_carry: bool):
    """The chunked backward in one library call.  Returns (dQ, dK, dV, dlog_G or None)."""
    h = K.shape[2]
    prob = _problem(Q, h, c, scale)
    scratch = _workspace(prob, 2, Q.device)
    dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
    dG = torch.empty_like(log_G) if log_G is not None else None
    _call("pr_retention_bwd", ctypes.byref(prob), ptr(Q), ptr(K), ptr(V), ptr(log_G), ptr(O), ptr(dO),
          c_int(1 if had_carry else 0), ptr(saved), ptr(scratch), ptr(dQ), ptr(dK), ptr(dV), ptr(dG), c_int(_dev(Q)),
          stream_ptr(Q.device))
    launch_log.count += 10 if log_G is not None else 9  # eleven (ten ungated) kernels behind one call
    return dQ, dK, dV, dG


def state_to_chunk_layout(state, sum_of_keys, want16: bool = False, want32: bool = False, want_gram: bool = False,
                          want_gram_halves: bool = False):
    """Exact-layout (state [b,h,D,d], sum_of_keys [b,h,D]) -> dict with the requested forms in the kernels'
    chunk-state layout: "z16" [b,h,DR,d], "z32" fp32, "gram" [b,h,d,d] fp32, "ghi"/"glo" 16-bit."""
    b, h, _, d = state.shape
    dev, DR = state.device, state_rows(d)
    out = {
        "z16": torch.empty(b, h, DR, d, device=dev, dtype=state.dtype) if want16 else None,
        "z32": torch.empty(b, h, DR, d, device=dev, dtype=torch.float32) if want32 else None,
        "gram": torch.empty(b, h, d, d, device=dev, dtype=torch.float32) if want_gram else None,
        "ghi": torch.empty(b, h, d, d, device=dev, dtype=state.dtype) if want_gram_halves else None,
        "glo": torch.empty(b, h, d, d, device=dev, dtype=state.dtype) if want_gram_halves else None,
    }
    _call("pr_state_to_chunk_layout", c_int(dtype_code(state.dtype)), c_int(b), c_int(h), c_int(d), ptr(state),
          ptr(sum_of_keys), ptr(out["z16"]), ptr(out["z32"]), ptr(out["gram"]), ptr(out["ghi"]), ptr(out["glo"]),
          c_int(_dev(state)), stream_ptr(dev))
    return out


_decode_ws = {}


def _decode_partials(dev, b: int, h: int, hq: int, d: int):
    """Partial-sum workspace of a split decode step, or (None, None) when the step runs unsplit.  One
    workspace per (device, stream, shape): calls that may overlap on the GPU (other streams) get their own;
    calls on one stream are ordered and share it."""
    if lib().pr_decode_split(c_int(b), c_int(h), c_int(hq)) <= 1:
        return None, None
    key = (dev, torch.cuda.current_stream(dev).cuda_stream, b, hq, d)
    ws = _decode_ws.get(key)
    if ws is None:
        ns = lib().pr_decode_nsplit()
        ws = (torch.empty(b, hq, ns, d, device=dev, dtype=torch.float32),
              torch.empty(b, hq, ns, device=dev, dtype=torch.float32))
        _decode_ws[key] = ws
    return ws


def _batch_strided(t: torch.Tensor):
    """(tensor, batch stride in elements) with everything inside a batch entry dense.  A slice [:, :tk] of a
    longer preallocated cache qualifies as it is; anything else is copied."""
    if t is None:
        return None, 0
    if t.dim() >= 2:
        inner = 1
        dense = True
        for size, stride in zip(reversed(t.shape[1:]), reversed(t.stride()[1:])):
            if size != 1 and stride != inner:
                dense = False
                break
            inner *= size
        if dense and (t.shape[0] == 1 or t.stride(0) >= inner):
            return t, (t.stride(0) if t.shape[0] > 1 else inner)
    t = t.contiguous()
    return t, (t.stride(0) if t.dim() >= 1 else 0)


def decode_step(Q, K, V, log_g, state, sum_of_keys, scale: float, h: int):
    """One decode step (tq = 1) in a single library call and a single kernel.  Returns O [b,1,hq,d].  Q, K, V
    and log_g may be slices along the token axis of longer tensors (a preallocated cache): they are read in place.
    The partial-sum workspace a small problem needs is kept per (device, stream, shape), see _decode_partials."""
    b, _, hq, d = Q.shape
    tk = K.shape[1] if K is not None else 0
    Q, q_bs = _batch_strided(Q)
    if q_bs % 8 != 0 or Q.data_ptr() % 16:
        Q = Q.contiguous()
        q_bs = hq * d
    K, k_bs = _batch_strided(K)
    V, v_bs = _batch_strided(V)
    if K is not None and (k_bs != v_bs or k_bs % 8 != 0 or K.data_ptr() % 16 or V.data_ptr() % 16):
        K, V = K.contiguous(), V.contiguous()
        k_bs = v_bs = tk * h * d
    log_g, g_bs = _batch_strided(log_g)
    O = torch.empty(b, 1, hq, d, device=Q.device, dtype=Q.dtype)
    part_y, part_l = _decode_partials(Q.device, b, h, hq, d)
    _call("pr_decode_step_strided", c_int(dtype_code(Q.dtype)), c_int(b), c_int(tk), c_int(h), c_int(hq), c_int(d),
          ptr(Q), c_longlong(q_bs), ptr(K), ptr(V), c_longlong(k_bs), ptr(log_g), c_longlong(g_bs), ptr(state),
          ptr(sum_of_keys), c_float(scale), ptr(None), ptr(part_y), ptr(part_l), ptr(O), c_int(_dev(Q)),
          stream_ptr(Q.device))
    return O


def decode_recurrent(q, k, v, log_g, state, sum_of_keys, new_state, new_sum_of_keys, scale: float):
    """Pure-recurrent step: advances (state, sum_of_keys) by the token (k, v, log_g) into (new_state,
    new_sum_of_keys) - which may be the same tensors when hq / h <= 4 - and reads it with q.  Returns O [b,1,hq,d]."""
    b, _, hq, d = q.shape
    h = k.shape[2]
    q, q_bs = _batch_strided(q)
    k, k_bs = _batch_strided(k)
    v, v_bs = _batch_strided(v)
    if k_bs != v_bs:
        k, v = k.contiguous(), v.contiguous()
        k_bs = v_bs = h * d
    if q_bs % 8 != 0 or q.data_ptr() % 16:
        q, q_bs = q.contiguous(), hq * d
    log_g, g_bs = _batch_strided(log_g)
    O = torch.empty(b, 1, hq, d, device=q.device, dtype=q.dtype)
    part_y, part_l = _decode_partials(q.device, b, h, hq, d)
    _call("pr_decode_recurrent", c_int(dtype_code(q.dtype)), c_int(b), c_int(h), c_int(hq), c_int(d), ptr(q),
          c_longlong(q_bs), ptr(k), ptr(v), c_longlong(k_bs), ptr(log_g), c_longlong(g_bs), ptr(state),
          ptr(sum_of_keys), ptr(new_state), ptr(new_sum_of_keys), c_float(scale), ptr(part_y), ptr(part_l), ptr(O),
          c_int(_dev(q)), stream_ptr(q.device))
    return O


def caller_prep_fwd(qkvg, cos, sin, h: int, hq: int, d: int, gated: bool, gate_bias: float, half_split: bool):
    """qkvg [b,t,W] 16-bit (W a multiple of 8, W >= (hq+2h)d + h when gated); cos, sin [t,d/2] or [b,t,d/2] fp32
    -> Q [b,t,hq,d], K, V [b,t,h,d], log_g [b,t,h] fp32 or None (pr_caller_prep_fwd)."""
    b, t, W = qkvg.shape
    dev = qkvg.device
    Q = torch.empty(b, t, hq, d, device=dev, dtype=qkvg.dtype)
    K = torch.empty(b, t, h, d, device=dev, dtype=qkvg.dtype)
    V = torch.empty(b, t, h, d, device=dev, dtype=qkvg.dtype)
    log_g = torch.empty(b, t, h, device=dev, dtype=torch.float32) if gated else None
    bstride = 0 if cos.dim() == 2 else t * (d // 2)
    _call("pr_caller_prep_fwd", c_int(dtype_code(qkvg.dtype)), c_int(b), c_int(t), c_int(h), c_int(hq), c_int(d),
          ptr(qkvg), c_longlong(W), ptr(cos), ptr(sin), c_longlong(bstride), c_int(int(half_split)), c_int(int(gated)),
          c_float(gate_bias), ptr(Q), ptr(K), ptr(V), ptr(log_g), c_int(_dev(qkvg)), stream_ptr(dev))
    return Q, K, V, log_g


def caller_prep_bwd(qkvg, cos, sin, h: int, hq: int, d: int, gated: bool, gate_bias: float, half_split: bool, dQ, dK,
                    dV, dlog_g):
    """Gradient of caller_prep_fwd with respect to qkvg (same shape; columns past the used ones are zero)."""
    b, t, W = qkvg.shape
    used = (hq + 2 * h) * d + (h if gated else 0)
    out = torch.empty_like(qkvg) if W == used else torch.zeros_like(qkvg)
    bstride = 0 if cos.dim() == 2 else t * (d // 2)
    _call("pr_caller_prep_bwd", c_int(dtype_code(qkvg.dtype)), c_int(b), c_int(t), c_int(h), c_int(hq), c_int(d),
          ptr(qkvg), c_longlong(W), ptr(cos), ptr(sin), c_longlong(bstride), c_int(int(half_split)), c_int(int(gated)),
          c_float(gate_bias), ptr(dQ), ptr(dK), ptr(dV), ptr(dlog_g), ptr(out), c_int(_dev(qkvg)),
          stream_ptr(qkvg.device))
    return out

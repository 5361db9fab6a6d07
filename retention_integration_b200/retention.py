"""`power_retention` and `power_retention_inference` with the reference's signatures
(retention/power_retention_maker.py:72-73 and :287-288), running on libpr_b200.so.

The host side only validates arguments, pads, allocates and sequences kernel launches;
every arithmetic step of the path is a kernel of the C-ABI library.  There is no
PyTorch or CPU fallback: inputs must be CUDA tensors of dtype bfloat16 or float16.
"""
from __future__ import annotations

import math

import torch

from . import layout, ops
from ._lib import PRError

_SUPPORTED_D = (64,)

# True: forward and backward of the chunked branch are one library call each (the launch sequence runs in native
# code); False: the same kernels are launched one by one from Python (per-kernel timing, the sequence-parallel
# variant, debugging).  Both orders of launches are identical.
NATIVE_SEQUENCER = True


def _check_inputs(Q, K, V, log_G, deg, state_free=False):
    if deg != 2 and not (deg == 4 and state_free):
        raise PRError(f"deg={deg}: the state kernels implement deg=2 (as the reference's state operators do); "
                      "deg=4 runs on the state-free branch only (chunk_size=None or t <= switch_over_seq_len)")
    if not (Q.is_cuda and K.is_cuda and V.is_cuda):
        raise PRError("Q, K, V must be CUDA tensors: this package has no CPU path")
    assert Q.dtype == K.dtype == V.dtype, f"dtypes of inputs must match: {Q.dtype=}, {K.dtype=}, {V.dtype=}"
    if Q.dtype not in (torch.bfloat16, torch.float16):
        raise PRError(f"dtype {Q.dtype} unsupported: use bfloat16 or float16")
    b, t, hq, d = Q.shape
    h = K.shape[2]
    assert hq % h == 0, f"Q heads must be a multiple of KV heads: {hq=} {h=}"
    if d not in _SUPPORTED_D:
        raise PRError(f"head dim {d} unsupported by this build (supported: {_SUPPORTED_D})")
    if log_G is not None:
        assert log_G.shape == K.shape[:3], "log_G must be [batch, seq_len, kv_heads]"


class _ChunkedRetention(torch.autograd.Function):
    """Chunked forward/backward.  Sequence length is a multiple of the chunk size here.

    `carry` is None or (Cs [b,h,DR*d], Cg [b,h,d*d]) fp32: the state and Gram matrix entering the first
    chunk, in the kernels' chunk-state layout (initial_state).  With `want_final` the state and Gram matrix
    leaving the last chunk come back in the same form (not differentiable)."""

    @staticmethod
    def forward(ctx, Q, K, V, log_G, c, scale, carry, want_final):
        b, t, hq, d = Q.shape
        h = K.shape[2]
        n = t // c
        Cs, Cg = carry if carry is not None else (None, None)
        first = carry is None
        ctx.c, ctx.scale, ctx.first = c, scale, first
        ctx.native = NATIVE_SEQUENCER
        if ctx.native:
            O, saved, Fs, Fg = ops.retention_fwd(Q, K, V, log_G, c, scale, carry, want_final)
            ctx.save_for_backward(Q, K, V, log_G, O, saved)
            if want_final:
                ctx.mark_non_differentiable(Fs, Fg)
            return O, Fs, Fg
        a, A, KT = ops.gate_prep(K, log_G, c, query_side=False)
        S, gram = ops.chunk_state(KT, None, V, c, h, key_weights=True, want_gram=True)
        del KT
        Z, zhi, zlo, zfull, Fs, Fg = ops.state_scan_fwd(S, gram, A, Q.dtype, Cs, Cg, want_carry=want_final)
        O, l = ops.chunk_out(Q, K, V, a, Z, zhi, zlo, n, c, c, 1 if first else 0, scale)
        ctx.save_for_backward(Q, K, V, log_G, a, A, O, l, Z, zhi, zlo, zfull)
        if want_final:
            ctx.mark_non_differentiable(Fs, Fg)
        return O, Fs, Fg

    @staticmethod
    def backward(ctx, dO, _dFs=None, _dFg=None):
        c, scale = ctx.c, ctx.scale
        if ctx.native:
            Q, K, V, log_G, O, saved = ctx.saved_tensors
            dQ, dK, dV, dlog_G = ops.retention_bwd(Q, K, V, log_G, O, dO.contiguous(), saved, c, scale, not ctx.first)
            return dQ, dK, dV, dlog_G, None, None, None, None
        Q, K, V, log_G, a, A, O, l, Z, zhi, zlo, zfull = ctx.saved_tensors
        b, t, hq, d = Q.shape
        h = K.shape[2]
        n = t // c
        dO = dO.contiguous()
        dy, dl = ops.dout_prep(O, dO, l)
        # state read-out: dZ_m = sum_i phi(q~_i) dy_i^T, dZg_m = sum_i dl_i q~_i q~_i^T
        _, _, QT, QTs = ops.gate_prep(Q, log_G, c, query_side=True, mult=scale, row_scale=dl, a_in=a)
        dZ, dZg = ops.chunk_state(QT, QTs, dy, c, h, key_weights=False, want_gram=True)
        del QT, QTs
        # reverse scans: dS_m (with key weights folded in) and the chunk-gate gradient
        wdS, dA_state, ghi, glo, dA_gram = ops.state_scan_bwd(dZ, Z, dZg, zfull, A, Q.dtype)
        # gradients through the expansions (chunk 0 reads a state only when one was carried in)
        gate_A = A if a is not None else None
        dq_state, gq = ops.expand_grad(dy, Q, Z, zhi, zlo, a, gate_A, dl, c, h, True, scale, 2.0,
                                       1 if ctx.first else 0, n - 1)
        dk_state, wk = ops.expand_grad(V, K, wdS, ghi, glo, a, gate_A, None, c, h, False, 1.0, 1.0, 0, n - 2)
        # intra-chunk attention backward, merged with the state-path terms
        dQ, da_q = ops.chunk_dq(Q, dO, K, V, a, dl, l, dq_state, c, scale)
        dK, dV, da_k = ops.chunk_dkv(Q, dO, K, V, wdS, a, gate_A, dl, l, dk_state, c, n - 2, scale)
        dlog_G = None
        if log_G is not None:
            dlog_G = ops.gate_grad(da_q, gq, da_k, wk, dA_state, dA_gram, c)
        return dQ, dK, dV, dlog_G, None, None, None, None


class _QuadraticRetention(torch.autograd.Function):
    """Whole-sequence causal power attention (no state): the branch the reference takes for
    t <= switch_over_seq_len (retention/power_retention_maker.py:128-132)."""

    @staticmethod
    def forward(ctx, Q, K, V, log_G, scale, deg):
        t = Q.shape[1]
        a = None
        if log_G is not None:
            a, _, _ = ops.gate_prep(K, log_G, t, query_side=False, want_xt=False)
        O, l = ops.chunk_out(Q, K, V, a, None, None, None, 1, t, t, 1, scale, deg=deg)
        ctx.save_for_backward(Q, K, V, a, O, l)
        ctx.scale, ctx.deg = scale, deg
        ctx.gated = log_G is not None
        return O

    @staticmethod
    def backward(ctx, dO):
        Q, K, V, a, O, l = ctx.saved_tensors
        t = Q.shape[1]
        dO = dO.contiguous()
        _, dl = ops.dout_prep(O, dO, l)
        dQ, da_q = ops.chunk_dq(Q, dO, K, V, a, dl, l, None, t, ctx.scale, deg=ctx.deg)
        dK, dV, da_k = ops.chunk_dkv(Q, dO, K, V, None, a, None, dl, l, None, t, -1, ctx.scale, deg=ctx.deg)
        dlog_G = ops.gate_grad(da_q, None, da_k, None, None, None, t) if ctx.gated else None
        return dQ, dK, dV, dlog_G, None, None


def _pad_head_dim(x, d_to):
    return torch.nn.functional.pad(x, (0, d_to - x.shape[-1]))


# `chunk_size` blocks the computation; the result does not depend on it (the reference pads, chunks and scans
# to the same function for every chunk size, and so do the kernels here - tested).  Small chunks are slow on
# this hardware for a reason the arithmetic does not care about: every chunk's state (2560 x 64 per head) is written,
# scanned and read again, 1.3 GB per pass at chunk 128 against 0.17 GB at chunk 1024 for the benchmark's shape
# (5.3 vs 2.6 ms per step).  With AUTO_CHUNK the Python API therefore runs a request for a chunk below 1024 with the
# largest multiple of it that is at most 1024 and pads the sequence by at most 1/16 more than the request would
# (padding tokens are zero keys and values behind gates of 1: they change neither the outputs of the real tokens nor
# the state after the last one).  The C ABI (pr_retention_fwd) always takes the chunk it is given.
AUTO_CHUNK = True
_FAST_CHUNK = 1024


def effective_chunk(t: int, chunk_size, deg: int = 2):
    """The chunk size power_retention runs with for a sequence of t tokens and a requested chunk_size.

    Below 1024: the largest multiple of the request up to 1024 that pads by at most 1/16 more.  Above 1024 (slower
    again: the intra-chunk attention grows with the chunk): the largest divisor of the request in [256, 1024], which
    leaves the padded length as it is.  None (no chunking) on a long sequence: 1024 or 512 if that pads by at most
    1/16; the quadratic form otherwise.  deg 4 forms no states and is never chunked."""
    if not AUTO_CHUNK or deg != 2:
        return chunk_size
    if chunk_size is None:
        if t <= 2 * _FAST_CHUNK:
            return None
        for ce in (_FAST_CHUNK, _FAST_CHUNK // 2):
            if -(-t // ce) * ce <= t + t // 16:
                return ce
        return None
    if chunk_size > _FAST_CHUNK:
        for ce in range(_FAST_CHUNK, 255, -1):
            if chunk_size % ce == 0:
                return ce
        return chunk_size
    if chunk_size == _FAST_CHUNK:
        return chunk_size
    padded = -(-t // chunk_size) * chunk_size  # what the request itself pads to
    for m in range(_FAST_CHUNK // chunk_size, 1, -1):
        ce = m * chunk_size
        if -(-t // ce) * ce <= padded + padded // 16:
            return ce
    return chunk_size


def power_retention(Q, K, V, log_G=None, initial_state=None, return_final_state=False, deg=2, scale=None,
                    chunk_size=None, switch_over_seq_len=None):
    """Symmetric power retention, training forward (differentiable).

    Same arguments as the reference (retention/power_retention_maker.py:72-73):
    Q [b,t,hq,d]; K, V [b,t,h,d]; log_G [b,t,h] float32 or None; returns [b,t,hq,d].

    `initial_state` / `return_final_state` (retention/power_retention_maker.py:131-140,158-172, left
    unfinished there: the state is passed without its normaliser and the returned one is the state
    *entering* the last chunk) are finished here: the state is the pair (state [b,h,D,d], sum_of_keys [b,h,D]
    fp32) in the exact layout, exactly what power_retention_inference takes and returns; the sequence
    continues from it, and with return_final_state the call returns (out, (state, sum_of_keys)) after the
    last token.  Gradients flow to Q, K, V and log_G; the states are treated as constants.

    Head dims 16, 32 and 48 run on the d = 64 kernels with zero-padded features (exact: the padded
    features contribute nothing to any dot product); they take no states.
    """
    assert deg % 2 == 0, f"deg must be even: {deg=}"
    d_orig = Q.shape[-1]
    if d_orig in (16, 32, 48):
        if initial_state is not None or return_final_state:
            raise PRError(f"states are kept for head dim 64 only (got {d_orig})")
        if not scale:
            scale = 1.0 / math.sqrt(d_orig)
        out = power_retention(_pad_head_dim(Q, 64), _pad_head_dim(K, 64), _pad_head_dim(V, 64), log_G, None, False,
                              deg, scale, chunk_size, switch_over_seq_len)
        return out[..., :d_orig]
    b, t, hq, d = Q.shape
    h = K.shape[2]
    requested = chunk_size
    chunk_size = effective_chunk(t, chunk_size, deg)
    if chunk_size != requested:
        # the blocking is this function's own choice: one chunk is the quadratic form, several the chunked one
        switch_over_seq_len = chunk_size
    elif chunk_size is not None and switch_over_seq_len is None:
        switch_over_seq_len = chunk_size
    t_padded = t if chunk_size is None else -(-t // chunk_size) * chunk_size
    state_free = (switch_over_seq_len is None or t_padded <= switch_over_seq_len or chunk_size is None) and \
        initial_state is None and not return_final_state
    _check_inputs(Q, K, V, log_G, deg, state_free)
    if log_G is not None:
        log_G = log_G.to(torch.float32).contiguous()
    if not scale:
        scale = 1.0 / math.sqrt(d)
    t_pad = 0
    if chunk_size is not None and t % chunk_size != 0:
        # pad with zero tokens whose gate is 1, as the reference does (:75-83)
        t_pad = chunk_size - t % chunk_size
        Q = torch.nn.functional.pad(Q, (0, 0, 0, 0, 0, t_pad))
        K = torch.nn.functional.pad(K, (0, 0, 0, 0, 0, t_pad))
        V = torch.nn.functional.pad(V, (0, 0, 0, 0, 0, t_pad))
        if log_G is not None:
            log_G = torch.nn.functional.pad(log_G, (0, 0, 0, t_pad))
    Q, K, V = Q.contiguous(), K.contiguous(), V.contiguous()
    tt = t + t_pad
    quadratic = switch_over_seq_len is None or tt <= switch_over_seq_len or chunk_size is None
    with_state = initial_state is not None or return_final_state
    if quadratic and not with_state:
        out = _QuadraticRetention.apply(Q, K, V, log_G, float(scale), int(deg))
        return out[:, :t] if t_pad else out
    carry = None
    if initial_state is not None:
        state, sok = initial_state
        D = layout.exact_dim(d)
        assert state.shape == (b, h, D, d), f"state must be [b,h,{D},{d}] (exact layout)"
        assert sok.shape == (b, h, D) and sok.dtype == torch.float32
        conv = ops.state_to_chunk_layout(state.to(Q.dtype).contiguous(), sok.contiguous(), want32=True, want_gram=True)
        carry = (conv["z32"].view(b, h, -1), conv["gram"].view(b, h, -1))
    # a short sequence that carries a state is one chunk of the chunked form (same arithmetic as the quadratic branch)
    c = tt if quadratic else int(chunk_size)
    out, Fs, Fg = _ChunkedRetention.apply(Q, K, V, log_G, c, float(scale), carry, bool(return_final_state))
    out = out[:, :t] if t_pad else out
    if not return_final_state:
        return out
    DR = ops.state_rows(d)
    final = ops.state_merge(None, None, Fs.to(Q.dtype).view(b, 1, h, DR, d), Fg.view(b, 1, h, d, d), None)
    return out, final


def power_retention_inference(Q, K, V, log_G=None, initial_state=None, sum_of_keys=None, deg=2, scale=None,
                              switch_over_seq_len=512):
    """Decode / prefill-to-state step with the reference's signature and semantics
    (retention/power_retention_maker.py:287-390, the variant with an explicit sum_of_keys).

    Q [b,tq,hq,d]; K, V [b,tk,h,d] or None (the tokens cached since the last switch-over);
    log_G [b,tk,h] or None; initial_state [b,h,D,d], sum_of_keys [b,h,D] fp32 or None.
    Returns (Y [b,tq,hq,d], state, sum_of_keys); when tk >= switch_over_seq_len the cache is
    compressed into a new state, otherwise the very same state objects come back.

    States use the exact expansion layout, D = d*(d+1)/2 (2080 at d = 64); the reference's
    padded layout (2560) converts with layout.to_reference_layout / from_reference_layout.
    """
    has_cache = K is not None and V is not None
    assert has_cache or initial_state is not None, "initial_state or cache must be provided for inference"
    assert (initial_state is None) == (sum_of_keys is None), "initial_state and sum_of_keys come together"
    if deg != 2:
        raise PRError(f"deg={deg}: the state kernels implement deg=2")
    if not Q.is_cuda:
        raise PRError("tensors must be CUDA tensors: this package has no CPU path")
    b, tq, hq, d = Q.shape
    if d not in _SUPPORTED_D:
        raise PRError(f"head dim {d} unsupported by this build (supported: {_SUPPORTED_D})")
    if has_cache:
        assert Q.dtype == K.dtype == V.dtype, "dtypes of inputs must match"
        assert K.shape[1] == V.shape[1], "key and value must have the same seq_len"
        tk, h = K.shape[1], K.shape[2]
    else:
        tk, h = 0, initial_state.shape[1]
    assert hq % h == 0
    if initial_state is not None:
        D = layout.exact_dim(d)
        assert initial_state.shape == (b, h, D, d), f"state must be [b,h,{D},{d}] (exact layout)"
        assert sum_of_keys.shape == (b, h, D) and sum_of_keys.dtype == torch.float32
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    gated = has_cache and log_G is not None
    if gated:
        assert log_G.shape == K.shape[:3]
        log_G = log_G.to(torch.float32)
    switch = switch_over_seq_len is not None and tk >= switch_over_seq_len
    decode = tq == 1 and initial_state is not None
    if not decode or switch:
        # every path but the plain decode step wants dense tensors; the decode step reads a query and a cache
        # that are slices of longer preallocated tensors in place
        Q = Q.contiguous()
        if has_cache:
            K, V = K.contiguous(), V.contiguous()
        if gated:
            log_G = log_G.contiguous()

    # ---- read-out
    a = None
    if decode:
        # the decode step proper: one library call (gate cumsum, state read, cache attention)
        Y = ops.decode_step(Q, K if tk > 0 else None, V if tk > 0 else None, log_G if gated else None,
                            initial_state.contiguous(), sum_of_keys.contiguous(), scale, h)
    else:
        if gated:
            a, _, _ = ops.gate_prep(K, log_G, tk, query_side=False, want_xt=False)
        if initial_state is None:
            Y, _ = ops.chunk_out(Q, K, V, a, None, None, None, 1, tq, tk, 1, scale, want_l=False)
        else:
            # several query tokens against a state: the tensor-core path, state converted to its layout
            conv = ops.state_to_chunk_layout(initial_state.contiguous(), sum_of_keys.contiguous(), want16=True,
                                             want_gram_halves=True)
            Z, zhi, zlo = conv["z16"].unsqueeze(1), conv["ghi"].unsqueeze(1), conv["glo"].unsqueeze(1)
            if tk > 0:
                Y, _ = ops.chunk_out(Q, K, V, a, Z, zhi, zlo, 1, tq, tk, 0, scale, q_gate_last=True, want_l=False)
            else:
                Y, _ = ops.chunk_out(Q, None, None, None, Z, zhi, zlo, 1, tq, tq, 0, scale, want_l=False)

    # ---- optionally compress the cache into the state
    if switch:
        a2, _, KT = ops.gate_prep(K, log_G if gated else None, tk, query_side=False)
        a_last = a2[:, -1, :].contiguous() if a2 is not None else None
        S, gram = ops.chunk_state(KT, None, V, tk, h, key_weights=True, want_gram=True)
        new_state, new_sok = ops.state_merge(initial_state, sum_of_keys, S, gram, a_last)
        return Y, new_state, new_sok
    return Y, initial_state, sum_of_keys

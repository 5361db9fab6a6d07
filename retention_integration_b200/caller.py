"""The glue between a model's projection and the operator, as the reference's callers write it
(deploy/nanoGPT/model.py:66-84; deploy/models/powercoder/modeling_powercoder.py:152-159), in one
kernel each way: split of the projection output, gate `logsigmoid(bias + proj)` in fp32, rotary on
queries and keys, and the contiguous `[b,t,h,d]` tensors `power_retention` takes.

    qkvg = c_attn(x)                                            # [b, t, (hq+2h)d + h]
    sin, cos = rotary_tables(t, d, x.device)                    # once per sequence length
    q, k, v, log_g = prepare_qkvg(qkvg, sin, cos, h, hq, d)     # one kernel; autograd gives dqkvg
    y = power_retention(q, k, v, log_g, deg=2, chunk_size=c)

No fallback: CUDA 16-bit tensors only; anything else raises PRError.
"""
from __future__ import annotations

import math

import torch

from . import ops
from ._lib import PRError

__all__ = ["rotary_tables", "prepare_qkvg", "GATE_BIAS"]

GATE_BIAS = 6.906768  # logsigmoid(GATE_BIAS) = log 0.999: the callers' initial gate (model.py:75-76)


def rotary_tables(t: int, d: int, device):
    """sin, cos [t, d/2] fp32 as deploy/nanoGPT/model.py:143-151 builds them for positions 0..t-1 (the
    wavelengths depend on the sequence length itself, :79-80).  Half-split callers pass the first half of their
    own cos / sin instead (modeling_powercoder.py:159: the two halves of those tables are equal)."""
    pos = torch.arange(t, dtype=torch.float32, device=device).unsqueeze(-1)
    div = (2.0 * math.pi) / (float(t) ** (torch.arange(0, d, 2, dtype=torch.float32, device=device) / d))
    ang = pos * div.view(1, -1)
    return torch.sin(ang), torch.cos(ang)


class _PrepareQKVG(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkvg, sin, cos, h, hq, d, gated, gate_bias, half_split):
        Q, K, V, log_g = ops.caller_prep_fwd(qkvg, cos, sin, h, hq, d, gated, gate_bias, half_split)
        ctx.save_for_backward(qkvg, sin, cos)
        ctx.cfg = (h, hq, d, gated, gate_bias, half_split)
        return (Q, K, V, log_g) if gated else (Q, K, V)

    @staticmethod
    def backward(ctx, dQ, dK, dV, dlog_g=None):
        qkvg, sin, cos = ctx.saved_tensors
        h, hq, d, gated, gate_bias, half_split = ctx.cfg
        dQ, dK, dV = (x.contiguous() for x in (dQ, dK, dV))
        if gated:
            dlog_g = torch.zeros(dQ.shape[0], dQ.shape[1], h, device=dQ.device) if dlog_g is None else dlog_g.float().contiguous()
        dqkvg = ops.caller_prep_bwd(qkvg, cos, sin, h, hq, d, gated, gate_bias, half_split, dQ, dK, dV, dlog_g)
        return dqkvg, None, None, None, None, None, None, None, None


def prepare_qkvg(qkvg, sin, cos, h: int, hq: int, d: int, gated: bool = True, gate_bias: float = GATE_BIAS,
                 half_split: bool = False):
    """qkvg [b, t, W]: a token's row holds hq*d query, h*d key, h*d value features and (gated) h gate
    pre-activations, as `c_attn` of deploy/nanoGPT/model.py:66 lays them out.  sin, cos [t, d/2] or [b, t, d/2]
    fp32.  Returns Q [b,t,hq,d], K, V [b,t,h,d] with the rotary applied to Q and K, and log_g [b,t,h] fp32
    (None when not gated).  `half_split`: pairs (i, i + d/2) instead of (2i, 2i+1).

    W must be a multiple of 8 for 16-byte rows; a narrower projection (W = (hq+2h)d + h with h not a multiple
    of 8) is padded here with one extra copy - size `c_attn`'s out_features to a multiple of 8 to avoid it."""
    if not (qkvg.is_cuda and qkvg.dtype in (torch.bfloat16, torch.float16) and qkvg.dim() == 3):
        raise PRError("prepare_qkvg wants a CUDA bf16/fp16 tensor [b, t, W]")
    used = (hq + 2 * h) * d + (h if gated else 0)
    if qkvg.shape[-1] < used:
        raise PRError(f"a row of {qkvg.shape[-1]} elements cannot hold {used}")
    if d % 8 or (half_split and d % 16):
        raise PRError(f"head dim {d}: a multiple of 8 (16 for half-split pairs)")
    if qkvg.shape[-1] % 8 or not qkvg.is_contiguous() or qkvg.data_ptr() % 16:
        pad = (-qkvg.shape[-1]) % 8
        qkvg = torch.nn.functional.pad(qkvg, (0, pad)).contiguous()  # differentiable: the gradient is cut back
    sin, cos = sin.float().contiguous(), cos.float().contiguous()
    t = qkvg.shape[1]
    if sin.shape[-2:] != (t, d // 2) or cos.shape != sin.shape:
        raise PRError(f"sin / cos must be [t, d/2] = [{t}, {d // 2}] (or [b, t, d/2]), got {tuple(sin.shape)}")
    out = _PrepareQKVG.apply(qkvg, sin, cos, h, hq, d, gated, float(gate_bias), bool(half_split))
    return (*out, None) if not gated else out

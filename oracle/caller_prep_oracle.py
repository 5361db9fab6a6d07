"""CPU oracle for the callers' glue between the projection and the operator.  TEST INFRASTRUCTURE,
NOT A PRODUCT PATH: only `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU legs may import it.

A restatement in plain PyTorch CPU ops of what the reference's two callers do to the output of
their projection before they call `power_retention`:

  * `deploy/nanoGPT/model.py:66-84` - split of `qkvg`, `log_g = logsigmoid(6.906768 + gate.float())`,
    sinusoidal tables (`:143-151`) and the interleaved-pair rotary (`:153-164`);
  * `deploy/models/powercoder/modeling_powercoder.py:152-159` - separate projections,
    `logsigmoid(gate.float())`, and the half-split rotary of `:43-74`.

Parity status: the interleaved form is PINNED by `tests/golden/caller_prep_nanogpt.npz`, which
`tests/golden/make_golden.py` produces with the reference's own `get_sinusoidal_embeddings` and
`apply_rotary_position_embeddings`.  The half-split form is UNPINNED (its module needs the
transformers model scaffolding to import); it differs from the pinned one in which elements pair up.

Gradients are autograd's, as in the reference.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

__all__ = ["sinusoidal_tables", "rotary", "caller_prep"]


def sinusoidal_tables(t: int, d: int):
    """sin, cos [t, d/2] fp32 for positions 0..t-1 (deploy/nanoGPT/model.py:143-151, with the position
    tensor of :79: the wavelengths depend on the sequence length itself)."""
    pos = torch.arange(t, dtype=torch.float32).unsqueeze(-1)
    div = (2.0 * math.pi) / (float(t) ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = pos * div.view(1, -1)
    return torch.sin(ang), torch.cos(ang)


def rotary(x, sin, cos, half_split: bool):
    """x [b,t,heads,d]; sin, cos [t, d/2] (or [b,t,d/2]).  Interleaved pairs: model.py:153-164;
    half-split: modeling_powercoder.py:43-74.  Computed in fp32, cast to x.dtype."""
    if sin.dim() == 2:
        sin, cos = sin.unsqueeze(0), cos.unsqueeze(0)
    sin, cos = sin.unsqueeze(2), cos.unsqueeze(2)  # [b|1, t, 1, d/2]
    if half_split:
        s, c = torch.cat((sin, sin), -1), torch.cat((cos, cos), -1)
        h = x.shape[-1] // 2
        rot = torch.cat((-x[..., h:], x[..., :h]), -1)
    else:
        s, c = sin.repeat_interleave(2, dim=3), cos.repeat_interleave(2, dim=3)
        rot = torch.stack((-x[..., 1::2], x[..., ::2]), -1).reshape(x.shape)
    return ((x * c) + (rot * s)).to(x.dtype)


def caller_prep(qkvg, sin, cos, h: int, hq: int, d: int, gated: bool = True, gate_bias: float = 6.906768,
                half_split: bool = False):
    """qkvg [b,t,(hq+2h)d (+h)] -> Q [b,t,hq,d], K, V [b,t,h,d], log_g [b,t,h] fp32 or None."""
    b, t, _ = qkvg.shape
    q, k, v = qkvg[..., : (hq + 2 * h) * d].split([hq * d, h * d, h * d], dim=2)
    q, k, v = q.reshape(b, t, hq, d), k.reshape(b, t, h, d), v.reshape(b, t, h, d)
    log_g = None
    if gated:
        log_g = F.logsigmoid(gate_bias + qkvg[..., (hq + 2 * h) * d : (hq + 2 * h) * d + h].to(torch.float32))
    return rotary(q, sin, cos, half_split), rotary(k, sin, cos, half_split), v.contiguous(), log_g

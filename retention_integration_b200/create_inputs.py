"""Seeded sample inputs and shape/dtype contracts of the two public operators.

These restate the contracts of the reference's retention/create_inputs.py:10-86 so that tests
written against that module (its perf/tests/common_tests.py:24-62 checks shapes, dtypes and
devices of inputs, outputs and gradients from exactly these tables) run against this package:
same argument names, same defaults, same value distributions (`randn / sqrt(d)`, training
gates `logsigmoid(randn)`, inference gates `logsigmoid(6.906768 + randn)`, seed 42, scale 1.0).

One deliberate difference: inference states use the exact expansion layout
(D = d (d + 1) / 2 rows, see layout.py), and the normaliser is always passed explicitly as
`sum_of_keys`; the reference's `fused_normalizer=True` form (normaliser folded into a padded
state, a vidrial-backend convention) has no counterpart here and is refused.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import layout

INFERENCE_GATE_BIAS = 6.906768  # the reference's bias for slowly decaying inference gates (:39)


def _grad_leaf(x, requires_grad):
    if x is None or not requires_grad:
        return x
    return x.clone().detach().requires_grad_(True)


def create_inputs(b=2, t=1024, h=8, d=32, qhead_ratio=1, dtype=torch.bfloat16, device="cuda", gating=False,
                  chunk_size=None, deg=2, requires_grad=False, seed=42, scale=1.0, switch_over_seq_len=None):
    """Keyword arguments for `power_retention` (retention/create_inputs.py:10-32)."""
    torch.manual_seed(seed)
    inv = 1.0 / math.sqrt(d)
    Q = torch.randn(b, t, h * qhead_ratio, d, dtype=dtype, device=device) * inv
    K = torch.randn(b, t, h, d, dtype=dtype, device=device) * inv
    V = torch.randn(b, t, h, d, dtype=dtype, device=device) * inv
    log_G = F.logsigmoid(torch.randn(b, t, h, dtype=torch.float32, device=device)) if gating else None
    Q, K, V, log_G = (_grad_leaf(x, requires_grad) for x in (Q, K, V, log_G))
    return dict(Q=Q, K=K, V=V, log_G=log_G, initial_state=None, return_final_state=False, deg=deg, scale=scale,
                chunk_size=chunk_size, switch_over_seq_len=switch_over_seq_len)


def create_inference_inputs(b=2, tq=1, tk=1024, h=8, d=32, qhead_ratio=1, dtype=torch.bfloat16, device="cuda",
                            gating=False, chunk_size=None, deg=2, requires_grad=False, seed=42, scale=1.0,
                            initial_state=False, switch_over_seq_len=512, fused_normalizer=False):
    """Keyword arguments for `power_retention_inference` (retention/create_inputs.py:34-58)."""
    if fused_normalizer:
        raise ValueError("fused_normalizer=True is a convention of the reference's vidrial backend; "
                         "this package always takes sum_of_keys explicitly")
    assert tk > 0 or initial_state, "tk must be greater than 0 or initial_state must be True"
    torch.manual_seed(seed)
    inv = 1.0 / math.sqrt(d)
    Q = torch.randn(b, tq, h * qhead_ratio, d, dtype=dtype, device=device) * inv
    K = torch.randn(b, tk, h, d, dtype=dtype, device=device) * inv if tk > 0 else None
    V = torch.randn(b, tk, h, d, dtype=dtype, device=device) * inv if tk > 0 else None
    log_G = None
    if gating and tk > 0:
        log_G = F.logsigmoid(INFERENCE_GATE_BIAS + torch.randn(b, tk, h, dtype=torch.float32, device=device))
    D = layout.exact_dim(d)
    state = torch.randn(b, h, D, d, dtype=dtype, device=device) if initial_state else None
    sok = torch.randn(b, h, D, dtype=torch.float32, device=device).abs() if initial_state else None
    Q, K, V, log_G, state, sok = (_grad_leaf(x, requires_grad) for x in (Q, K, V, log_G, state, sok))
    return dict(Q=Q, K=K, V=V, log_G=log_G, initial_state=state, sum_of_keys=sok, deg=deg, scale=scale,
                switch_over_seq_len=switch_over_seq_len)


def input_properties(b=2, t=1024, h=8, d=32, qhead_ratio=1, dtype=torch.float16, device="cuda", gating=False,
                     **_unused):
    """name -> (shape, dtype, device) of the tensor inputs of `power_retention` (:60-65)."""
    props = dict(Q=((b, t, h * qhead_ratio, d), dtype, device), K=((b, t, h, d), dtype, device),
                 V=((b, t, h, d), dtype, device))
    if gating:
        props["log_G"] = ((b, t, h), torch.float32, device)
    return props


def output_properties(b=2, t=1024, h=8, d=32, qhead_ratio=1, dtype=torch.float16, device="cuda", **_unused):
    """name -> (shape, dtype, device) of the output of `power_retention` (:79-83)."""
    return dict(Y=((b, t, h * qhead_ratio, d), dtype, device))


def inference_input_properties(b=2, tq=1, tk=1024, h=8, d=32, qhead_ratio=1, dtype=torch.float16, device="cuda",
                               gating=False, initial_state=False, **_unused):
    """Tensor inputs of `power_retention_inference` (:67-77), states in the exact layout."""
    D = layout.exact_dim(d)
    props = dict(Q=((b, tq, h * qhead_ratio, d), dtype, device))
    if tk > 0:
        props["K"] = ((b, tk, h, d), dtype, device)
        props["V"] = ((b, tk, h, d), dtype, device)
        if gating:
            props["log_G"] = ((b, tk, h), torch.float32, device)
    if initial_state:
        props["initial_state"] = ((b, h, D, d), dtype, device)
        props["sum_of_keys"] = ((b, h, D), torch.float32, device)
    return props


def inference_output_properties(b=2, tq=1, tk=1024, h=8, d=32, qhead_ratio=1, dtype=torch.bfloat16, device="cuda",
                                initial_state=False, switch_over_seq_len=512, **_unused):
    """Outputs of `power_retention_inference` (:85-86): a state pair comes back when one went in or when
    the cache reached the switch-over length."""
    D = layout.exact_dim(d)
    has_state = bool(initial_state) or (switch_over_seq_len is not None and tk >= switch_over_seq_len)
    return dict(Y=((b, tq, h * qhead_ratio, d), dtype, device),
                state=((b, h, D, d), dtype, device) if has_state else None,
                sum_of_keys=((b, h, D), torch.float32, device) if has_state else None)


# Parameter grids of the reference's own test tables for the two operators (perf/tests/test_list.py:248-259
# for the full operator, :274-335 for inference), restricted to what exists in this package (head dim 64 for
# inference, explicit sum_of_keys).  tests/ walks these.
TRAIN_GRID = dict(b=[1], t=[31, 128, 1024, 2000], h=[2], d=[32, 64], qhead_ratio=[1], dtype=[torch.bfloat16],
                  gating=[False, True], chunk_size=[None, 128], deg=[2])
INFERENCE_GRID = dict(b=[1], tq=[1, 63], tk=[64, 128], h=[2], d=[64], qhead_ratio=[1, 12], dtype=[torch.bfloat16],
                      gating=[True], deg=[2], initial_state=[True, False], switch_over_seq_len=[128, 512])
INFERENCE_GRID_NO_CACHE = dict(b=[1], tq=[1], tk=[0], h=[2], d=[64], qhead_ratio=[1, 8], dtype=[torch.bfloat16],
                               gating=[True], deg=[2], initial_state=[True])


def grid_cases(grid: dict):
    """Cross product of a parameter grid as a list of keyword dicts."""
    import itertools

    keys = list(grid)
    return [dict(zip(keys, vals)) for vals in itertools.product(*(grid[k] for k in keys))]

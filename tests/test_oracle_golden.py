"""Pins the CPU oracle to the reference: oracle outputs vs fixtures produced by the
reference's own retention/reference.py (tests/golden/make_golden.py)."""
import math

import pytest
import torch

from oracle import power_retention_oracle as oracle
from tests._golden import load, rel_l2

FP32_TOL = 2e-5  # relative L2, fp32 arithmetic on both sides (summation order differs)


def _train(name, dtype):
    g = load(name)
    b, t, h, d, r, gated, chunk, stride = g["meta"]
    Q, K, V = (g[k].to(dtype).requires_grad_(True) for k in ("Q", "K", "V"))
    lg = g["log_G"].clone().requires_grad_(True) if gated else None
    O = oracle.power_retention(Q, K, V, lg, deg=2, chunk_size=chunk or None)
    O.backward(g["dO"].to(dtype))
    sl = slice(None, None, stride)
    got = {"O": O[:, sl], "dQ": Q.grad[:, sl], "dK": K.grad[:, sl], "dV": V.grad[:, sl]}
    if gated:
        got["dlog_G"] = lg.grad[:, sl]
    return g, got


@pytest.mark.parametrize("name", ["train_cfg1_fp32", "train_gated_fp32", "train_ungated_gqa_pad_fp32",
                                  "train_short_quadratic_fp32", "train_slow_decay_fp32"])
def test_training_fp32_matches_reference(name):
    g, got = _train(name, torch.float32)
    for key, val in got.items():
        assert rel_l2(val.float(), g[key]) < FP32_TOL, key


def test_training_bf16_matches_reference():
    # both sides round at the same places; only summation order differs
    g, got = _train("train_gated_bf16", torch.bfloat16)
    for key, val in got.items():
        assert rel_l2(val.float(), g[key]) < 6e-3, key


def test_operators_match_reference():
    g = load("ops_fp32")
    Q, K, V, a = g["Q"], g["K"], g["V"], g["a"]
    b, n, c, hq, d = Q.shape
    h = K.shape[3]
    o, l, m = oracle.attention(Q.view(b * n, c, hq, d), K.view(b * n, c, h, d), V.view(b * n, c, h, d),
                               a.view(b * n, c, h), 2, 1.0 / math.sqrt(d), norm=False)
    assert rel_l2(o, g["attn_o"]) < FP32_TOL and rel_l2(l, g["attn_l"]) < FP32_TOL
    assert torch.allclose(m, g["attn_m"], atol=1e-5)
    S, N = oracle.update_state(K, V, 2)
    assert S.shape == g["S"].shape == (b, n, h, oracle.expanded_dim(d), d)
    assert rel_l2(S, g["S"]) < FP32_TOL and rel_l2(N, g["N"]) < FP32_TOL
    A = a[:, :, -1].contiguous()
    Y, y = oracle.discumsum(S, A), oracle.discumsum(N, A)
    assert rel_l2(Y, g["Y"]) < FP32_TOL and rel_l2(y, g["y"]) < FP32_TOL
    assert torch.count_nonzero(Y[:, 0]) == 0
    O = oracle.query_state(Q, g["Y"][:, :n], g["y"][:, :n], g["attn_o"].view(b, n, c, hq, d),
                           g["attn_l"].view(b, n, c, hq), g["attn_m"].view(b, n, c, hq), 2, 1.0 / math.sqrt(d), True)
    assert rel_l2(O, g["O"]) < FP32_TOL


@pytest.mark.parametrize("name", ["infer_decode_state", "infer_switch_over", "infer_no_state_switch",
                                  "infer_state_only", "infer_prefill_with_state"])
def test_inference_matches_reference(name):
    g = load(name)
    b, tq, tk, h, r, d, with_state, sw = g["meta"]
    Y, ns, nk = oracle.power_retention_inference(g["Q"], g.get("K"), g.get("V"), g.get("log_G"), g.get("state"),
                                                 g.get("sum_of_keys"), deg=2, switch_over_seq_len=sw)
    assert rel_l2(Y, g["Y"]) < FP32_TOL
    if tk >= sw:
        assert rel_l2(ns, g["new_state"]) < FP32_TOL and rel_l2(nk, g["new_sum_of_keys"]) < FP32_TOL
    else:  # the reference hands back the very same objects when nothing is compressed
        assert ns is g.get("state") and nk is g.get("sum_of_keys")


def test_chunked_equals_tokenwise_quadratic():
    g = load("train_gated_fp32")
    O = oracle.power_retention(g["Q"], g["K"], g["V"], g["log_G"], deg=2, chunk_size=64)
    assert rel_l2(O, oracle.power_retention_quadratic(g["Q"], g["K"], g["V"], g["log_G"]).float()) < 2e-5

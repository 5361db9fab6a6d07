"""Generates the golden fixtures in this directory by running the reference's own CPU
implementation (`retention/reference.py` of raizoken23/retention_integration).

    python tests/golden/make_golden.py /path/to/reference_checkout

`import retention` does not work from a plain checkout (its __init__ imports the optional
`vidrial` dependency and its Triton modules write files next to themselves at import),
so the reference package's sub-modules are imported through empty package stubs.  Only
torch and einops are needed.  Inputs are stored with the outputs so the tests never
depend on a random-number generator's bit pattern.
"""
import importlib
import math
import os
import sys
import types

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    pkg = os.path.join(root, "retention")

    def stub(name, path):
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m

    stub("retention", pkg)
    for sub in ("_attention", "_update_state", "_discumsum", "_query_state"):
        stub(f"retention.{sub}", os.path.join(pkg, sub))
    return importlib.import_module("retention.reference")


def npy(x):
    return None if x is None else x.detach().to(torch.float32).numpy()


def bits(x):
    """Inputs are generated bf16-representable and stored as their 16-bit patterns
    (key suffix `__bf16`), which halves the fixture size without losing a bit."""
    if x is None:
        return None
    xb = x.detach().to(torch.bfloat16)
    assert torch.equal(xb.to(torch.float32), x.detach().to(torch.float32))
    return xb.view(torch.int16).numpy().view(np.uint16)


def rb(x):
    return x.to(torch.bfloat16).to(torch.float32)


def save(name, **arrays):
    arrays = {k: v for k, v in arrays.items() if v is not None}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
    print(name, {k: tuple(np.shape(v)) for k, v in arrays.items()})


def make_inputs(seed, b, t, h, d, r, dtype, gated, in_scale=1.0, gate_shift=0.0):
    g = torch.Generator().manual_seed(seed)
    Q = rb(torch.randn(b, t, h * r, d, generator=g) * in_scale).to(dtype)
    K = rb(torch.randn(b, t, h, d, generator=g) * in_scale).to(dtype)
    V = rb(torch.randn(b, t, h, d, generator=g) * in_scale).to(dtype)
    log_G = F.logsigmoid(torch.randn(b, t, h, generator=g) + gate_shift) if gated else None
    dO = rb(torch.randn(b, t, h * r, d, generator=g)).to(dtype)
    return Q, K, V, log_G, dO


def training_case(ref, name, seed, b, t, h, d, r, dtype, gated, chunk, in_scale=1.0, gate_shift=0.0, stride=1):
    Q, K, V, log_G, dO = make_inputs(seed, b, t, h, d, r, dtype, gated, in_scale, gate_shift)
    leaves = [x.clone().requires_grad_(True) for x in (Q, K, V)]
    lg = log_G.clone().requires_grad_(True) if gated else None
    O = ref.power_retention(leaves[0], leaves[1], leaves[2], lg, deg=2, chunk_size=chunk)
    O.backward(dO)
    sl = slice(None, None, stride)
    save(name, Q__bf16=bits(Q), K__bf16=bits(K), V__bf16=bits(V), log_G=npy(log_G), dO__bf16=bits(dO),
         O=npy(O)[:, sl], dQ=npy(leaves[0].grad)[:, sl], dK=npy(leaves[1].grad)[:, sl],
         dV=npy(leaves[2].grad)[:, sl], dlog_G=None if lg is None else npy(lg.grad)[:, sl],
         meta=np.array([b, t, h, d, r, int(gated), chunk or 0, stride]))


def op_cases(ref):
    att = sys.modules["retention._attention.reference"].attention
    upd = sys.modules["retention._update_state.reference"].update_state
    dcs = sys.modules["retention._discumsum.reference"].discumsum_reference
    qst = sys.modules["retention._query_state.reference"].query_state_reference
    g = torch.Generator().manual_seed(7)
    b, n, c, h, r, d = 1, 3, 32, 2, 2, 32
    Q = rb(torch.randn(b, n, c, h * r, d, generator=g))
    K = rb(torch.randn(b, n, c, h, d, generator=g))
    V = rb(torch.randn(b, n, c, h, d, generator=g))
    a = F.logsigmoid(torch.randn(b, n, c, h, generator=g)).cumsum(2)
    o, l, m = att(Q.view(b * n, c, h * r, d), K.view(b * n, c, h, d), V.view(b * n, c, h, d), a.view(b * n, c, h), 2,
                  scale=1.0 / math.sqrt(d), norm=False)
    S, N = upd(K, V, 2)
    A = a[:, :, -1].contiguous()
    Y = dcs(S, A)
    y = dcs(N, A)
    O = qst(Q, Y[:, :n].contiguous(), y[:, :n].contiguous(), o.view(b, n, c, h * r, d), l.view(b, n, c, h * r),
            m.view(b, n, c, h * r), 2, 1.0 / math.sqrt(d), True)
    save("ops_fp32", Q__bf16=bits(Q), K__bf16=bits(K), V__bf16=bits(V), a=npy(a), attn_o=npy(o), attn_l=npy(l), attn_m=npy(m), S=npy(S),
         N=npy(N), Y=npy(Y), y=npy(y), O=npy(O))


def inference_cases(ref):
    Dref = {32: 768, 64: 2560}
    for name, seed, b, tq, tk, h, r, d, with_state, sw in [
        ("infer_decode_state", 11, 1, 1, 48, 1, 1, 64, True, 512),
        ("infer_switch_over", 12, 1, 1, 64, 1, 2, 64, True, 64),
        ("infer_no_state_switch", 13, 1, 5, 64, 2, 1, 64, False, 64),
        ("infer_state_only", 14, 1, 1, 0, 1, 4, 64, True, 512),
        ("infer_prefill_with_state", 15, 1, 63, 128, 1, 2, 64, True, 512),
    ]:
        g = torch.Generator().manual_seed(seed)
        Q = rb(torch.randn(b, tq, h * r, d, generator=g) / math.sqrt(d))
        K = rb(torch.randn(b, tk, h, d, generator=g) / math.sqrt(d)) if tk else None
        V = rb(torch.randn(b, tk, h, d, generator=g) / math.sqrt(d)) if tk else None
        log_G = F.logsigmoid(2.0 + torch.randn(b, tk, h, generator=g)) if tk else None
        state = sk = None
        if with_state:
            # a realistic state: the reference's own update_state over 96 earlier tokens, so that the
            # normaliser phi(q).sum_of_keys is a sum of squares (a random state makes it cancel)
            upd = sys.modules["retention._update_state.reference"].update_state
            K0 = rb(torch.randn(b, 96, h, d, generator=g) / math.sqrt(d))
            V0 = rb(torch.randn(b, 96, h, d, generator=g) / math.sqrt(d))
            state, sk = upd(K0, V0, 2)
            state = rb(state)
            assert state.shape == (b, h, Dref[d], d)
        Y, ns, nk = ref.power_retention_inference(Q, K, V, log_G, state, sk, deg=2, switch_over_seq_len=sw)
        switched = tk >= sw
        save(name, Q__bf16=bits(Q), K__bf16=bits(K), V__bf16=bits(V), log_G=npy(log_G), state__bf16=bits(state),
             sum_of_keys=npy(sk), Y=npy(Y), new_state=npy(ns) if switched else None,
             new_sum_of_keys=npy(nk) if switched else None, meta=np.array([b, tq, tk, h, r, d, int(with_state), sw]))


def caller_case(root):
    """The glue of deploy/nanoGPT/model.py:66-84 on a random projection output, with the reference's own
    rotary helpers (the module is loaded with a stub for its `retention.triton` import)."""
    import importlib.util

    stub = types.ModuleType("retention.triton")
    stub.power_retention = None
    sys.modules["retention.triton"] = stub
    spec = importlib.util.spec_from_file_location("ref_nanogpt_model", os.path.join(root, "deploy", "nanoGPT", "model.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    g = torch.Generator().manual_seed(21)
    B, T, h, r, d = 2, 48, 2, 2, 64
    hq = h * r
    qkv_size = (hq + 2 * h) * d
    qkvg = rb(torch.randn(B, T, qkv_size + h, generator=g)).to(torch.bfloat16).requires_grad_(True)
    # model.py:68-84, line by line
    qkv = qkvg[..., :qkv_size]
    q, k, v = qkv.split([hq * d, h * d, h * d], dim=2)
    q, k, v = q.view(B, T, hq, d), k.view(B, T, h, d), v.view(B, T, h, d)
    log_g = torch.nn.functional.logsigmoid(6.906768 + qkvg[..., qkv_size:].to(dtype=torch.float32)).contiguous()
    pos = torch.arange(T, dtype=torch.float32).unsqueeze(0).unsqueeze(2)
    sincos = m.get_sinusoidal_embeddings(pos, d, "cpu")
    q = m.apply_rotary_position_embeddings(q, sincos)
    k = m.apply_rotary_position_embeddings(k, sincos)
    dq, dk, dv = (rb(torch.randn(*x.shape, generator=g)).to(torch.bfloat16) for x in (q, k, v))
    dlg = torch.randn(B, T, h, generator=g)
    torch.autograd.backward([q, k, v, log_g], [dq, dk, dv, dlg])
    save("caller_prep_nanogpt", qkvg__bf16=bits(qkvg), Q__bf16=bits(q), K__bf16=bits(k), V__bf16=bits(v), log_g=npy(log_g),
         sin=npy(sincos[0][0, :, 0]), cos=npy(sincos[1][0, :, 0]), dQ__bf16=bits(dq), dK__bf16=bits(dk), dV__bf16=bits(dv),
         dlog_g=npy(dlg), dqkvg=npy(qkvg.grad), meta=np.array([B, T, h, r, d]))


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference>")
    ref = load_reference(sys.argv[1])
    torch.set_num_threads(os.cpu_count() or 1)
    # the reference's CPU-runnable case (b1 t1024 h4 d64 fp32 c128 gated); outputs kept for every 8th token
    training_case(ref, "train_cfg1_fp32", 1, 1, 1024, 4, 64, 1, torch.float32, True, 128, stride=8)
    training_case(ref, "train_gated_fp32", 2, 1, 256, 2, 64, 1, torch.float32, True, 64)
    training_case(ref, "train_ungated_gqa_pad_fp32", 3, 2, 200, 2, 32, 2, torch.float32, False, 64)
    training_case(ref, "train_short_quadratic_fp32", 4, 1, 31, 2, 32, 1, torch.float32, True, None)
    training_case(ref, "train_slow_decay_fp32", 5, 1, 256, 1, 64, 1, torch.float32, True, 64, gate_shift=4.0)
    training_case(ref, "train_gated_bf16", 6, 1, 256, 2, 64, 1, torch.bfloat16, True, 64)
    op_cases(ref)
    inference_cases(ref)
    caller_case(sys.argv[1])


if __name__ == "__main__":
    main()

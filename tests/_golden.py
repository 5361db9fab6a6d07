"""Loader for the fixtures written by tests/golden/make_golden.py."""
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    out = {}
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        for key in z.files:
            arr = z[key]
            if key.endswith("__bf16"):
                t = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16).to(torch.float32)
                out[key[: -len("__bf16")]] = t
            elif key == "meta":
                out[key] = [int(v) for v in arr]
            else:
                out[key] = torch.from_numpy(arr.copy())
    return out


def rel_l2(x, ref):
    x, ref = x.detach().double(), ref.detach().double()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-30))


def make_state(b, h, d, n_tokens, gen, dtype=torch.bfloat16):
    """A state pair in the exact layout as real tokens leave it: S = sum_j w phi(k_j) v_j^T,
    z = sum_j w phi(k_j) over n_tokens random keys and values (so the normaliser q -> phi(q).z =
    sum_j (q.k_j)^2 is positive, unlike that of a random tensor)."""
    K = torch.randn(b, n_tokens, h, d, generator=gen).to(dtype).float()
    V = torch.randn(b, n_tokens, h, d, generator=gen).to(dtype).float()
    ia, ib = torch.triu_indices(d, d)
    w = torch.where(ia == ib, 1.0, 2.0)
    S = torch.zeros(b, h, ia.numel(), d)
    z = torch.zeros(b, h, ia.numel())
    for j in range(n_tokens):  # token by token: the expanded keys of all tokens at once would not fit for large b*h
        phi = K[:, j, :, ia] * K[:, j, :, ib] * w
        S += phi.unsqueeze(-1) * V[:, j].unsqueeze(-2)
        z += phi
    return S.to(dtype), z

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

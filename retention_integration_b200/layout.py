"""Layouts of the degree-2 symmetric-power expansion and converters between them.

Two layouts of the expanded dimension exist for head dim d:

* ``exact``      C(d+1, 2) entries, pair (a <= b) at  a*d - a*(a-1)/2 + (b-a)
                 (2080 at d = 64).  States returned by ``power_retention_inference``.
* ``reference``  the reference package's padded layout (2560 at d = 64): entry
                 256*y*(y+1)/2 + 16*x + i  holds the pair (x, 16*y+i) for x < 16*(y+1)
                 (retention/_update_state/reference.py:5-29).  The kernels and the chunk
                 states of the training path use this layout too.

States and sums of keys carry the key-side multiplicity: weight 2 on a pair a != b in
``exact``.  The reference stores weight 2 only on pairs whose two indices lie
in different 16-blocks; inside a diagonal block it stores (a,b) and (b,a) separately with
weight 1, so converting to the reference layout halves those entries and converting
back adds the two halves.
"""
from __future__ import annotations

from functools import lru_cache

import torch


def exact_dim(d: int) -> int:
    return d * (d + 1) // 2


def reference_dim(d: int) -> int:
    nb = d // 16
    return 256 * nb * (nb + 1) // 2


def _exact_index(d: int, a: int, b: int) -> int:
    return a * d - a * (a - 1) // 2 + (b - a)


@lru_cache(maxsize=None)
def _tables(d: int):
    """(ref_src_exact [Dref], ref_coef [Dref], exact_from_ref_1 [Dex], exact_from_ref_2 [Dex]
    (-1 if the pair has a single entry))."""
    ref_src = torch.empty(reference_dim(d), dtype=torch.long)
    ref_coef = torch.empty(reference_dim(d), dtype=torch.float32)
    ex1 = torch.full((exact_dim(d),), -1, dtype=torch.long)
    ex2 = torch.full((exact_dim(d),), -1, dtype=torch.long)
    for y in range(d // 16):
        base = 256 * y * (y + 1) // 2
        for x in range(16 * (y + 1)):
            for i in range(16):
                yy = 16 * y + i
                I = base + 16 * x + i
                a, b = min(x, yy), max(x, yy)
                e = _exact_index(d, a, b)
                ref_src[I] = e
                same_block = x >= 16 * y
                ref_coef[I] = 0.5 if (same_block and a != b) else 1.0
                if ex1[e] < 0:
                    ex1[e] = I
                else:
                    ex2[e] = I
    return ref_src, ref_coef, ex1, ex2


def _move(x: torch.Tensor, dim: int):
    return x.movedim(dim, -1)


def exact_to_reference(x: torch.Tensor, d: int, dim: int = -2) -> torch.Tensor:
    """State / sum-of-keys in the exact layout -> the reference package's layout."""
    ref_src, ref_coef, _, _ = _tables(d)
    xm = _move(x, dim)
    out = xm.index_select(-1, ref_src.to(x.device)) * ref_coef.to(device=x.device, dtype=x.dtype)
    return out.movedim(-1, dim).contiguous()


def reference_to_exact(x: torch.Tensor, d: int, dim: int = -2) -> torch.Tensor:
    """The reference package's layout -> exact (the two halves of in-block pairs are added)."""
    _, _, ex1, ex2 = _tables(d)
    xm = _move(x, dim)
    out = xm.index_select(-1, ex1.to(x.device))
    second = xm.index_select(-1, ex2.clamp_min(0).to(x.device)) * (ex2 >= 0).to(device=x.device, dtype=x.dtype)
    return (out + second).movedim(-1, dim).contiguous()


def to_reference_layout(x: torch.Tensor, d: int, dim: int = -2) -> torch.Tensor:
    return exact_to_reference(x, d, dim)


def from_reference_layout(x: torch.Tensor, d: int, dim: int = -2) -> torch.Tensor:
    return reference_to_exact(x, d, dim)


def gram_to_exact_sum_of_keys(gram: torch.Tensor) -> torch.Tensor:
    """d x d Gram matrix of the keys (last two dims) -> sum of keys in the exact layout:
    entry (a <= b) = weight(a, b) * gram[a, b]."""
    d = gram.shape[-1]
    ia, ib = torch.triu_indices(d, d, device=gram.device)
    w = torch.where(ia == ib, 1.0, 2.0).to(gram.dtype)
    return gram[..., ia, ib] * w


def exact_sum_of_keys_to_gram(s: torch.Tensor, d: int) -> torch.Tensor:
    """Inverse of gram_to_exact_sum_of_keys (symmetric result)."""
    ia, ib = torch.triu_indices(d, d, device=s.device)
    w = torch.where(ia == ib, 1.0, 0.5).to(s.dtype)
    g = torch.zeros(*s.shape[:-1], d, d, device=s.device, dtype=s.dtype)
    g[..., ia, ib] = s * w
    g[..., ib, ia] = s * w
    return g

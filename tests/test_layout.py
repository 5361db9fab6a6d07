"""Expansion layouts and their converters against the oracle's reference-layout tables."""
import torch

from oracle import power_retention_oracle as oracle
from retention_integration_b200 import layout


def _weighted_exact(k):
    d = k.shape[-1]
    ia, ib = torch.triu_indices(d, d)
    w = torch.where(ia == ib, 1.0, 2.0)
    return k[..., ia] * k[..., ib] * w


def test_dims():
    assert (layout.exact_dim(64), layout.reference_dim(64)) == (2080, 2560)
    assert layout.reference_dim(32) == oracle.expanded_dim(32) == 768
    assert layout.reference_dim(128) == oracle.expanded_dim(128) == 9216


def test_exact_to_reference_matches_reference_expansion():
    for d in (32, 64):
        k = torch.randn(3, d, dtype=torch.float64)
        ref = oracle.expand(k, key_side=True)
        got = layout.exact_to_reference(_weighted_exact(k), d, dim=-1)
        assert torch.allclose(got, ref, atol=1e-12)
        back = layout.reference_to_exact(ref, d, dim=-1)
        assert torch.allclose(back, _weighted_exact(k), atol=1e-12)


def test_query_key_inner_product_is_squared_dot():
    d = 64
    q, k = torch.randn(d, dtype=torch.float64), torch.randn(d, dtype=torch.float64)
    ia, ib = torch.triu_indices(d, d)
    phi_q = q[ia] * q[ib]
    assert torch.allclose((phi_q * _weighted_exact(k)).sum(), (q @ k) ** 2)


def test_gram_sum_of_keys_roundtrip():
    d = 32
    K = torch.randn(10, d, dtype=torch.float64)
    gram = K.T @ K
    s = layout.gram_to_exact_sum_of_keys(gram)
    assert torch.allclose(s, _weighted_exact(K).sum(0))
    assert torch.allclose(layout.exact_sum_of_keys_to_gram(s, d), gram)

"""CPU oracle for power retention.  TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

A restatement, in plain PyTorch CPU ops, of the algorithm of the reference package
`retention` (reference backend, `retention/reference.py:8-9`).  Only `tests/`,
`__graft_entry__.smoke()` and the CPU-baseline legs of `bench.py` may import this
module; the shipped package never does.

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own
`retention/reference.py` (imported from a checkout of the reference) on seeded
inputs and stores its outputs, gradients, states and per-operator results;
`tests/test_oracle_golden.py` checks this restatement against those fixtures.

Every function is differentiable by autograd, which is how gradients are defined
for the reference too (its operators' hand-written backward passes are either
absent or wrap the same formulas).

Layouts follow the reference: the expanded dimension is the padded
D = 16 * sum_{y<d/16} 16*(y+1)  (768 / 2560 / 9216 for d = 32 / 64 / 128).
"""
from __future__ import annotations

import math
from functools import lru_cache

import torch

__all__ = [
    "expanded_dim",
    "expansion_index",
    "expand",
    "attention",
    "update_state",
    "discumsum",
    "query_state",
    "power_retention",
    "power_retention_inference",
    "power_retention_quadratic",
]

_BLOCK = 16  # inner block of the reference layout (retention/_utils.py:5-8)


def expanded_dim(d: int, deg: int = 2) -> int:
    """Padded expanded dimension; equals compute_expanded_dim (retention/_utils.py:18-19)."""
    assert deg == 2 and d % _BLOCK == 0
    nb = d // _BLOCK
    return _BLOCK * _BLOCK * nb * (nb + 1) // 2


@lru_cache(maxsize=None)
def expansion_index(d: int):
    """Index tables of the reference phi layout.

    Entry I = 256*y*(y+1)/2 + 16*x + i  holds  v[x] * v[16*y + i]  for
    y in [0, d/16), x in [0, 16*(y+1)), i in [0, 16).  On the key side entries
    with x < 16*y (blocks strictly left of the diagonal block) carry weight 2
    (retention/_update_state/reference.py:21-27; the query side has no weight,
    retention/_query_state/reference.py:25-31).
    Returns (ia, ib, key_weight) as int64/int64/float32 tensors of length D.
    """
    ia, ib, w = [], [], []
    for y in range(d // _BLOCK):
        for x in range(_BLOCK * (y + 1)):
            for i in range(_BLOCK):
                ia.append(x)
                ib.append(_BLOCK * y + i)
                w.append(2.0 if x < _BLOCK * y else 1.0)
    return torch.tensor(ia), torch.tensor(ib), torch.tensor(w)


def expand(X: torch.Tensor, key_side: bool) -> torch.Tensor:
    """phi(X) along the last dim, rounded to X's dtype after the product (as the
    reference's einsum + cast does, retention/_update_state/reference.py:17)."""
    ia, ib, w = expansion_index(X.shape[-1])
    phi = X.index_select(-1, ia) * X.index_select(-1, ib)
    if key_side:
        phi = phi * w.to(X.dtype)
    return phi


def attention(Q, K, V, log_G_cum, deg: int, scale: float, norm: bool):
    """Causal power attention of one block of tokens (retention/_attention/reference.py:10-69).

    Q [b,tq,hq,d]; K,V [b,tk,h,d]; log_G_cum [b,tk,h] fp32 (inclusive cumulative log
    gates) or None.  The tq queries are the LAST tq positions of the tk keys.  hq = r*h:
    query head j reads kv head j // r.
    Returns O [b,tq,hq,d] if norm else (O, l [b,tq,hq] fp32, rowmax [b,tq,hq] fp32) with
    O and l expressed relative to exp(rowmax).
    """
    b, tq, hq, d = Q.shape
    tk, h = K.shape[1], K.shape[2]
    r = hq // h
    assert deg % 2 == 0 and hq == r * h
    Kx = K.repeat_interleave(r, dim=2) if r > 1 else K
    Vx = V.repeat_interleave(r, dim=2) if r > 1 else V
    s = torch.einsum("bihd,bjhd->bhij", Q, Kx) * scale  # [b,hq,tq,tk]
    z = float(deg) * torch.log(s.abs() + 1e-7)  # :47
    qi = torch.arange(tq).unsqueeze(1) + (tk - tq)
    kj = torch.arange(tk).unsqueeze(0)
    z = torch.where(qi >= kj, z, torch.full_like(z, -float("inf")))
    if log_G_cum is not None:
        g = log_G_cum.transpose(1, 2)  # [b,h,tk]
        gx = g.repeat_interleave(r, dim=1) if r > 1 else g
        z = z + (gx[..., -tq:, None] - gx[..., None, :])
    rowmax = z.max(dim=-1, keepdim=True).values.detach()  # :50
    p = torch.exp(z - rowmax).to(V.dtype)
    l = p.sum(-1).to(torch.float32) + 1e-6  # :55
    o = torch.einsum("bhij,bjhe->bihe", p, Vx)
    l = l.transpose(1, 2)
    rowmax = rowmax.squeeze(-1).transpose(1, 2).to(torch.float32)
    if norm:
        return (o / l[..., None]).to(V.dtype)
    return o, l, rowmax


def update_state(K, V, deg: int = 2):
    """Chunk states (retention/_update_state/reference.py:31-53,85-94).

    K,V [b,n,c,h,d] (or [b,c,h,d] for the inference call) ->
    S [b,n,h,D,d] in K's dtype, N [b,n,h,D] fp32.
    """
    assert deg == 2
    if K.dim() == 4:
        S, N = update_state(K.unsqueeze(1), V.unsqueeze(1), deg)
        return S.squeeze(1), N.squeeze(1)
    phi = expand(K.transpose(2, 3), key_side=True)  # [b,n,h,c,D]
    N = phi.to(torch.float32).sum(dim=3)
    S = torch.matmul(phi.transpose(-1, -2), V.transpose(2, 3))
    return S, N


def discumsum(X, log_G):
    """Gated prefix scan over the chunk axis with a leading zero entry
    (retention/_discumsum/reference.py:3-15): Y[0]=0, Y[1]=X[0],
    Y[j+1] = round(Y[j]*exp(log_G[j])) + X[j].   X [b,n,h,...], log_G [b,n,h]."""
    n = X.shape[1]
    extra = X.dim() - 3
    g = torch.exp(log_G).reshape(*log_G.shape, *([1] * extra))
    state = X[:, 0].to(torch.float32)
    out = [torch.zeros_like(X[:, 0]), state.to(X.dtype)]
    for j in range(1, n):
        state = (state * g[:, j]).to(X.dtype) + X[:, j]
        out.append(state)
    return torch.stack(out, dim=1)


def query_state(Q, S, s, Y_attn, l_attn, rowmax, deg: int, scale: float, zero_initial_state: bool):
    """State read-out merged with the intra-chunk attention and normalised
    (retention/_query_state/reference.py:36-96,166-191).

    Q [b,n,c,hq,d]; S [b,n,h,D,e]; s [b,n,h,D]; Y_attn [b,n,c,hq,e], l_attn, rowmax
    [b,n,c,hq] or None.  4-D Q = inference call (n squeezed).
    """
    if Q.dim() == 4:
        un = lambda x: None if x is None else x.unsqueeze(1)
        return query_state(un(Q), un(S), un(s), un(Y_attn), un(l_attn), un(rowmax), deg, scale,
                           zero_initial_state).squeeze(1)
    b, n, c, hq, d = Q.shape
    h, D = S.shape[2], S.shape[3]
    r = hq // h
    gamma = torch.full((n,), math.sqrt(float(D)), dtype=torch.float32)
    if zero_initial_state:
        gamma[0] = 1.0  # :63-66
    gamma = gamma.view(1, n, 1, 1)
    phi = expand(Q, key_side=False)  # [b,n,c,hq,D]
    Sg = (S / gamma.unsqueeze(-1)).to(S.dtype)
    sg = s / gamma
    Sx = Sg.repeat_interleave(r, dim=2) if r > 1 else Sg
    sx = sg.repeat_interleave(r, dim=2) if r > 1 else sg
    Y_qs = torch.einsum("bnchD,bnhDe->bnche", phi, Sx.to(Q.dtype)).to(Q.dtype)
    l_qs = torch.einsum("bnchD,bnhD->bnch", phi.to(torch.float32), sx.to(torch.float32))
    sp = scale ** deg
    if Y_attn is not None:
        alpha = torch.maximum(gamma, torch.exp(rowmax))
        fa = torch.exp(rowmax) / alpha
        fq = gamma / alpha
        O = Y_attn * fa.unsqueeze(-1) + Y_qs * sp * fq.unsqueeze(-1)
        l = l_attn * fa + l_qs * sp * fq
    else:
        O, l = Y_qs, l_qs
    return (O.to(torch.float32) / l.unsqueeze(-1)).to(Y_qs.dtype)


def power_retention(Q, K, V, log_G=None, initial_state=None, return_final_state=False, deg=2, scale=None,
                    chunk_size=None, switch_over_seq_len=None):
    """Training forward (retention/power_retention_maker.py:71-197).  Q [b,t,hq,d],
    K,V [b,t,h,d], log_G [b,t,h] fp32 or None -> O [b,t,hq,d]."""
    assert initial_state is None and not return_final_state, "unfinished in the reference (:43,:158-160)"
    assert deg % 2 == 0
    b, t, hq, d = Q.shape
    h = K.shape[2]
    r = hq // h
    t_orig = t
    if chunk_size is not None and t % chunk_size:
        pad = chunk_size - t % chunk_size  # :75-83, gate 1 on padded tokens
        zp = lambda x: torch.nn.functional.pad(x, (0, 0, 0, 0, 0, pad))
        Q, K, V = zp(Q), zp(K), zp(V)
        if log_G is not None:
            log_G = torch.nn.functional.pad(log_G, (0, 0, 0, pad))
        t += pad
    if log_G is not None:
        log_G = log_G.to(torch.float32)
    if not scale:
        scale = 1.0 / math.sqrt(d)
    if chunk_size is None:
        c, n, sw = t, 1, switch_over_seq_len
    else:
        c, n = chunk_size, t // chunk_size
        sw = chunk_size if switch_over_seq_len is None else switch_over_seq_len
    if sw is None or t <= sw:  # :128-132
        G = log_G.cumsum(1) if log_G is not None else None
        return attention(Q, K, V, G, deg, scale, norm=True)[:, :t_orig]
    Qc, Kc, Vc = Q.view(b, n, c, hq, d), K.view(b, n, c, h, d), V.view(b, n, c, h, d)
    if log_G is not None:
        a = log_G.view(b, n, c, h).cumsum(2)
        disc = torch.exp((a[:, :, -1:] - a) / deg).unsqueeze(-1).to(K.dtype)  # :151-153
        Kd = Kc * disc
        A = a[:, :, -1].contiguous()
    else:
        a, Kd = None, Kc
        A = torch.zeros(b, n, h, dtype=torch.float32)
    S, s = update_state(Kd, Vc, deg)
    S = discumsum(S, A)[:, :n]  # state entering each chunk, :167-170
    s = discumsum(s, A)[:, :n]
    Ya, la, m = attention(Qc.reshape(b * n, c, hq, d), Kc.reshape(b * n, c, h, d), Vc.reshape(b * n, c, h, d),
                          None if a is None else a.reshape(b * n, c, h), deg, scale, norm=False)
    Ya, la, m = Ya.view(b, n, c, hq, d), la.view(b, n, c, hq), m.view(b, n, c, hq)
    if a is not None:
        ax = a.repeat_interleave(r, dim=3) if r > 1 else a
        Qg = Qc * torch.exp(ax / deg).unsqueeze(-1).to(Q.dtype)  # :183-186
    else:
        Qg = Qc
    Y = query_state(Qg, S, s, Ya, la, m, deg, scale, True)
    return Y.reshape(b, t, hq, d).to(Q.dtype)[:, :t_orig]


def power_retention_inference(Q, K, V, log_G=None, initial_state=None, sum_of_keys=None, deg=2, scale=None,
                              switch_over_seq_len=512):
    """Decode / prefill-to-state step (retention/power_retention_maker.py:287-390, the
    variant with an explicit sum_of_keys, retention/reference.py:9).
    Returns (Y [b,tq,hq,d], state [b,h,D,d] or None, sum_of_keys [b,h,D] or None)."""
    has_cache = K is not None and V is not None
    assert has_cache or initial_state is not None
    b, tq, hq, d = Q.shape
    tk = K.shape[1] if has_cache else 0
    h = K.shape[2] if has_cache else initial_state.shape[1]
    r = hq // h
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    G = log_G.cumsum(1) if log_G is not None else None
    if initial_state is None:
        Y = attention(Q, K, V, G, deg, scale, norm=True)
    else:
        if tk > 0:
            Ya, la, m = attention(Q, K, V, G, deg, scale, norm=False)
        else:
            Ya = la = m = None
        Qs = Q
        if G is not None:
            Qs = Q * torch.exp(G[:, -1:] / deg).repeat_interleave(r, dim=-1).unsqueeze(-1).to(Q.dtype)  # :358-359
        Y = query_state(Qs, initial_state, sum_of_keys, Ya, la, m, deg, scale, False)
    if switch_over_seq_len is not None and tk >= switch_over_seq_len:  # :366-382
        Kd = K
        if G is not None:
            Kd = (K * torch.exp((G[:, -1:] - G) / deg).unsqueeze(-1)).to(K.dtype)
        upd, upd_s = update_state(Kd.contiguous(), V.contiguous(), deg)
        if initial_state is None:
            new_state, new_s = upd, upd_s
        elif G is None:
            new_state, new_s = initial_state + upd, sum_of_keys + upd_s
        else:
            decay = torch.exp(G[:, -1, :])
            new_state = initial_state * decay[..., None, None].to(initial_state.dtype) + upd
            new_s = sum_of_keys * decay[..., None].to(sum_of_keys.dtype) + upd_s
    else:
        new_state, new_s = initial_state, sum_of_keys
    return Y, new_state, new_s


def power_retention_quadratic(Q, K, V, log_G=None, deg=2):
    """The same map written token by token in float64 with no chunking and no rounding:
    O_i = sum_{j<=i} (q_i.k_j)^deg e^{a_i-a_j} v_j / sum_{j<=i} (q_i.k_j)^deg e^{a_i-a_j}.
    The scale cancels for even deg.  Used for size-independent checks."""
    Q, K, V = Q.double(), K.double(), V.double()
    b, t, hq, d = Q.shape
    r = hq // K.shape[2]
    Kx, Vx = K.repeat_interleave(r, dim=2), V.repeat_interleave(r, dim=2)
    w = torch.einsum("bihd,bjhd->bhij", Q, Kx) ** deg
    if log_G is not None:
        a = log_G.double().cumsum(1).transpose(1, 2).repeat_interleave(r, dim=1)
        w = w * torch.exp(torch.tril(a[..., :, None] - a[..., None, :]))
    w = torch.tril(w)
    y = torch.einsum("bhij,bjhe->bihe", w, Vx)
    return y / w.sum(-1).transpose(1, 2).unsqueeze(-1)

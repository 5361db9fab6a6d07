"""Multi-GPU use of the path.  The reference has no counterpart: it is single-device.

Two ways to spread one layer over the GPUs of a box, one process per GPU:

* by (batch, kv head): every operator of the path is independent across batch and kv
  head, so each rank runs `power_retention` on its slice and nothing is exchanged
  (`head_slice` picks the slice; query heads stay with their kv head).

* by sequence (`power_retention_sequence_parallel`): rank r owns a contiguous block of
  chunks.  The chunk scan is one linear recurrence cut into pieces, so each rank
  1. reduces its block to (F_r, L_r): the state its block alone would leave behind and its
     total log gate (a carry-only pass of the scan kernel);
  2. takes part in a chain r -> r+1 that turns these into the state entering each block,
     C_{r+1} = C_r * exp(L_r) + F_r, C_0 = 0  (one small fp32 message per hop);
  3. runs the real scan seeded with C_r.
  The backward pass mirrors it from the last rank to the first with the gradient carries.
  Messages are fp32 and land in the receiver's own memory before any kernel reads them.

The chain itself is plain tensor code behind a tiny `Comm` interface, so it runs over NCCL on
GPUs, over gloo on CPU tensors (tests), or through an in-process mailbox that emulates the
ranks one after another on a single GPU.
"""
from __future__ import annotations

import math

import torch

from . import ops
from ._lib import PRError


def head_slice(n_kv_heads: int, ratio: int, rank: int, world: int):
    """(kv head slice, query head slice) of `rank` when heads are split evenly over `world`."""
    if n_kv_heads % world:
        raise PRError(f"{n_kv_heads} kv heads do not divide over {world} ranks")
    per = n_kv_heads // world
    return slice(rank * per, (rank + 1) * per), slice(rank * per * ratio, (rank + 1) * per * ratio)


class ExchangeTimeout(PRError):
    """A boundary-state exchange did not complete within the process group's timeout: a peer never
    joined, left, or its message was lost.  The host-side counterpart of PR_ERR_TIMEOUT."""


class DistComm:
    """Boundary-state exchange over torch.distributed (NCCL for CUDA tensors, gloo for CPU ones).

    Failure handling is the process group's: create the group with a short `timeout=` and a peer that
    never shows up ends the exchange with `ExchangeTimeout` on the ranks that waited, instead of blocking
    them for ever.  Nothing is retried here; the caller decides whether to rebuild the group."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def _peer(self, r):
        return self.dist.get_global_rank(self.group, r) if self.group is not None else r

    def _guard(self, what, fn):
        try:
            return fn()
        except RuntimeError as exc:  # DistBackendError, gloo timeouts and lost connections all derive from it
            raise ExchangeTimeout(f"{what} on rank {self.rank} of {self.world} failed or timed out: {exc}") from exc

    def send(self, t, to_rank):
        self._guard("send", lambda: self.dist.send(t.contiguous(), self._peer(to_rank), group=self.group))

    def recv(self, like, from_rank):
        buf = torch.empty_like(like)
        self._guard("recv", lambda: self.dist.recv(buf, self._peer(from_rank), group=self.group))
        return buf

    def all_gather(self, t):
        """[world, *t.shape]: every rank's tensor, in rank order (one collective)."""
        flat = t.contiguous().view(-1)
        out = torch.empty(self.world * flat.numel(), device=t.device, dtype=t.dtype)
        self._guard("all_gather", lambda: self.dist.all_gather_into_tensor(out, flat, group=self.group))
        return out.view((self.world,) + tuple(t.shape))


class ChainComm:
    """A DistComm restricted to neighbour send / recv: forces the rank-to-rank chain (used by tests and
    by callers whose backend has no gather)."""

    def __init__(self, inner: DistComm):
        self.inner, self.rank, self.world = inner, inner.rank, inner.world

    def send(self, t, to_rank):
        self.inner.send(t, to_rank)

    def recv(self, like, from_rank):
        return self.inner.recv(like, from_rank)


class MailboxComm:
    """Emulates `world` ranks inside one process: ranks must run in chain order (forward:
    0..world-1, backward: world-1..0).  Used to check the arithmetic on a single GPU."""

    def __init__(self, rank: int, world: int, box: dict):
        self.rank, self.world, self.box = rank, world, box

    def send(self, t, to_rank):
        self.box[(self.rank, to_rank)] = t.clone()

    def recv(self, like, from_rank):
        return self.box.pop((from_rank, self.rank))


def forward_chain(comm, F: torch.Tensor, L: torch.Tensor):
    """F [b,h,E] fp32: what this rank's block alone leaves behind; L [b,h]: its total log gate.
    Returns the state entering this rank's block (None on rank 0).

    With a communicator that can gather (torch.distributed) the summaries of all ranks are exchanged
    in ONE collective and every rank runs the short recurrence C_{q+1} = C_q exp(L_q) + F_q over the
    ranks before it on its own copy: the latency of one exchange instead of world-1 dependent hops.
    Otherwise (the in-process mailbox) the summaries travel rank to rank."""
    if hasattr(comm, "all_gather"):
        if comm.world == 1:
            return None
        Fs, Ls = comm.all_gather(F), comm.all_gather(L)
        C = None
        for q in range(comm.rank):
            C = Fs[q].clone() if C is None else torch.addcmul(Fs[q], C, torch.exp(Ls[q]).unsqueeze(-1))
        return C
    C = None
    if comm.rank > 0:
        C = comm.recv(F, comm.rank - 1)
    if comm.rank < comm.world - 1:
        nxt = F if C is None else torch.addcmul(F, C, torch.exp(L).unsqueeze(-1))
        comm.send(nxt, comm.rank + 1)
    return C


def backward_chain(comm, G: torch.Tensor, L: torch.Tensor):
    """G [b,h,E] fp32: gradient carry this rank's block produces with nothing coming in from
    the right.  Returns the carry entering from rank+1 (None on the last rank) after sending
    the completed carry G + exp(L) * incoming to rank-1.  One gather instead of the chain where the
    communicator offers it (see forward_chain)."""
    if hasattr(comm, "all_gather"):
        if comm.world == 1:
            return None
        Gs, Ls = comm.all_gather(G), comm.all_gather(L)
        inc = None
        for q in range(comm.world - 1, comm.rank, -1):
            inc = Gs[q].clone() if inc is None else torch.addcmul(Gs[q], inc, torch.exp(Ls[q]).unsqueeze(-1))
        return inc
    inc = None
    if comm.rank < comm.world - 1:
        inc = comm.recv(G, comm.rank + 1)
    if comm.rank > 0:
        out = G if inc is None else torch.addcmul(G, inc, torch.exp(L).unsqueeze(-1))
        comm.send(out, comm.rank - 1)
    return inc


class _SeqParallelRetention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, log_G, c, scale, comm):
        b, t, hq, d = Q.shape
        h = K.shape[2]
        n = t // c
        first, last = comm.rank == 0, comm.rank == comm.world - 1
        a, A, KT = ops.gate_prep(K, log_G, c, query_side=False)
        S, gram = ops.chunk_state(KT, None, V, c, h, key_weights=True, want_gram=True)
        del KT
        L = A.sum(dim=1)  # [b,h]
        F = ops.discumsum_fwd(S, A, carry_only=True)
        Fg = ops.gram_scan_fwd(gram, A, Q.dtype, want_full=False, want_carry=True)[3]
        C = forward_chain(comm, torch.cat([F, Fg], dim=-1), L)
        Cs = Cg = None
        if C is not None:
            E = F.shape[-1]
            Cs, Cg = C[..., :E].contiguous(), C[..., E:].contiguous()
        Z = ops.discumsum_fwd(S, A, inplace=True, carry_in=Cs)
        zhi, zlo, zfull = ops.gram_scan_fwd(gram, A, Q.dtype, want_full=True, carry_in=Cg)
        O, l = ops.chunk_out(Q, K, V, a, Z, zhi, zlo, n, c, c, 1 if first else 0, scale)
        ctx.save_for_backward(Q, K, V, log_G, a, A, O, l, Z, zhi, zlo, zfull, L)
        ctx.c, ctx.scale, ctx.comm, ctx.first, ctx.last = c, scale, comm, first, last
        return O

    @staticmethod
    def backward(ctx, dO):
        Q, K, V, log_G, a, A, O, l, Z, zhi, zlo, zfull, L = ctx.saved_tensors
        c, scale, comm, first, last = ctx.c, ctx.scale, ctx.comm, ctx.first, ctx.last
        b, t, hq, d = Q.shape
        h = K.shape[2]
        n = t // c
        dO = dO.contiguous()
        dy, dl = ops.dout_prep(O, dO, l)
        _, _, QT, QTs = ops.gate_prep(Q, log_G, c, query_side=True, mult=scale, row_scale=dl, a_in=a)
        dZ, dZg = ops.chunk_state(QT, QTs, dy, c, h, key_weights=False, want_gram=True)
        del QT, QTs
        # gradient carries: what this block sends left if nothing came from the right
        G = ops.discumsum_bwd_carry(dZ, A)
        Gg = ops.gram_scan_bwd(dZg, zfull, A, Q.dtype, want_carry=True)[3]
        inc = backward_chain(comm, torch.cat([G, Gg], dim=-1), L)
        inc_s = inc_g = None
        if inc is not None:
            E = G.shape[-1]
            inc_s, inc_g = inc[..., :E].contiguous(), inc[..., E:].contiguous()
        wdS, dA_state = ops.discumsum_bwd(dZ, Z, A, row_len=d, row_weights=True, inplace=True, carry_in=inc_s)
        ghi, glo, dA_gram = ops.gram_scan_bwd(dZg, zfull, A, Q.dtype, carry_in=inc_g)
        hi_k = n - 2 if last else n - 1
        gate_A = A if a is not None else None
        dq_state, gq = ops.expand_grad(dy, Q, Z, zhi, zlo, a, gate_A, dl, c, h, True, scale, 2.0, 1 if first else 0,
                                       n - 1)
        dk_state, wk = ops.expand_grad(V, K, wdS, ghi, glo, a, gate_A, None, c, h, False, 1.0, 1.0, 0, hi_k)
        dQ, da_q = ops.chunk_dq(Q, dO, K, V, a, dl, l, dq_state, c, scale)
        dK, dV, da_k = ops.chunk_dkv(Q, dO, K, V, wdS, a, gate_A, dl, l, dk_state, c, hi_k, scale)
        dlog_G = ops.gate_grad(da_q, gq, da_k, wk, dA_state, dA_gram, c) if log_G is not None else None
        return dQ, dK, dV, dlog_G, None, None, None


def power_retention_sequence_parallel(Q, K, V, log_G=None, deg=2, scale=None, chunk_size=None, comm=None):
    """`power_retention` for a sequence split over ranks: this rank passes its contiguous block
    of tokens (a multiple of chunk_size; rank order = sequence order) and gets its block of the
    output; gradients flow through the same chain in reverse.  `comm` defaults to the default
    torch.distributed group."""
    from .retention import _check_inputs

    if chunk_size is None:
        raise PRError("sequence-parallel retention needs a chunk_size")
    _check_inputs(Q, K, V, log_G, deg)
    t, d = Q.shape[1], Q.shape[3]
    if t % chunk_size:
        raise PRError(f"the local block ({t} tokens) must be a multiple of chunk_size={chunk_size}")
    from . import retention

    if retention.AUTO_CHUNK and deg == 2 and chunk_size < 1024:
        # as in power_retention: a small chunk is run with a multiple of it (here one that needs no padding)
        for m in range(1024 // chunk_size, 1, -1):
            if t % (m * chunk_size) == 0:
                chunk_size = m * chunk_size
                break
    comm = comm if comm is not None else DistComm()
    if log_G is not None:
        log_G = log_G.to(torch.float32).contiguous()
    scale = float(scale) if scale else 1.0 / math.sqrt(d)
    return _SeqParallelRetention.apply(Q.contiguous(), K.contiguous(), V.contiguous(), log_G, int(chunk_size), scale,
                                       comm)

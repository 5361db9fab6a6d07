"""Caller-side cache for decoding with power retention: one layer's keys, values, gates and
recurrent state, with the switch-over policy the reference's model code applies around
`power_retention_inference` (deploy/models/powercoder/kvgs_dynamic_cache.py:111-172 for the
storage, deploy/models/powercoder/modeling_powercoder.py:161-196 for the policy).

Differences from the reference's DynamicLayer, all on the storage side:

* keys, values and gates live in preallocated tensors [b, capacity, h, d] / [b, capacity, h]
  that are written in place; the reference concatenates (`torch.cat`) on every step.  The
  decode kernel reads the filled prefix `[:, :length]` of these tensors without a copy.
* tensors use the operator's own axis order [batch, token, head, feature]; the reference's
  model keeps [batch, head, token, feature] and transposes on every call.
* a pure-recurrent mode (`recurrent=True`) keeps no token cache at all: every step advances
  the state by one token and reads it in the same pass over it (the reference reaches the same
  arithmetic with switch_over_seq_len = 1, at one cache round trip per token).

Method names follow the reference's cache (`update_kv`, `update_state`, `clean_kv`,
`get_seq_length`) so that model code written against it reads the same.
"""
from __future__ import annotations

import math

import torch

from . import layout, ops
from ._lib import PRError
from .retention import power_retention_inference


class RetentionCache:
    def __init__(self, batch: int, kv_heads: int, head_dim: int, dtype=torch.bfloat16, device="cuda",
                 capacity: int = 1024, switch_over_seq_len: int | None = 1024, recurrent: bool = False):
        if head_dim != 64:
            raise PRError(f"head dim {head_dim} unsupported by the decode kernels (64 only)")
        self.b, self.h, self.d = batch, kv_heads, head_dim
        self.dtype, self.device = dtype, torch.device(device)
        self.switch_over_seq_len = switch_over_seq_len
        self.recurrent = recurrent
        self.length = 0
        self.state = None
        self.sum_of_keys = None
        self.keys = self.values = self.gatings = None
        if not recurrent:
            self._allocate(max(int(capacity), 1))

    # ------------------------------------------------------------------ storage
    def _allocate(self, capacity: int):
        mk = lambda *shape, dt: torch.empty(*shape, device=self.device, dtype=dt)
        keys = mk(self.b, capacity, self.h, self.d, dt=self.dtype)
        values = mk(self.b, capacity, self.h, self.d, dt=self.dtype)
        gatings = mk(self.b, capacity, self.h, dt=torch.float32)
        if self.length:
            keys[:, :self.length] = self.keys[:, :self.length]
            values[:, :self.length] = self.values[:, :self.length]
            gatings[:, :self.length] = self.gatings[:, :self.length]
        self.keys, self.values, self.gatings = keys, values, gatings
        self.capacity = capacity

    def get_seq_length(self) -> int:
        """Tokens cached since the last switch-over (kvgs_dynamic_cache.py:160-164)."""
        return self.length

    def update_kv(self, key_states, value_states, gate_states):
        """Appends [b, n, h, d] keys / values and [b, n, h] log gates; returns views of everything cached,
        plus the state pair, like the reference's update_kv (kvgs_dynamic_cache.py:131-148)."""
        n = key_states.shape[1]
        if self.length + n > self.capacity:
            self._allocate(max(2 * self.capacity, self.length + n))  # grows geometrically; rare once warmed up
        lo, hi = self.length, self.length + n
        self.keys[:, lo:hi] = key_states
        self.values[:, lo:hi] = value_states
        self.gatings[:, lo:hi] = gate_states
        self.length = hi
        return self.keys[:, :hi], self.values[:, :hi], self.gatings[:, :hi], self.state, self.sum_of_keys

    def update_state(self, state, sum_of_keys):
        """Stores the recurrent state pair (kvgs_dynamic_cache.py:150-158)."""
        self.state, self.sum_of_keys = state, sum_of_keys
        return self.state, self.sum_of_keys

    def clean_kv(self):
        """Forgets the cached tokens after they were compressed into the state; storage is kept."""
        self.length = 0

    # ------------------------------------------------------------------- policy
    def decode(self, q, k, v, log_g, scale: float | None = None):
        """One generated token: q [b,1,hq,d], k, v [b,1,h,d], log_g [b,1,h] fp32.  Returns y [b,1,hq,d].

        Token-cache mode applies modeling_powercoder.py:181-196: append, call the inference operator on the
        cached prefix, and when the cache has reached switch_over_seq_len compress it into the state and clear
        it.  Recurrent mode advances the state by this token and reads it (no cache)."""
        scale = 1.0 / math.sqrt(self.d) if scale is None else scale
        if self.recurrent:
            return self._decode_recurrent(q, k, v, log_g, scale)
        K, V, G, state, sok = self.update_kv(k, v, log_g)
        y, new_state, new_sok = power_retention_inference(q, K, V, G, state, sok, deg=2, scale=scale,
                                                          switch_over_seq_len=self.switch_over_seq_len)
        if self.switch_over_seq_len is not None and self.length >= self.switch_over_seq_len:
            self.clean_kv()
            self.update_state(new_state, new_sok)
        return y

    def _decode_recurrent(self, q, k, v, log_g, scale):
        hq = q.shape[2]
        if self.state is None:
            D = layout.exact_dim(self.d)
            self.state = torch.zeros(self.b, self.h, D, self.d, device=self.device, dtype=self.dtype)
            self.sum_of_keys = torch.zeros(self.b, self.h, D, device=self.device, dtype=torch.float32)
        if hq // self.h <= 4:
            new_state, new_sok = self.state, self.sum_of_keys  # every row is read and written by one thread
        else:
            new_state, new_sok = torch.empty_like(self.state), torch.empty_like(self.sum_of_keys)
        y = ops.decode_recurrent(q, k, v, log_g, self.state, self.sum_of_keys, new_state, new_sok, scale)
        self.state, self.sum_of_keys = new_state, new_sok
        return y

    def prefill(self, Q, K, V, log_G, chunk_size: int, scale: float | None = None):
        """Processes a prompt through the chunked training-path kernels and leaves the cache ready for
        decode().  The reference's model runs `power_retention` for the prompt, keeps every prompt token in
        the cache and compresses them at the first decode call (modeling_powercoder.py:198-209, :181-196);
        here the state after the prompt comes out of the same pass (return_final_state), so nothing of the
        prompt has to stay cached.  Returns Y [b,t,hq,d]."""
        from .retention import power_retention

        if self.length:
            raise PRError("prefill() wants an empty token cache: decode past the next switch-over first")
        init = (self.state, self.sum_of_keys) if self.state is not None else None
        with torch.no_grad():
            Y, (state, sok) = power_retention(Q, K, V, log_G, initial_state=init, return_final_state=True, deg=2,
                                              scale=scale, chunk_size=chunk_size)
        self.update_state(state, sok)
        self.clean_kv()
        return Y

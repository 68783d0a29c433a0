"""KV caches and ModelArgs base with the reference's constructor / field / method surface.

Mirrors mlx_parallm/models/base.py (reference):
  BatchedKVCache  42-90   (head_dim, n_kv_heads, batch_size=1); .keys .values .offset .step
                          .offsets .reset(bs) .update_and_fetch(k, v)
  PagedKVCache    93-149  adds per-row .offsets_list
  BaseModelArgs   151-161 from_dict drops unknown keys

  RowState / LatentKVCache / DeltaRuleState / TokenState: per-sequence state of layer kinds the reference does not have
                          (latent attention, gated delta rule, previous-token embedding) under the same row protocol

B200 design: one dense device buffer [B, Hkv, Tcap, D] per layer in the model's 16-bit storage type
(the reference allocates float32, base.py:111-112 -- deliberate deviation), plus a device
int32 ``lengths[B]`` the kernels read, so that a captured decode graph stays valid while rows
advance.  The model's fused kernels (b200p_rope_kv_append / b200p_attn) write and read the buffers
directly; ``update_and_fetch`` is kept for API compatibility with callers that poke the cache.
"""
from __future__ import annotations

import inspect
from dataclasses import dataclass
from typing import List, Optional

import torch


class RowState:
    """Bookkeeping every kind of per-sequence state shares: one row per live sequence, host offsets per row and a device
    int32 ``lengths[B]`` (one tensor for all layers of a generation) that the kernels read.  On its own it is the entry of
    a layer that keeps no state (for instance an attention layer that reads another layer's cache)."""

    def __init__(self, batch_size=1):
        self.batch_size = batch_size
        self.offset = 0
        self.step = 256
        self._offsets: List[int] = [0] * batch_size
        self._lengths: Optional[torch.Tensor] = None     # device int32 [B]; may be shared across layers
        self._lengths_shared = False

    @property
    def offsets(self):
        """Per-row offsets (base.py:87-90 / 141-143)."""
        return list(self._offsets)

    @property
    def offsets_list(self):
        return self._offsets

    @offsets_list.setter
    def offsets_list(self, v):
        self._offsets = list(v)
        self._sync_lengths()

    def _drop_buffers(self):
        """Forget the device buffers (the batch size changed)."""

    def buffers(self) -> tuple:
        """Device tensors a captured decode step holds pointers to."""
        return ()

    def reset(self, batch_size: int | None = None):
        """base.py:52-64 / 145-148: keep buffers when the batch size is unchanged."""
        if batch_size is not None and batch_size != self.batch_size:
            self.batch_size = batch_size
            self._drop_buffers()
            if not self._lengths_shared:
                self._lengths = None
        self.offset = 0
        self._offsets = [0] * self.batch_size
        if self._lengths is not None:
            if self._lengths.numel() != self.batch_size:
                self._lengths = None if not self._lengths_shared else torch.zeros(
                    (self.batch_size,), dtype=torch.int32, device=self._lengths.device)
            else:
                self._lengths.zero_()          # shared across layers: zeroing it from every layer is idempotent

    @property
    def capacity(self) -> int:
        return 0

    def lengths(self, device) -> torch.Tensor:
        if self._lengths is None:
            self._lengths = torch.tensor(self._offsets, dtype=torch.int32, device=device)
        return self._lengths

    def share_lengths(self, t: torch.Tensor):
        """Let every layer of one generation read (and the step advance) a single lengths tensor."""
        self._lengths = t
        self._lengths_shared = True

    def _sync_lengths(self):
        if self._lengths is not None:
            self._lengths.copy_(torch.tensor(self._offsets, dtype=torch.int32), non_blocking=False)

    def advance_host(self, L: int):
        self._offsets = [o + L for o in self._offsets]
        self.offset = max(self._offsets) if self._offsets else 0

    def advance_rows_host(self, rows: List[int], counts: List[int]):
        """Ragged step: row rows[i] took counts[i] tokens (the device lengths are advanced by the step itself)."""
        for r, n in zip(rows, counts):
            self._offsets[r] += n
        self.offset = max(self._offsets) if self._offsets else 0

    def release_rows_host(self, rows: List[int]):
        """Give rows back: their next sequence starts at position 0, which every kernel reads as "no history"."""
        for r in rows:
            self._offsets[r] = 0
        self.offset = max(self._offsets) if self._offsets else 0

    def ensure_capacity(self, needed: int, dtype, device) -> bool:
        return False


class BatchedKVCache(RowState):
    def __init__(self, head_dim, n_kv_heads, batch_size=1, value_dim=None, values_are_keys=False):
        super().__init__(batch_size)
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim
        self.value_dim = head_dim if value_dim is None else value_dim     # designs whose values are not the keys' size
        self.values_are_keys = bool(values_are_keys)                      # designs that attend over their keys: one buffer
        if self.values_are_keys and self.value_dim != head_dim:
            raise ValueError("values that are the keys have the keys' size")
        self.keys: Optional[torch.Tensor] = None
        self.values: Optional[torch.Tensor] = None

    def _drop_buffers(self):
        self.keys = None
        self.values = None

    def buffers(self) -> tuple:
        return (self.keys, self.values)

    def update_and_fetch(self, keys, values):
        """Append [B, Hkv, L, D] at each row's offset and return views up to the max end
        (base.py:66-85 / 119-140).  Compatibility path only -- the model forward does not use it."""
        B, _, L, _ = keys.shape
        assert B == self.batch_size, "KV cache batch size mismatch"
        self.ensure_capacity(max(self._offsets) + L, keys.dtype, keys.device)
        for i in range(B):
            s = self._offsets[i]
            self.keys[i, :, s:s + L] = keys[i]
            self.values[i, :, s:s + L] = values[i]
        self.advance_host(L)
        self._sync_lengths()
        m = max(self._offsets)
        return self.keys[:, :, :m], self.values[:, :, :m]

    # -- B200 internals ---------------------------------------------------------------------
    @property
    def capacity(self) -> int:
        return 0 if self.keys is None else self.keys.shape[2]

    def ensure_capacity(self, needed: int, dtype, device) -> bool:
        """Grow in ``step`` blocks (base.py:68-80 / 104-117).  Returns True if buffers were (re)allocated
        (a captured decode graph must then be rebuilt)."""
        cap = self.capacity
        if self.keys is not None and cap >= needed and self.keys.dtype == dtype:
            return False
        n_steps = (needed + self.step - 1) // self.step
        new_cap = n_steps * self.step
        if cap > 0 and self.keys is not None and self.keys.dtype == dtype:
            # growing a live cache: at least 1.5x, so a long generation re-copies its KV (and re-captures its decode graph)
            # O(log T) times instead of every ``step`` tokens (the reference concatenates a step-sized block each time,
            # base.py:104-117).  Only ONE layer's old + new buffers are alive at a time.
            new_cap = max(new_cap, ((cap * 3 // 2 + self.step - 1) // self.step) * self.step)
        nk = torch.zeros((self.batch_size, self.n_kv_heads, new_cap, self.head_dim), dtype=dtype, device=device)
        nv = nk if self.values_are_keys else torch.zeros((self.batch_size, self.n_kv_heads, new_cap, self.value_dim), dtype=dtype,
                                                          device=device)
        if self.keys is not None and cap > 0:
            keep = min(cap, max(self._offsets) if self._offsets else 0)
            if keep > 0:
                nk[:, :, :keep] = self.keys[:, :, :keep]
                if not self.values_are_keys:
                    nv[:, :, :keep] = self.values[:, :, :keep]
        self.keys, self.values = nk, nv
        return True


class LatentKVCache(RowState):
    """One low-rank vector per position that serves as key and value of every head of a latent-attention layer (and of the
    later layers that share it): ``latent [B, Tcap, rank]`` in the model's storage type, grown like the KV buffers above."""

    def __init__(self, rank, batch_size=1):
        super().__init__(batch_size)
        self.rank = rank
        self.latent: Optional[torch.Tensor] = None

    def _drop_buffers(self):
        self.latent = None

    def buffers(self) -> tuple:
        return (self.latent,)

    @property
    def capacity(self) -> int:
        return 0 if self.latent is None else self.latent.shape[1]

    def ensure_capacity(self, needed: int, dtype, device) -> bool:
        cap = self.capacity
        if self.latent is not None and cap >= needed and self.latent.dtype == dtype:
            return False
        new_cap = ((needed + self.step - 1) // self.step) * self.step
        if cap > 0 and self.latent.dtype == dtype:
            new_cap = max(new_cap, ((cap * 3 // 2 + self.step - 1) // self.step) * self.step)
        nl = torch.zeros((self.batch_size, new_cap, self.rank), dtype=dtype, device=device)
        if self.latent is not None and cap > 0 and self.latent.dtype == dtype:
            keep = min(cap, max(self._offsets) if self._offsets else 0)
            if keep > 0:
                nl[:, :keep] = self.latent[:, :keep]
        self.latent = nl
        return True


class DeltaRuleState(RowState):
    """State of a gated-delta-rule layer: per row and head the fp32 matrix ``state [B, H, dk, dv]`` and the last
    ``taps - 1`` inputs of the short convolutions ``conv [B, taps-1, C]`` (fp32).  Constant size per row; never grows."""

    def __init__(self, heads, key_dim, value_dim, conv_channels, taps, batch_size=1):
        super().__init__(batch_size)
        self.heads, self.key_dim, self.value_dim = heads, key_dim, value_dim
        self.conv_channels, self.taps = conv_channels, taps
        self.state: Optional[torch.Tensor] = None
        self.conv: Optional[torch.Tensor] = None

    def _drop_buffers(self):
        self.state = None
        self.conv = None

    def buffers(self) -> tuple:
        return (self.state, self.conv)

    def ensure_capacity(self, needed: int, dtype, device) -> bool:
        if self.state is not None:
            return False
        self.state = torch.zeros((self.batch_size, self.heads, self.key_dim, self.value_dim), dtype=torch.float32, device=device)
        self.conv = torch.zeros((self.batch_size, max(self.taps - 1, 1), self.conv_channels), dtype=torch.float32, device=device)
        return True


class ConvTailState(RowState):
    """The last ``taps - 1`` inputs of a causal convolution over time, ``conv [B, taps-1, C]`` (fp32): what a layer that
    convolves its input (or its projections) carries from step to step.  Constant size per row; never grows."""
    def __init__(self, channels, taps, batch_size=1):
        super().__init__(batch_size)
        self.channels, self.taps = channels, taps
        self.conv: Optional[torch.Tensor] = None
    def _drop_buffers(self):
        self.conv = None
    def buffers(self) -> tuple:
        return (self.conv,)
    def ensure_capacity(self, needed: int, dtype, device) -> bool:
        if self.conv is not None:
            return False
        self.conv = torch.zeros((self.batch_size, max(self.taps - 1, 1), self.channels), dtype=torch.float32, device=device)
        return True
class StateGroup(RowState):
    """The states of a layer whose mixer is several mixers side by side (say a KV cache and a matrix state): one entry of the
    cache list that owns its parts' buffers.  The parts keep no bookkeeping of their own; they follow this entry's rows."""

    def __init__(self, parts: List[RowState], batch_size=1):
        super().__init__(batch_size)
        self.parts = list(parts)

    def _follow(self):
        for p in self.parts:
            p._offsets = self._offsets
            p.step = self.step

    def _drop_buffers(self):
        for p in self.parts:
            p.batch_size = self.batch_size
            p._drop_buffers()

    def buffers(self) -> tuple:
        return tuple(b for p in self.parts for b in p.buffers())

    @property
    def capacity(self) -> int:
        return max((p.capacity for p in self.parts), default=0)

    def ensure_capacity(self, needed: int, dtype, device) -> bool:
        self._follow()
        moved = False
        for p in self.parts:
            moved |= p.ensure_capacity(needed, dtype, device)
        return moved


class TokenState(RowState):
    """The last token of every row (``last_token [B]`` int32): what an embedding that looks at the previous token needs
    when a sequence goes on in a later step."""

    def __init__(self, batch_size=1):
        super().__init__(batch_size)
        self.last_token: Optional[torch.Tensor] = None

    def _drop_buffers(self):
        self.last_token = None

    def buffers(self) -> tuple:
        return (self.last_token,)

    def ensure_capacity(self, needed: int, dtype, device) -> bool:
        if self.last_token is not None:
            return False
        self.last_token = torch.zeros((self.batch_size,), dtype=torch.int32, device=device)
        return True


class PagedKVCache(BatchedKVCache):
    """Per-sequence offsets on one dense buffer (base.py:93-149).  In this build both classes carry
    per-row device lengths, so PagedKVCache only restates the constructor for API parity."""

    def __init__(self, head_dim, n_kv_heads, batch_size=1):
        super().__init__(head_dim, n_kv_heads, batch_size)


@dataclass
class BaseModelArgs:
    @classmethod
    def from_dict(cls, params):
        return cls(**{k: v for k, v in params.items() if k in inspect.signature(cls).parameters})

"""Building blocks for decoder designs outside the Llama mould, and the ragged-batch model that runs them.

The reference has no counterpart (its graphs are models/llama.py and models/qwen3.py): these blocks carry designs whose
layers mix a recurrent state with windowed attention over a shared low-rank latent, with dense (unquantised) weights.

    Linear                  dense [out, in] weight                                 b200p_gemm
    HashedBigramEmbedding   token row * scale + a row picked by (previous, current)  b200p_embed_hashed
    GatedDeltaMixer         short convolutions + gated delta rule; decay per head   b200p_delta_prep / _conv_commit / _scan / _out
                            or per key channel, decay and gate optionally low-rank
    SinkAttention           grouped-head attention, normed q / k, distance bias,    b200p_sink_attn_prep / b200p_sink_attn
                            query temperature, a sink in the softmax
    DecayLinearAttention    S <- lambda S + k v^T with constant per-head decays      b200p_linear_attn_prep / b200p_delta_scan / _out
    SideBySideMixer         several of the above on one input, one fused in- and     b200p_gemm
                            out-projection, a scale per branch
    StateSpaceMixer         short convolution + selective state-space recurrence     b200p_ssm_prep / b200p_delta_scan / b200p_ssm_out
                            (scalar decay per head and token), gated group norm
    DifferentialAttention   grouped-head attention with two score maps per head      b200p_rope_attn_prep / b200p_diff_attn
                            whose outputs are subtracted, partial pairwise rotation,
                            position chunks
    GatedFF                 W_down (act(W_gate x) * W_up x), act in the epilogue     b200p_gemm (fused epilogue)
    ActivatedFF             W_down act(W_up x), act in the epilogue                  b200p_gemm (fused epilogue)
    RoutedExperts           top-k routed GatedFF experts + a shared one; softmax     b200p_moe_* / b200p_gemm_grouped
                            over the chosen logits, or sigmoid scores picked inside
                            the best expert groups with a gated shared expert
    LatentAttention         queries and keys/values through low-rank latents,       b200p_latent_prep / b200p_latent_attn
                            sliding window, optional sharing of another layer's latents,  b200p_latent_rope_prep / _q_rope
                            optionally a rotated key part shared by the heads
    WindowAttention         grouped-head attention without rotation over a sliding    b200p_window_attn_prep / b200p_window_attn
                            window: short convolutions on q and k, values that are the
                            keys, capped scores, logarithmic distance penalty, output gate
    ClampedGLU              g * sigmoid(1.702 g) * (u + 1) on clamped gate / up      b200p_gemm (fused epilogue)
    TokenSideInput          a small per-layer table indexed by the token, gated      b200p_token_gate
    SequenceModel           the layer chain over a ragged batch: norm -> sublayer -> norm -> residual (b200p_norm_add_norm), or
                            one norm feeding a mixer and a feed-forward that are added together, or a norm before each of the
                            two, with an optional span of layers that runs several times on the same weights
                            (b200p_residual_add_norm), or several copies of the stream that every sublayer reads as a weighted sum
                            and writes back through a mixing matrix, with a tanh norm and a short convolution on what a sublayer
                            reads (b200p_hyper_step / b200p_canon_conv)

A step is a ragged batch: entry e brings ``counts[e]`` tokens for cache row ``rows[e]``; prompts of different lengths are
packed back to back (no padding), decode steps bring one token per live row.  Every kernel works from the per-token plan
(row, position, offset in the portion), so the logits of a position do not depend on how the prompt was cut or on the
other rows.  Matrix products run in the model's storage type with fp32 accumulation; the residual stream, every norm,
softmax, the recurrence and what feeds it are fp32.  A float32 model runs true fp32 FMAs throughout.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
import math

from .._lib import (GATE_SIGMOID, GATE_SILU, GEMM_GLU_CLAMP, GEMM_GLU_GELU_TANH, GEMM_GLU_SILU, GEMM_RELU_SQ, GEMM_STORE, GEMM_STORE_F32,
                    SCAN_ACCUMULATE, SCAN_DELTA, SCAN_DELTA_CHANNEL)
from .base import BatchedKVCache, ConvTailState, DeltaRuleState, LatentKVCache, RowState, StateGroup, TokenState

MAX_TOKENS_PER_FORWARD = 8192     # packed tokens of one pass through the layers


class Linear:
    """Dense linear layer, weight [out, in] in the model's storage type, applied as W x."""

    def __init__(self, in_features: int, out_features: int):
        self.in_features, self.out_features = in_features, out_features
        self.weight: Optional[torch.Tensor] = None

    def __call__(self, x, epilogue=GEMM_STORE, out=None, limit=0.0):
        return ops.gemm(x, self.weight, epilogue, out=out, limit=limit)


class Scratch:
    """Flat per-step buffers, sized for the largest layer, handed out as [M, n] views."""

    def __init__(self, device, rows: int):
        self.device, self.rows = device, rows
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self._need: Dict[tuple, int] = {}
        self._flat: Dict[tuple, int] = {}

    def reserve(self, name: str, dtype, cols: int):
        key = (name, dtype)
        self._need[key] = max(self._need.get(key, 0), cols)

    def reserve_flat(self, name: str, dtype, n: int):
        """A buffer of n elements whatever the number of rows (per-step tables such as segment offsets)."""
        key = (name, dtype)
        self._flat[key] = max(self._flat.get(key, 0), n)

    def allocate(self):
        for key, cols in self._need.items():
            self._bufs[key] = torch.empty((self.rows * cols,), dtype=key[1], device=self.device)
        for key, n in self._flat.items():
            self._bufs[key] = torch.zeros((n,), dtype=key[1], device=self.device)

    def flat(self, name: str, dtype) -> torch.Tensor:
        return self._bufs[(name, dtype)]

    def get(self, name: str, dtype, M: int, cols: int) -> torch.Tensor:
        return self._bufs[(name, dtype)][:M * cols].view(M, cols)


def _round8(n: int) -> int:
    return (n + 7) // 8 * 8


class GatedDeltaMixer:
    """Gated delta rule with short causal convolutions on q, k and v.

    q, k: ``kv_heads`` heads of ``dim``; v: ``heads`` heads of ``vdim``; head h reads q/k head h // (heads // kv_heads).
    Per head the fp32 state S [dim, vdim] goes S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with
    g = exp(-exp(A_log) softplus(a + dt_bias)) and beta = sigmoid(b).  o is rms-normed over vdim, weighted and gated before
    the output projection.  Options (each a constructor argument):
      channel_decay  g is a vector over the key channels (one decay per row of S, ``a`` and ``dt_bias`` of heads * dim values)
                     instead of one number per head;
      decay_rank     a = W_a2 (W_a1 x) through ``decay_rank`` inner values instead of one projection (0);
      gate_rank      the gate's pre-activation likewise W_g2 (W_g1 x) (0: one projection);
      gate_act       "silu" or "sigmoid".
    Ranks given as None are read from the tensors when the weights are loaded (``set_ranks``)."""

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 channel_decay: bool = False, decay_rank: Optional[int] = 0, gate_rank: Optional[int] = 0, gate_act: str = "silu"):
        self.width, self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.eps = width, heads, kv_heads, dim, vdim, taps, eps
        self.channel_decay = channel_decay
        self.gate_act = {"silu": GATE_SILU, "sigmoid": GATE_SIGMOID}[gate_act]
        self.c_qk = kv_heads * dim
        self.c_v = heads * vdim
        self.n_decay = heads * (dim if channel_decay else 1)
        self.conv_channels = 2 * self.c_qk + self.c_v
        self.col_b = self.conv_channels
        self.col_g = self.col_b + heads
        self.o_proj = Linear(self.c_v, width)
        self.conv_w = self.A_log = self.dt_bias = self.norm_w = None     # fp32
        self.decay_rank = self.gate_rank = None
        self.in_proj = self.decay_up = self.gate_up = None
        if decay_rank is not None and gate_rank is not None:
            self.set_ranks(decay_rank, gate_rank)

    def set_ranks(self, decay_rank: int, gate_rank: int):
        """Lay out the fused input projection: rows [q | k | v | b | gate part | decay part]; a low-rank part holds the inner
        values (the gate's padded to a multiple of 8 columns so that the decay's start on a 16-byte boundary)."""
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.n_g = _round8(gate_rank) if gate_rank else self.c_v
        self.col_a = self.col_g + self.n_g
        self.n_proj = self.col_a + (decay_rank if decay_rank else self.n_decay)
        self.in_proj = Linear(self.width, self.n_proj)
        self.gate_up = Linear(gate_rank, self.c_v) if gate_rank else None
        self.decay_up = Linear(decay_rank, self.n_decay) if decay_rank else None

    def stack_in_proj(self, q, k, v, b, gate, decay):
        """The fused weight from its parts (``gate`` / ``decay``: the first-stage matrices when they are low-rank)."""
        parts = [q, k, v, b, gate]
        if self.n_g != gate.shape[0]:
            parts.append(torch.zeros((self.n_g - gate.shape[0], gate.shape[1]), dtype=gate.dtype))
        return torch.cat(parts + [decay], 0)

    def new_state(self, batch_size: int) -> RowState:
        return DeltaRuleState(self.heads, self.dim, self.vdim, self.conv_channels, self.taps, batch_size)

    def reserve(self, s: Scratch, dt):
        s.reserve("proj", torch.float32, self.n_proj)
        s.reserve("qn", torch.float32, self.c_qk)
        s.reserve("kn", torch.float32, self.c_qk)
        s.reserve("v", torch.float32, self.c_v)
        s.reserve("beta", torch.float32, self.heads)
        s.reserve("decay", torch.float32, self.n_decay)
        s.reserve("o", torch.float32, self.c_v)
        s.reserve("mix", dt, self.c_v)
        if self.gate_rank or self.decay_rank:
            s.reserve("inner", dt, self.n_proj - self.col_g)
        if self.gate_rank:
            s.reserve("gate", torch.float32, self.c_v)
        if self.decay_rank:
            s.reserve("step", torch.float32, self.n_decay)

    def __call__(self, x, y_out, st: DeltaRuleState, plan: dict, s: Scratch, caches):
        M, dt, f32 = x.shape[0], x.dtype, torch.float32
        proj = self.in_proj(x, GEMM_STORE_F32, out=s.get("proj", f32, M, self.n_proj))
        gate, step = proj[:, self.col_g:self.col_g + self.c_v], proj[:, self.col_a:self.col_a + self.n_decay]
        if self.gate_rank or self.decay_rank:
            # second stage of the low-rank parts: the inner values go through the GEMM in the model's storage type
            inner = proj[:, self.col_g:]
            if dt != f32:
                inner = s.get("inner", dt, M, self.n_proj - self.col_g)
                ops.cast_columns(proj[:, self.col_g:], inner)
            if self.gate_rank:
                gate = self.gate_up(inner[:, :self.gate_rank], GEMM_STORE_F32, out=s.get("gate", f32, M, self.c_v))
            if self.decay_rank:
                a0 = self.col_a - self.col_g
                step = self.decay_up(inner[:, a0:a0 + self.decay_rank], GEMM_STORE_F32, out=s.get("step", f32, M, self.n_decay))
        qn, kn = s.get("qn", f32, M, self.c_qk), s.get("kn", f32, M, self.c_qk)
        v, o = s.get("v", f32, M, self.c_v), s.get("o", f32, M, self.c_v)
        beta, decay = s.get("beta", f32, M, self.heads), s.get("decay", f32, M, self.n_decay)
        ops.delta_prep(proj, self.col_b, step, self.conv_w, st.conv, self.A_log, self.dt_bias, plan["t_row"], plan["t_pos"],
                       plan["t_off"], qn, kn, v, beta, decay, self.heads, self.kv_heads, self.dim, self.vdim, self.taps)
        ops.delta_conv_commit(proj, st.conv, plan["cu"], plan["rows"], plan["nb"], self.conv_channels, self.taps)
        ops.delta_scan(qn, kn, v, beta, decay, st.state, plan["cu"], plan["rows"], plan["lengths"], o, plan["nb"], self.heads,
                       self.kv_heads, self.dim, self.vdim, SCAN_DELTA_CHANNEL if self.channel_decay else SCAN_DELTA)
        mix = s.get("mix", dt, M, self.c_v)
        ops.delta_out(o, gate, self.norm_w, mix, self.heads, self.vdim, self.eps, self.gate_act)
        return self.o_proj(mix, GEMM_STORE_F32, out=y_out)


class SinkAttention:
    """A branch of ``SideBySideMixer``: causal attention with ``heads`` query heads over ``kv_heads`` key/value heads (query
    head h reads h // (heads // kv_heads)), keys of ``dim`` and values of ``vdim``, no rotation.  q and k are rms-normed per
    head (weights shared by the heads; ``qk_norm`` False: not at all); q at position p is multiplied by
    1 + temp_coef ln(floor((p + 1) / temp_every) + 1); score = q . k * scale - slope_h (i - j) with
    slope_h = 2^(slope_log2 (h + 1) / heads) (0: no bias); the softmax denominator also holds exp(sink_h) (``sink`` False:
    none).  Projection columns [q | k | v]; K and V are cached per position."""

    def __init__(self, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float, qk_norm: bool = True,
                 temp_coef: float = 0.0, temp_every: float = 1.0, slope_log2: float = 0.0, sink: bool = True):
        self.heads, self.kv_heads, self.dim, self.vdim, self.scale, self.eps = heads, kv_heads, dim, vdim, scale, eps
        self.qk_norm, self.temp_coef, self.temp_every, self.slope_log2, self.has_sink = qk_norm, temp_coef, temp_every, slope_log2, sink
        self.col_k = heads * dim
        self.col_v = self.col_k + kv_heads * dim
        self.n_proj = self.col_v + kv_heads * vdim
        self.n_mix = heads * vdim
        self.q_norm_w = self.k_norm_w = self.sink = None      # fp32

    def new_state(self, batch_size: int) -> RowState:
        return BatchedKVCache(self.dim, self.kv_heads, batch_size, value_dim=self.vdim)

    DECODE_WS_ROWS = 256          # decode batches up to this size get the full split of their keys over CTAs, larger ones fewer

    def reserve(self, s: Scratch, dt):
        s.reserve("aq", torch.float32, self.heads * self.dim)
        if dt != torch.float32:
            s.reserve_flat("attn_ws", torch.float32, ops.sink_attn_workspace_floats(min(s.rows, self.DECODE_WS_ROWS), self.heads, self.vdim))

    def core(self, proj, mix_out, out_scale: float, st: BatchedKVCache, plan: dict, s: Scratch):
        M = proj.shape[0]
        q = s.get("aq", torch.float32, M, self.heads * self.dim)
        ops.sink_attn_prep(proj, 0, self.col_k, self.col_v, self.q_norm_w, self.k_norm_w, self.eps, self.scale, self.temp_coef,
                           self.temp_every, q, st.keys, st.values, plan["t_row"], plan["t_pos"], self.heads, self.kv_heads, self.dim,
                           self.vdim)
        ops.sink_attn(q, st.keys, st.values, plan["t_row"], plan["t_pos"], self.sink, self.slope_log2, mix_out, self.heads,
                      self.kv_heads, self.dim, self.vdim, out_scale, cu=plan["cu"], rows=plan["rows"], nb=plan["nb"],
                      max_n=plan["max_n"], workspace=s.flat("attn_ws", torch.float32) if proj.dtype != mix_out.dtype else None)


class DecayLinearAttention:
    """A branch of ``SideBySideMixer``: linear attention with a constant decay per head.  q, k (``heads`` x ``dim``) and v
    (``heads`` x ``vdim``) are silu of their projections; per head the fp32 state S [dim, vdim] goes S <- decay_h S + k v^T,
    o = S^T q.  All heads are rms-normed as ONE vector (weight of heads * vdim values), gated by sigmoid of a fourth
    projection.  Projection columns [q | k | v | gate]."""

    def __init__(self, heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float):
        if len(decay) != heads:
            raise ValueError("one decay per head")
        self.heads, self.dim, self.vdim, self.decay_values, self.eps = heads, dim, vdim, [float(d) for d in decay], eps
        self.c_qk, self.c_v = heads * dim, heads * vdim
        self.col_g = 2 * self.c_qk + self.c_v
        self.n_proj = self.col_g + self.c_v
        self.n_mix = self.c_v
        self.norm_w = self.decay = None                         # fp32

    def new_state(self, batch_size: int) -> RowState:
        return DeltaRuleState(self.heads, self.dim, self.vdim, 1, 1, batch_size)

    def reserve(self, s: Scratch, dt):
        s.reserve("qn", torch.float32, self.c_qk)
        s.reserve("kn", torch.float32, self.c_qk)
        s.reserve("v", torch.float32, self.c_v)
        s.reserve("decay", torch.float32, self.heads)
        s.reserve("o", torch.float32, self.c_v)

    def core(self, proj, mix_out, out_scale: float, st: DeltaRuleState, plan: dict, s: Scratch):
        M, f32 = proj.shape[0], torch.float32
        qn, kn = s.get("qn", f32, M, self.c_qk), s.get("kn", f32, M, self.c_qk)
        v, o, decay = s.get("v", f32, M, self.c_v), s.get("o", f32, M, self.c_v), s.get("decay", f32, M, self.heads)
        ops.linear_attn_prep(proj, self.decay, qn, kn, v, decay, self.heads, self.dim, self.vdim)
        ops.delta_scan(qn, kn, v, None, decay, st.state, plan["cu"], plan["rows"], plan["lengths"], o, plan["nb"], self.heads,
                       self.heads, self.dim, self.vdim, SCAN_ACCUMULATE)
        ops.delta_out(o, proj[:, self.col_g:self.col_g + self.c_v], self.norm_w, mix_out, 1, self.c_v, self.eps, GATE_SIGMOID, out_scale)


class SideBySideMixer:
    """Several mixers that read the same input, y = sum_i scale_i * W_o,i branch_i(x): ONE input projection of all their
    columns and ONE output projection over their concatenated outputs (each branch scales its output by scale_i before it is
    rounded to the storage type).  A branch offers n_proj, n_mix, new_state, reserve and
    core(projection columns, output columns, scale, state, plan, scratch)."""

    def __init__(self, width: int, branches: Sequence, scales: Sequence[float]):
        self.width, self.branches, self.scales = width, list(branches), [float(c) for c in scales]
        self.col0, self.mix0 = [], []
        n = k = 0
        for b in self.branches:
            self.col0.append(n)
            self.mix0.append(k)
            n += _round8(b.n_proj)             # every branch's columns start on a 32-byte boundary of the fp32 projection
            k += _round8(b.n_mix)
        self.n_proj, self.n_mix = n, k
        self.in_proj = Linear(width, n)
        self.o_proj = Linear(k, width)

    def stack_in_proj(self, parts: Sequence[torch.Tensor]) -> torch.Tensor:
        rows = []
        for b, w in zip(self.branches, parts):
            rows.append(w)
            if _round8(b.n_proj) != w.shape[0]:
                rows.append(torch.zeros((_round8(b.n_proj) - w.shape[0], w.shape[1]), dtype=w.dtype))
        return torch.cat(rows, 0)

    def stack_o_proj(self, parts: Sequence[torch.Tensor]) -> torch.Tensor:
        cols = []
        for b, w in zip(self.branches, parts):
            cols.append(w)
            if _round8(b.n_mix) != w.shape[1]:
                cols.append(torch.zeros((w.shape[0], _round8(b.n_mix) - w.shape[1]), dtype=w.dtype))
        return torch.cat(cols, 1)

    def new_state(self, batch_size: int) -> RowState:
        return StateGroup([b.new_state(batch_size) for b in self.branches], batch_size)

    def reserve(self, s: Scratch, dt):
        s.reserve("proj", torch.float32, self.n_proj)
        s.reserve("mix", dt, self.n_mix)
        for b in self.branches:
            b.reserve(s, dt)

    def __call__(self, x, y_out, st: StateGroup, plan: dict, s: Scratch, caches):
        M, dt = x.shape[0], x.dtype
        proj = self.in_proj(x, GEMM_STORE_F32, out=s.get("proj", torch.float32, M, self.n_proj))
        mix = s.get("mix", dt, M, self.n_mix)
        if any(_round8(b.n_mix) != b.n_mix for b in self.branches):
            mix.zero_()                                        # padding columns meet zero weights, but must not hold NaN
        for b, c0, m0, scale, part in zip(self.branches, self.col0, self.mix0, self.scales, st.parts):
            b.core(proj[:, c0:c0 + b.n_proj], mix[:, m0:m0 + b.n_mix], scale, part, plan, s)
        return self.o_proj(mix, GEMM_STORE_F32, out=y_out)


class StateSpaceMixer:
    """Selective state-space layer with a scalar decay per head and token.  One projection gives [z | x | B | C | dt]
    (inner = heads * vdim channels of z and x, groups * state of B and C, heads of dt).  x, B, C pass a causal convolution of
    ``taps`` taps with bias and silu; dt = softplus(dt + dt_bias).  Per head (reading the B / C of group h // (heads // groups))
    the fp32 state S [state, vdim] goes S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x.  Then y * silu(z), an rms norm
    over each of ``norm_groups`` equal runs of the channels, a weight per channel, the output projection.  The recurrence is the
    plain-accumulation mode of the delta-rule scan (k = B, q = C, v = dt x)."""

    def __init__(self, width: int, heads: int, vdim: int, state: int, groups: int, norm_groups: int, taps: int, eps: float):
        if heads % groups or (heads * vdim) % norm_groups:
            raise ValueError("heads must be a multiple of groups and the channels a multiple of norm_groups")
        self.width, self.heads, self.vdim, self.state, self.groups, self.norm_groups = width, heads, vdim, state, groups, norm_groups
        self.taps, self.eps = taps, eps
        self.inner = heads * vdim
        self.c_bc = groups * state
        self.conv_channels = self.inner + 2 * self.c_bc
        self.col_x = self.inner
        self.col_dt = self.inner + self.conv_channels
        self.n_proj = self.col_dt + heads
        self.in_proj = Linear(width, self.n_proj)
        self.o_proj = Linear(self.inner, width)
        self.conv_w = self.conv_b = self.A_log = self.dt_bias = self.D = self.norm_w = None      # fp32

    def new_state(self, batch_size: int) -> RowState:
        return DeltaRuleState(self.heads, self.state, self.vdim, self.conv_channels, self.taps, batch_size)

    def reserve(self, s: Scratch, dt):
        s.reserve("proj", torch.float32, self.n_proj)
        s.reserve("qn", torch.float32, self.c_bc)
        s.reserve("kn", torch.float32, self.c_bc)
        s.reserve("v", torch.float32, self.inner)
        s.reserve("xs", torch.float32, self.inner)
        s.reserve("decay", torch.float32, self.heads)
        s.reserve("o", torch.float32, self.inner)
        s.reserve("mix", dt, self.inner)

    def __call__(self, x, y_out, st: DeltaRuleState, plan: dict, s: Scratch, caches):
        M, dt, f32 = x.shape[0], x.dtype, torch.float32
        proj = self.in_proj(x, GEMM_STORE_F32, out=s.get("proj", f32, M, self.n_proj))
        qn, kn = s.get("qn", f32, M, self.c_bc), s.get("kn", f32, M, self.c_bc)
        v, xs, o = s.get("v", f32, M, self.inner), s.get("xs", f32, M, self.inner), s.get("o", f32, M, self.inner)
        decay = s.get("decay", f32, M, self.heads)
        ops.ssm_prep(proj, self.col_x, self.col_dt, self.conv_w, self.conv_b, st.conv, self.A_log, self.dt_bias, plan["t_row"],
                     plan["t_pos"], plan["t_off"], xs, v, kn, qn, decay, self.heads, self.vdim, self.groups, self.state, self.taps)
        ops.delta_conv_commit(proj[:, self.col_x:self.col_dt], st.conv, plan["cu"], plan["rows"], plan["nb"], self.conv_channels, self.taps)
        ops.delta_scan(qn, kn, v, None, decay, st.state, plan["cu"], plan["rows"], plan["lengths"], o, plan["nb"], self.heads,
                       self.groups, self.state, self.vdim, SCAN_ACCUMULATE)
        mix = s.get("mix", dt, M, self.inner)
        ops.ssm_out(o, xs, proj[:, :self.inner], self.D, self.norm_w, mix, self.heads, self.vdim, self.norm_groups, self.eps)
        return self.o_proj(mix, GEMM_STORE_F32, out=y_out)


def rotary_rates(dims: int, base: float, scaling: Optional[dict] = None) -> List[float]:
    """Angle per position of the pairs (2i, 2i+1), i < dims / 2: f_i = base^(-2i / dims).  ``scaling`` (factor, low, high,
    original) slows the long wavelengths down: with l = 2 pi / f, f stays where l < original / high, becomes f / factor where
    l > original / low, and is blended linearly in between by s = (original / l - low) / (high - low)."""
    rates = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return rates
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for f in rates:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            blend = (original / wavelength - low) / (high - low)
            out.append((1.0 - blend) * f / factor + blend * f)
    return out


class DifferentialAttention:
    """Causal attention with ``heads`` query heads over ``kv_heads`` key/value heads and ``maps`` (1 or 2) score maps per head:
    q holds heads x maps vectors of ``dim``, k kv_heads x maps, v kv_heads vectors of ``vdim``; every map is a softmax attention
    over the same values and the head's output is a_1 - lam a_2 (one ``lam`` per layer; maps == 1: a_1), divided by its root
    mean square over vdim (``unit_norm``) and multiplied by ``post``.  The first ``len(rates) * 2`` dimensions of every q / k
    vector are rotated pairwise (2i with 2i+1) by position * rates[i]; score = q . k * scale; position i sees j <= i with
    floor(i / chunk) == floor(j / chunk) (``chunk`` 0: every j <= i).  Projection columns [q | k | v]; rotated keys and the
    values are cached per position."""

    DECODE_WS_ROWS = 256

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float, maps: int = 2,
                 rates: Sequence[float] = (), chunk: int = 0, lam: float = 0.0, post: float = 1.0, unit_norm: bool = True):
        if heads % kv_heads or maps not in (1, 2) or 2 * len(rates) > dim:
            raise ValueError("heads must be a multiple of kv_heads, maps 1 or 2, and the rotated dimensions at most dim")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim, self.scale, self.eps = width, heads, kv_heads, dim, vdim, scale, eps
        self.maps, self.rate_values, self.chunk, self.lam, self.post, self.unit_norm = maps, [float(r) for r in rates], int(chunk), lam, post, unit_norm
        self.col_k = heads * maps * dim
        self.col_v = self.col_k + kv_heads * maps * dim
        self.n_proj = self.col_v + kv_heads * vdim
        self.n_mix = heads * vdim
        self.in_proj = Linear(width, self.n_proj)
        self.o_proj = Linear(self.n_mix, width)
        self.rates: Optional[torch.Tensor] = None             # fp32 on the device

    def set_lambda(self, lq1, lk1, lq2, lk2, offset: float):
        """lam = exp(lq1 . lk1) - exp(lq2 . lk2) + offset, from the layer's four vectors."""
        f = lambda a, b: math.exp(float((a.double() * b.double()).sum()))
        self.lam = f(lq1, lk1) - f(lq2, lk2) + float(offset)

    def new_state(self, batch_size: int) -> RowState:
        return BatchedKVCache(self.maps * self.dim, self.kv_heads, batch_size, value_dim=self.vdim)

    def reserve(self, s: Scratch, dt):
        s.reserve("proj", torch.float32, self.n_proj)
        s.reserve("aq", torch.float32, self.col_k)
        s.reserve("mix", dt, self.n_mix)
        n = ops.diff_attn_workspace_floats(min(s.rows, self.DECODE_WS_ROWS), self.heads, self.maps, self.vdim)
        if dt != torch.float32 and n:
            s.reserve_flat("attn_ws", torch.float32, n)

    def __call__(self, x, y_out, st: BatchedKVCache, plan: dict, s: Scratch, caches):
        M, dt, f32 = x.shape[0], x.dtype, torch.float32
        proj = self.in_proj(x, GEMM_STORE_F32, out=s.get("proj", f32, M, self.n_proj))
        q = s.get("aq", f32, M, self.col_k)
        ops.rope_attn_prep(proj, 0, self.col_k, self.col_v, self.rates, 2 * len(self.rate_values), self.scale, q, st.keys, st.values,
                           plan["t_row"], plan["t_pos"], self.heads, self.kv_heads, self.maps, self.dim, self.vdim)
        mix = s.get("mix", dt, M, self.n_mix)
        ws = s.flat("attn_ws", f32) if (dt != f32 and ("attn_ws", f32) in s._bufs) else None
        ops.diff_attn(q, st.keys, st.values, plan["t_row"], plan["t_pos"], mix, self.heads, self.kv_heads, self.maps, self.dim, self.vdim,
                      chunk=self.chunk, lam=self.lam, eps=self.eps if self.unit_norm else -1.0, post=self.post, cu=plan["cu"],
                      rows=plan["rows"], nb=plan["nb"], max_n=plan["max_n"], workspace=ws)
        return self.o_proj(mix, GEMM_STORE_F32, out=y_out)


class LatentAttention:
    """Attention whose queries and keys/values pass through low-rank latents; no positional rotation.

    c_q = rms_norm(W_dq x); q = W_uq c_q (``heads`` x ``dim``).  c = rms_norm(W_dkv x) (``kv_rank``) is the only thing cached;
    k = W_uk c, v = W_uv c per head.  Here the up-projections are folded around the attention: the query is carried into
    the latent space (W_uk^T q per head), the heads attend over c itself, and W_uv is applied to the attended latent.
    ``window`` > 0: position i sees j with 0 <= i - j < window.  ``kv_from``: index of the earlier layer whose latents this
    layer reads (it then has no W_dkv of its own).

    ``rot_dim`` > 0: every head's query is [dim unrotated | rot_dim rotated] and W_dkv has rot_dim more rows, one rotated key
    part that all heads share; the pairs (2i, 2i+1) of the rotated parts turn by position * rates[i] and are multiplied by
    ``mag``; score = (q_unrotated . k_unrotated + q_rotated . k_rotated) * scale.  The cache row is then
    [latent | rotated key part | zeros up to a multiple of 32] and the query row in latent space [W_uk^T q | rotated q | zeros], so
    the same attention kernels score and attend over whole rows; W_uv reads the first kv_rank columns of the attended row."""

    def __init__(self, width: int, heads: int, dim: int, vdim: int, q_rank: int, kv_rank: int, scale: float, window: int,
                 eps: float, kv_from: Optional[int] = None, rot_dim: int = 0, rates: Sequence[float] = (), mag: float = 1.0):
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.q_rank, self.kv_rank, self.scale, self.window, self.eps, self.kv_from = q_rank, kv_rank, scale, window, eps, kv_from
        self.own_kv = kv_from is None
        self.rot_dim, self.rate_values, self.mag = int(rot_dim), [float(r) for r in rates], float(mag)
        if self.rot_dim:
            if kv_from is not None or self.rot_dim % 2 or 2 * len(self.rate_values) != self.rot_dim:
                raise ValueError("a rotated key part needs the layer's own latents, an even size and one rate per pair")
        self.row = (kv_rank + self.rot_dim + 31) // 32 * 32 if self.rot_dim else kv_rank      # values per cache row
        self.rates: Optional[torch.Tensor] = None         # fp32 on the device
        self.down = Linear(width, q_rank + (kv_rank + self.rot_dim if self.own_kv else 0))      # rows [dq | dkv]
        self.uq = Linear(q_rank, heads * (dim + self.rot_dim))
        self.uk_t: Optional[torch.Tensor] = None          # [heads, kv_rank, dim]: W_uk per head, transposed
        self.uv: Optional[torch.Tensor] = None            # [heads * vdim, kv_rank]
        self.o_proj = Linear(heads * vdim, width)
        self.q_norm_w = self.kv_norm_w = None             # fp32

    def new_state(self, batch_size: int) -> RowState:
        return LatentKVCache(self.row, batch_size) if self.own_kv else RowState(batch_size)

    def reserve(self, s: Scratch, dt):
        s.reserve("proj", torch.float32, self.down.out_features)
        s.reserve("cq", dt, self.q_rank)
        s.reserve("q", dt, self.heads * (self.dim + self.rot_dim))
        s.reserve("qlat", torch.float32, self.heads * self.row)
        s.reserve("olat", dt, self.heads * self.row)
        s.reserve("mix", dt, self.heads * self.vdim)

    def __call__(self, x, y_out, st: RowState, plan: dict, s: Scratch, caches):
        M, dt, f32 = x.shape[0], x.dtype, torch.float32
        H, R, dk, dv = self.heads, self.kv_rank, self.dim, self.vdim
        proj = self.down(x, GEMM_STORE_F32, out=s.get("proj", f32, M, self.down.out_features))
        cq = s.get("cq", dt, M, self.q_rank)
        if self.rot_dim:
            dr, row = self.rot_dim, self.row
            ops.latent_rope_prep(proj, self.q_rank, R, dr, self.q_norm_w, self.kv_norm_w, self.eps, self.rates, self.mag, cq, st.latent,
                                 plan["t_row"], plan["t_pos"])
            q = self.uq(cq, GEMM_STORE, out=s.get("q", dt, M, H * (dk + dr)))
            qlat = s.get("qlat", f32, M, H * row)
            ops.gemm(q, self.uk_t, GEMM_STORE_F32, out=qlat, batch=H, strides=(dk + dr, R * dk, row), M=M, N=R, K=dk, ldx=H * (dk + dr),
                     ldw=dk, ldy=H * row)
            ops.latent_q_rope(q, H, dk, dr, R, self.rates, self.mag, plan["t_pos"], qlat)
            olat = s.get("olat", dt, M, H * row)
            ops.latent_attn(qlat, st.latent, plan["t_row"], plan["t_pos"], olat, H, row, self.window, self.scale, cu=plan["cu"],
                            rows=plan["rows"], nb=plan["nb"], max_n=plan["max_n"])
            mix = s.get("mix", dt, M, H * dv)
            ops.gemm(olat, self.uv, GEMM_STORE, out=mix, batch=H, strides=(row, dv * R, dv), M=M, N=dv, K=R, ldx=H * row, ldw=R, ldy=H * dv)
            return self.o_proj(mix, GEMM_STORE_F32, out=y_out)
        cache = st if self.own_kv else caches[self.kv_from]
        ops.latent_prep(proj, self.q_rank, R, self.q_norm_w, self.kv_norm_w, self.eps, cq, cache.latent if self.own_kv else None,
                        plan["t_row"], plan["t_pos"])
        q = self.uq(cq, GEMM_STORE, out=s.get("q", dt, M, H * dk))
        qlat = s.get("qlat", f32, M, H * R)
        ops.gemm(q, self.uk_t, GEMM_STORE_F32, out=qlat, batch=H, strides=(dk, R * dk, R), M=M, N=R, K=dk, ldx=H * dk, ldw=dk,
                 ldy=H * R)
        olat = s.get("olat", dt, M, H * R)
        ops.latent_attn(qlat, cache.latent, plan["t_row"], plan["t_pos"], olat, H, R, self.window, self.scale, cu=plan["cu"],
                        rows=plan["rows"], nb=plan["nb"], max_n=plan["max_n"])
        mix = s.get("mix", dt, M, H * dv)
        ops.gemm(olat, self.uv, GEMM_STORE, out=mix, batch=H, strides=(R, dv * R, dv), M=M, N=dv, K=R, ldx=H * R, ldw=R, ldy=H * dv)
        return self.o_proj(mix, GEMM_STORE_F32, out=y_out)


class WindowAttention:
    """Causal attention without rotation: ``heads`` query heads over ``kv_heads`` key heads of ``dim`` (query head h reads
    h // (heads // kv_heads)); the values are the keys, so one buffer is cached.  q and k pass a causal convolution of ``taps``
    taps over time right after their projections (the last taps - 1 projected values of a sequence are carried as state).
    score = q . k * scale; ``softcap`` > 0: score <- softcap tanh(score / softcap); ``distance_penalty``: minus
    r1_h ln(1 + r2_h (i - j)) with two numbers per head; ``window`` > 0: position i sees j with 0 <= i - j < window; softmax;
    ``gated``: the heads' outputs are multiplied by sigmoid(W_g x) before the output projection.  Projection rows [q | k | gate]."""

    DECODE_WS_ROWS = 256

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, scale: float, taps: int = 1, softcap: float = 0.0,
                 window: int = 0, distance_penalty: bool = False, gated: bool = False):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.width, self.heads, self.kv_heads, self.dim, self.scale, self.taps = width, heads, kv_heads, dim, float(scale), int(taps)
        self.softcap, self.window, self.distance_penalty, self.gated = float(softcap), int(window), bool(distance_penalty), bool(gated)
        self.conv_channels = (heads + kv_heads) * dim
        self.n_mix = heads * dim
        self.col_g = self.conv_channels
        self.n_proj = self.conv_channels + (self.n_mix if gated else 0)
        self.in_proj = Linear(width, self.n_proj)
        self.o_proj = Linear(self.n_mix, width)
        self.conv_w = self.r1 = self.r2 = None                 # fp32; the taps tap by tap: [taps, (heads + kv_heads) * dim]

    def new_state(self, batch_size: int) -> RowState:
        return StateGroup([BatchedKVCache(self.dim, self.kv_heads, batch_size, values_are_keys=True),
                           ConvTailState(self.conv_channels, self.taps, batch_size)], batch_size)

    def reserve(self, s: Scratch, dt):
        s.reserve("proj", torch.float32, self.n_proj)
        s.reserve("aq", torch.float32, self.n_mix)
        s.reserve("mix", dt, self.n_mix)
        if dt != torch.float32:
            s.reserve_flat("attn_ws", torch.float32, ops.sink_attn_workspace_floats(min(s.rows, self.DECODE_WS_ROWS), self.heads, self.dim))

    def __call__(self, x, y_out, st: StateGroup, plan: dict, s: Scratch, caches):
        M, dt, f32 = x.shape[0], x.dtype, torch.float32
        kv, tail = st.parts
        proj = self.in_proj(x, GEMM_STORE_F32, out=s.get("proj", f32, M, self.n_proj))
        q = s.get("aq", f32, M, self.n_mix)
        ops.window_attn_prep(proj, 0, self.conv_w, tail.conv, self.taps, self.scale, q, kv.keys, plan["t_row"], plan["t_pos"], plan["t_off"],
                             self.heads, self.kv_heads, self.dim)
        if self.taps > 1:
            ops.delta_conv_commit(proj, tail.conv, plan["cu"], plan["rows"], plan["nb"], self.conv_channels, self.taps)
        mix = s.get("mix", dt, M, self.n_mix)
        ops.window_attn(q, kv.keys, kv.keys, plan["t_row"], plan["t_pos"], mix, self.heads, self.kv_heads, self.dim, self.dim,
                        softcap=self.softcap, r1=self.r1 if self.distance_penalty else None, r2=self.r2 if self.distance_penalty else None,
                        window=self.window, gate=proj[:, self.col_g:] if self.gated else None, cu=plan["cu"], rows=plan["rows"],
                        nb=plan["nb"], max_n=plan["max_n"], workspace=s.flat("attn_ws", f32) if dt != f32 else None)
        return self.o_proj(mix, GEMM_STORE_F32, out=y_out)


class GatedFF:
    """Feed-forward y = W_down (act(W_gate x) * W_up x) with the gated unit computed in the GEMM epilogue; gate and up rows are
    interleaved in one matrix so that the epilogue holds both values of a hidden unit.  ``act``: "gelu_tanh", "silu", or
    "clamped" (g * sigmoid(1.702 g) * (u + 1) on g = min(gate, limit), u = clamp(up, -limit, limit))."""

    EPILOGUES = {"gelu_tanh": GEMM_GLU_GELU_TANH, "silu": GEMM_GLU_SILU, "clamped": GEMM_GLU_CLAMP}

    def __init__(self, width: int, ff: int, act: str, limit: float = 0.0):
        self.width, self.ff, self.limit = width, ff, limit
        self.epilogue = self.EPILOGUES[act]
        self.gate_up = Linear(width, 2 * ff)
        self.down = Linear(ff, width)

    @staticmethod
    def interleave(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """rows g0 u0 g1 u1 .. from [ff, width] gate and up."""
        return torch.stack([gate, up], 1).reshape(2 * gate.shape[0], gate.shape[1])

    def reserve(self, s: Scratch, dt):
        s.reserve("act", dt, self.ff)

    def __call__(self, x, y_out, s: Scratch):
        act = self.gate_up(x, self.epilogue, out=s.get("act", x.dtype, x.shape[0], self.ff), limit=self.limit)
        return self.down(act, GEMM_STORE_F32, out=y_out)


class ClampedGLU(GatedFF):
    def __init__(self, width: int, ff: int, limit: float):
        super().__init__(width, ff, "clamped", limit)


class ActivatedFF:
    """Ungated feed-forward y = W_down act(W_up x) with the activation in the GEMM epilogue; ``act``: "relu_squared"."""

    EPILOGUES = {"relu_squared": GEMM_RELU_SQ}

    def __init__(self, width: int, ff: int, act: str):
        self.width, self.ff = width, ff
        self.epilogue = self.EPILOGUES[act]
        self.up = Linear(width, ff)
        self.down = Linear(ff, width)

    def reserve(self, s: Scratch, dt):
        s.reserve("act", dt, self.ff)

    def __call__(self, x, y_out, s: Scratch):
        act = self.up(x, self.epilogue, out=s.get("act", x.dtype, x.shape[0], self.ff))
        return self.down(act, GEMM_STORE_F32, out=y_out)


class RoutedExperts:
    """Mixture of ``experts`` GatedFF experts of which every token uses ``top``; y = sum of the chosen experts' weighted
    outputs, plus a shared expert (``shared_ff`` > 0) that every token uses.  Two ways to choose (``scoring``):
      "softmax"  router logits W_r x + b in fp32, the ``top`` largest chosen, their weights the softmax over the chosen logits;
      "sigmoid"  scores s = sigmoid(W_r x); experts are picked by s + correction (a vector per layer) among the experts of the
                 ``groups[1]`` best of ``groups[0]`` equal groups of neighbouring experts (a group's score: the sum of its two
                 largest picking scores); weights s / sum(chosen s) * ``route_scale``.
      "scores"   the ``top`` largest s = sigmoid(W_r x) chosen, their weights those scores as they are.
    ``weight_on`` "input": the weight multiplies what the expert reads, y = sum expert_k(w_k x), instead of its output.
    ``limit``: the clamp of experts with the "clamped" unit.
    ``shared_gate``: the shared expert's output is multiplied by sigmoid(w_sg . x), one number per token (w_sg is stacked under
    the router's rows, so the router's product yields it).
    The tokens are sorted by expert on the device and every expert multiplies its own contiguous rows (grouped GEMMs), so the
    launches do not depend on the routing."""

    def __init__(self, width: int, experts: int, top: int, ff: int, act: str, shared_ff: int = 0, shared_act: Optional[str] = None,
                 router_bias: bool = True, scoring: str = "softmax", groups: Sequence[int] = (1, 1), route_scale: float = 1.0,
                 shared_gate: bool = False, weight_on: str = "output", limit: float = 0.0):
        if scoring not in ("softmax", "sigmoid", "scores"):
            raise ValueError(f"unknown expert scoring {scoring!r}")
        if weight_on not in ("output", "input"):
            raise ValueError(f"the routing weight goes on the experts' output or input, not {weight_on!r}")
        self.width, self.experts, self.top, self.ff = width, experts, top, ff
        self.weight_on, self.limit = weight_on, float(limit)
        self.scoring, self.groups, self.route_scale = scoring, (int(groups[0]), int(groups[1])), float(route_scale)
        self.shared_gate = bool(shared_gate and shared_ff)
        self.epilogue = GatedFF.EPILOGUES[act]
        self.n_router = _round8(experts + 1) if self.shared_gate else experts      # router rows, then the shared gate's, then zeros
        self.router = Linear(width, self.n_router)
        self.router_bias: Optional[torch.Tensor] = None       # fp32 [experts]: the logits' bias or the picking correction
        self.has_bias = router_bias
        self.gate_up: Optional[torch.Tensor] = None           # [experts, 2 ff, width], gate / up rows interleaved
        self.down: Optional[torch.Tensor] = None              # [experts, width, ff]
        self.shared = GatedFF(width, shared_ff, shared_act or act) if shared_ff else None

    def stack_router(self, router: torch.Tensor, shared_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The router's matrix with the shared expert's gate row (and zero rows up to a multiple of 8) under it."""
        if not self.shared_gate:
            return router
        pad = torch.zeros((self.n_router - self.experts - 1, router.shape[1]), dtype=router.dtype, device=router.device)
        return torch.cat([router, shared_gate.reshape(1, -1).to(device=router.device, dtype=router.dtype), pad], 0)

    def reserve(self, s: Scratch, dt):
        f32, i32 = torch.float32, torch.int32
        s.reserve("router", f32, self.n_router)
        s.reserve("moe_ids", i32, self.top)
        s.reserve("moe_wts", f32, self.top)
        s.reserve("moe_slot", i32, self.top)
        s.reserve("moe_tok", i32, self.top)
        s.reserve("moe_x", dt, self.top * self.width)
        s.reserve("moe_act", dt, self.top * self.ff)
        s.reserve("moe_y", f32, self.top * self.width)
        s.reserve_flat("moe_seg", i32, self.experts + 1)
        if self.shared is not None:
            s.reserve("y_shared", f32, self.width)
            self.shared.reserve(s, dt)

    def __call__(self, x, y_out, s: Scratch):
        M, dt, f32, i32 = x.shape[0], x.dtype, torch.float32, torch.int32
        n = M * self.top
        logits = self.router(x, GEMM_STORE_F32, out=s.get("router", f32, M, self.n_router))
        ids, wts = s.get("moe_ids", i32, M, self.top), s.get("moe_wts", f32, M, self.top)
        slot_of, token_of = s.get("moe_slot", i32, M, self.top), s.get("moe_tok", i32, M, self.top)
        seg = s.flat("moe_seg", i32)
        if self.scoring == "scores":
            ops.moe_route_scores(logits, ids, wts, seg, slot_of, token_of, self.top, experts=self.experts)
        elif self.scoring == "sigmoid":
            ops.moe_route_sigmoid(logits, self.router_bias, ids, wts, seg, slot_of, token_of, self.top, self.groups[0], self.groups[1],
                                  self.route_scale, experts=self.experts)
        else:
            ops.moe_route(logits, self.router_bias, ids, wts, seg, slot_of, token_of, self.top)
        xs = s.get("moe_x", dt, n, self.width)
        on_input = self.weight_on == "input"
        if on_input:
            ops.moe_scatter_scaled(x, slot_of, wts, xs, self.top)
        else:
            ops.moe_gather(x, token_of, xs)
        act = ops.gemm_grouped(xs, self.gate_up, seg, M, self.epilogue, out=s.get("moe_act", dt, n, self.ff), limit=self.limit)
        ye = ops.gemm_grouped(act, self.down, seg, M, GEMM_STORE_F32, out=s.get("moe_y", f32, n, self.width))
        ysh = None
        if self.shared is not None:
            ysh = self.shared(x, s.get("y_shared", f32, M, self.width), s)
        ops.moe_combine(ye, slot_of, None if on_input else wts, ysh, y_out, self.top, shared_gate=logits[:, self.experts:self.experts + 1] if self.shared_gate else None)
        return y_out


class TokenSideInput:
    """Per-layer token input: e = table[token, layer slice]; y = W_proj (gelu_tanh(W_gate x) * e), x the residual stream."""

    def __init__(self, width: int, dim: int, col0: int):
        self.width, self.dim, self.col0 = width, dim, col0
        self.gate = Linear(width, dim)
        self.proj = Linear(dim, width)

    def reserve(self, s: Scratch, dt):
        s.reserve("sgate", torch.float32, self.dim)
        s.reserve("sg", dt, self.dim)

    def __call__(self, x_raw, y_out, table, ids, s: Scratch):
        M = x_raw.shape[0]
        gate = self.gate(x_raw, GEMM_STORE_F32, out=s.get("sgate", torch.float32, M, self.dim))
        g = ops.token_gate(gate, table, ids, s.get("sg", x_raw.dtype, M, self.dim), self.col0)
        return self.proj(g, GEMM_STORE_F32, out=y_out)


class HashedBigramEmbedding:
    """x = embed[token] * scale + bigram[(prev * mul_prev + token * mul_cur) mod buckets]; the table's last row (index
    ``buckets``) serves a sequence's first token.  ``bigram`` may be absent."""

    def __init__(self, vocab: int, width: int, scale: float, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0):
        self.vocab, self.width, self.scale = vocab, width, scale
        self.buckets, self.mul_prev, self.mul_cur = buckets, mul_prev, mul_cur
        self.weight: Optional[torch.Tensor] = None
        self.bigram: Optional[torch.Tensor] = None


class Sublayer:
    """One residual branch: x <- x + post_norm(f(pre(x))); ``pre_w`` None means f reads the residual stream itself."""

    def __init__(self, kind: str, module, layer: int, pre_w_name: Optional[str], post_w_name: str):
        self.kind, self.module, self.layer = kind, module, layer
        self.pre_w_name, self.post_w_name = pre_w_name, post_w_name
        self.pre_w: Optional[torch.Tensor] = None
        self.post_w: Optional[torch.Tensor] = None


class LayerRun:
    """One execution of a layer of the "parallel" or the "prenorm" chain.  "parallel": x <- x + mixer(n(x)) + mlp(n(x)) with ONE
    norm n (weight ``norm_w``, fp32, applied as a plain factor).  "prenorm": x <- x + mixer(n(x)), then x <- x + mlp(n2(x)) with a
    second norm (``norm2_w``).  ``slot`` is the run's entry in the cache list: a layer that runs several times (a looped span)
    has one run and one state per pass on the same modules.  ``opens``: the run is the first of a pass of the span, which
    begins with x <- W_in [x ; embedding] (``SequenceModel.loop_in``; models without it leave every ``opens`` False)."""

    def __init__(self, layer: int, slot: int, mixer, mlp, norm_w_name: str, opens: bool = False, norm2_w_name: Optional[str] = None):
        self.layer, self.slot, self.mixer, self.mlp, self.norm_w_name, self.opens = layer, slot, mixer, mlp, norm_w_name, opens
        self.norm2_w_name = norm2_w_name
        self.port1: Optional[StreamPort] = None       # "hyper" chain: how the mixer and the feed-forward meet the stream's copies
        self.port2: Optional[StreamPort] = None
        self.norm_w: Optional[torch.Tensor] = None
        self.norm2_w: Optional[torch.Tensor] = None


class StreamPort:
    """How one sublayer of a "hyper" model meets the copies of the residual stream: it reads u = sum_s read[s] x_s, norms it with
    tanh(alpha u) w + b, adds the causal convolution ``conv_w`` (kept tap by tap, [taps, width]) of that over time, and its output y is
    written back
    as x_r <- sum_s mix[s, r] x_s + out[r] y.  All fp32 on the device."""

    def __init__(self, norm_name: str, hc_name: str, conv_name: str):
        self.norm_name, self.hc_name, self.conv_name = norm_name, hc_name, conv_name
        self.read = self.out = self.mix = self.alpha = self.w = self.b = self.conv_w = None


def unroll_layers(n_layers: int, start: int = 0, stop: int = 0, times: int = 1) -> List[tuple]:
    """(layer, opens a pass) in execution order when the layers start .. stop-1 run ``times`` times in a row."""
    if stop <= start:
        return [(i, False) for i in range(n_layers)]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n_layers)]


class SequenceModel:
    """callable(inputs [B, L], cache=None, last_only=False, prompt_lengths=None) -> float32 logits, like the other models,
    plus ``forward_ragged`` for prompts of unequal length and arbitrary logit positions.  Subclasses build ``self.embed``,
    ``self.final_norm_w`` / ``self.lm_head``, name their tensors in ``load_weights``, and describe their layers in one of two
    ways: ``block_style`` "sandwich": ``self.sublayers`` (in execution order) and ``self.mixers`` (one per layer), every
    sublayer between two norms; "parallel": ``self.runs`` (LayerRun, in execution order) and optionally ``self.loop_in``;
    "prenorm": ``self.runs`` whose mixer and feed-forward each read a norm of their own; "hyper": ``self.runs`` with a
    ``StreamPort`` per sublayer over ``self.streams`` copies of the stream, a tanh norm (also the model's last one,
    ``self.final_tanh_norm`` = (alpha, w, b)) and a convolution of ``self.canon_taps`` taps on every sublayer's input.
    ``self.logit_scale`` multiplies the logits."""

    block_style = "sandwich"

    supports_ragged = True
    dense = True                      # unquantised weights: no ``quantization`` block in config.json
    kernel_units = "sequence"         # key of _lib.UNIT_SETS: what a fresh checkout has to compile for this family

    def __init__(self, args):
        self.args = args
        self.model_type = args.model_type
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        self._arenas: Dict[tuple, dict] = {}
        self._lock = threading.RLock()
        self.tp_rank, self.tp_world = 0, 1
        self.embed: Optional[HashedBigramEmbedding] = None
        self.sublayers: List[Sublayer] = []
        self.mixers: list = []
        self.runs: List[LayerRun] = []
        self.loop_in: Optional[Linear] = None         # [width, 2 width]: opens every pass of a looped span
        self.side_table: Optional[torch.Tensor] = None
        self.final_norm_w: Optional[torch.Tensor] = None
        self.lm_head: Optional[Linear] = None
        self.eps = 1e-6
        self.logit_scale = 1.0
        self.streams, self.canon_taps = 1, 1          # "hyper" chain
        self.final_tanh_norm: Optional[tuple] = None  # (alpha, w, b): the last norm is tanh(alpha x) w + b instead of an rms norm
        # debugging aid: callable(layer, kind, h [M, width]) run after every closed branch of an eager pass (never set it
        # while a decode step is being captured)
        self.residual_tap = None

    # -- surface shared with DecoderModel ---------------------------------------------------------------
    @property
    def layers(self):
        return self.mixers

    def eval(self):
        return self

    def graph_safe(self, B: int) -> bool:
        return True

    def greedy_tokens(self, logits, tok_out, probs_out=None):
        ops.argmax(logits, out=tok_out, probs_out=probs_out)

    def sample_tokens(self, logits, temp, top_p, seed, offset, tok_out, probs_out=None):
        ops.sample_top_p(logits, temp, top_p, seed, offset, out=tok_out, probs_out=probs_out)

    def set_tensor_parallel(self, rank, world, allreduce):
        if world > 1:
            raise NotImplementedError("tensor parallelism is not built for this model family")

    # -- state ----------------------------------------------------------------------------------------------
    def cache_key(self) -> tuple:
        return ("sequence", id(self))

    def new_cache(self, batch_size: int) -> List[RowState]:
        """One entry per layer (its mixer's state) and a last one for the previous token of every row."""
        if self.block_style == "hyper":
            # per run: the mixer's state and the carried inputs of the two input convolutions
            W, taps = self.args.width, self.canon_taps
            return [StateGroup([r.mixer.new_state(batch_size), ConvTailState(W, taps, batch_size), ConvTailState(W, taps, batch_size)],
                               batch_size) for r in self.runs] + [TokenState(batch_size)]
        if self.block_style in ("parallel", "prenorm"):
            return [r.mixer.new_state(batch_size) for r in self.runs] + [TokenState(batch_size)]
        return [m.new_state(batch_size) for m in self.mixers] + [TokenState(batch_size)]

    def make_cache(self, batch_size: int, step: Optional[int] = None, paged: bool = True) -> List[RowState]:
        from ._transformer import bind_cache_group
        caches = self.new_cache(batch_size)
        bind_cache_group(caches, self.device, step)
        return caches

    # -- scratch ----------------------------------------------------------------------------------------------
    def _arena(self, M: int, B: int, ragged: bool = False) -> dict:
        """Buffers for up to M packed tokens of B entries on the current stream.  The decode step's arena (M == B, not
        ``ragged``) has its plan inputs preset (one token per entry, rows 0..B-1 unless the caller rewrites ``rows``) so that
        a captured graph can replay over them; ragged passes rewrite theirs every time and use arenas of their own."""
        key = (M, B, ragged, torch.cuda.current_stream(self.device).cuda_stream)
        a = self._arenas.get(key)
        if a is None:
            dev, dt, W = self.device, self.dtype, self.args.width
            s = Scratch(dev, M)
            for m in self.mixers:
                m.reserve(s, dt)
            for sl in self.sublayers:
                if sl.kind != "mixer":
                    sl.module.reserve(s, dt)
            for r in self.runs:
                r.mixer.reserve(s, dt)
                if r.mlp is not None:
                    r.mlp.reserve(s, dt)
                    s.reserve("y2", torch.float32, W)
            if self.loop_in is not None:
                s.reserve("cat", dt, 2 * W)
            if self.block_style == "hyper":
                s.reserve("xs", torch.float32, self.streams * W)
                s.reserve("n", torch.float32, W)
            s.reserve("y", torch.float32, W)
            s.reserve("x", dt, W)
            s.reserve("xl", dt, W)
            s.allocate()
            i32 = dict(dtype=torch.int32, device=dev)
            a = dict(
                s=s, cap=M,
                h=torch.empty((M, W), dtype=torch.float32, device=dev),
                ids=torch.zeros((M,), **i32), t_row=torch.zeros((M,), **i32), t_pos=torch.zeros((M,), **i32),
                t_off=torch.zeros((M,), **i32),
                cu=torch.arange(B + 1, **i32) if not ragged else torch.zeros((B + 1,), **i32),
                rows=torch.arange(B, **i32),
            )
            if len(self._arenas) > 8:
                self._arenas.clear()
            self._arenas[key] = a
        return a

    # -- forward ----------------------------------------------------------------------------------------------
    def _layers_forward(self, ids_i32: torch.Tensor, B: int, L: int, cache: List[RowState], a: dict, M: Optional[int] = None,
                        max_n: int = 1):
        """Run the packed tokens ``ids_i32`` ([M]) of the B entries described by a["cu"] / a["rows"] through every layer;
        the residual stream is left in a["h"][:M].  (L is 1 for a decode step and unused otherwise: entries are ragged;
        ``max_n`` is the longest entry's token count, which picks prompt or decode kernels.)"""
        M = ids_i32.numel() if M is None else M
        s: Scratch = a["s"]
        dt, W = self.dtype, self.args.width
        lengths = cache[-1].lengths(self.device)
        plan = dict(cu=a["cu"], rows=a["rows"], nb=B, lengths=lengths, max_n=max_n, t_row=a["t_row"][:M], t_pos=a["t_pos"][:M], t_off=a["t_off"][:M])
        ops.ragged_plan(a["cu"], a["rows"], lengths, plan["t_row"], plan["t_pos"], plan["t_off"], B, M)
        e = self.embed
        h = a["h"][:M]
        ops.embed_hashed(ids_i32, plan["t_row"], plan["t_pos"], plan["t_off"], cache[-1].last_token, e.weight, e.bigram, h, e.scale,
                         e.buckets, e.mul_prev, e.mul_cur)
        x, y = s.get("x", dt, M, W), s.get("y", torch.float32, M, W)
        if self.block_style == "parallel":
            return self._chain_parallel(h, x, y, plan, s, cache, M)
        if self.block_style == "prenorm":
            return self._chain_prenorm(h, x, y, plan, s, cache)
        if self.block_style == "hyper":
            return self._chain_hyper(h, x, y, plan, s, cache, M)
        subs = self.sublayers

        def feed(nxt: Optional[Sublayer], y_in, post_w):
            """Close a branch (h += post_norm(y)) and prepare the input of the next one in the same pass over the row."""
            pre = nxt.pre_w if nxt is not None else None
            raw = nxt is not None and nxt.pre_w is None
            ops.norm_add_norm(h, self.eps, dt, y=y_in, w_post=post_w, w_next=pre, x_out=x if pre is not None else None,
                              raw_out=x if raw else None)

        feed(subs[0] if subs else None, None, None)
        for i, sl in enumerate(subs):
            if sl.kind == "mixer":
                sl.module(x, y, cache[sl.layer], plan, s, cache)
            elif sl.kind == "mlp":
                sl.module(x, y, s)
            else:
                sl.module(x, y, self.side_table, ids_i32, s)
            feed(subs[i + 1] if i + 1 < len(subs) else None, y, sl.post_w)
            if self.residual_tap is not None:
                self.residual_tap(sl.layer, sl.kind, h)

    def _chain_parallel(self, h, x, y, plan: dict, s: Scratch, cache: List[RowState], M: int):
        """The runs of a "parallel" model over the residual stream h (fp32): every run reads x = n(h) and adds its branches to h
        in one pass over the rows, which also prepares what comes next: the next run's normed input, or (before a pass of a
        looped span) the storage-type copy of h that W_in multiplies beside the embedding."""
        dt, W, eps, runs = self.dtype, self.args.width, self.eps, self.runs
        cat = s.get("cat", dt, M, 2 * W) if self.loop_in is not None else None

        def close(i_next: int, y1, y2):
            nxt = runs[i_next] if i_next < len(runs) else None
            if nxt is None:
                if y1 is not None:
                    ops.residual_add_norm(h, eps, dt, y1=y1, y2=y2)
            elif nxt.opens:
                ops.residual_add_norm(h, eps, dt, y1=y1, y2=y2, raw_out=cat[:, :W])
            else:
                ops.residual_add_norm(h, eps, dt, y1=y1, y2=y2, w_next=nxt.norm_w, x_out=x)
            if i_next > 0 and self.residual_tap is not None:
                self.residual_tap(runs[i_next - 1].layer, "run", h)
            if nxt is not None and nxt.opens:
                self.loop_in(cat, GEMM_STORE_F32, out=h)
                ops.residual_add_norm(h, eps, dt, w_next=nxt.norm_w, x_out=x)

        if cat is not None:
            ops.residual_add_norm(h, eps, dt, raw_out=cat[:, W:])           # the embedding, for every pass
        close(0, None, None)
        for i, r in enumerate(runs):
            r.mixer(x, y, cache[r.slot], plan, s, cache)
            y2 = None
            if r.mlp is not None:
                y2 = r.mlp(x, s.get("y2", torch.float32, M, W), s)
            close(i + 1, y, y2)

    def _chain_prenorm(self, h, x, y, plan: dict, s: Scratch, cache: List[RowState]):
        """The runs of a "prenorm" model over the residual stream h (fp32): x <- n1(h), h += mixer(x); x <- n2(h), h += mlp(x).
        Every addition to the stream also writes the normed input of whatever reads it next, in the same pass over the row."""
        dt, eps, runs = self.dtype, self.eps, self.runs
        if runs:
            ops.residual_add_norm(h, eps, dt, w_next=runs[0].norm_w, x_out=x)
        for i, r in enumerate(runs):
            nxt = runs[i + 1].norm_w if i + 1 < len(runs) else None
            r.mixer(x, y, cache[r.slot], plan, s, cache)
            if r.mlp is not None:
                ops.residual_add_norm(h, eps, dt, y1=y, w_next=r.norm2_w, x_out=x)
                r.mlp(x, y, s)
            ops.residual_add_norm(h, eps, dt, y1=y, w_next=nxt, x_out=x if nxt is not None else None)
            if self.residual_tap is not None:
                self.residual_tap(r.layer, "run", h)

    def _chain_hyper(self, h, x, y, plan: dict, s: Scratch, cache: List[RowState], M: int):
        """The runs of a "hyper" model.  h holds the embedding; the copies of the stream live in one fp32 buffer [M, streams, W].
        Every sublayer's output is written back and the next sublayer's input read and normed in ONE pass over the copies
        (b200p_hyper_step); the input convolution follows (prompts: b200p_canon_conv over the portion's rows and the carried
        inputs, which b200p_delta_conv_commit then replaces; decode steps: inside the same pass).  The last pass leaves the sum of
        the copies in h for the model's last norm."""
        S, W, taps, dt, runs = self.streams, self.args.width, self.canon_taps, self.dtype, self.runs
        xs, n = s.get("xs", torch.float32, M, S * W), s.get("n", torch.float32, M, W)
        decode = plan["max_n"] == 1
        stops = []                                     # (run, port, its carried inputs) in execution order
        for r in runs:
            st = cache[r.slot]
            stops.append((r, r.port1, st.parts[1], True))
            if r.mlp is not None:
                stops.append((r, r.port2, st.parts[2], False))

        def step(y_in, prev: Optional[StreamPort], k_next: int, want_sum: bool):
            nxt = stops[k_next] if k_next < len(stops) else None
            kw = dict(y=y_in, mix=prev.mix if prev else None, out=prev.out if prev else None, src=h if prev is None else None,
                      sum_out=h if want_sum else None)
            if nxt is None:
                return ops.hyper_step(xs, S, **kw)
            port, tail = nxt[1], nxt[2]
            kw.update(read=port.read, alpha=port.alpha, w=port.w, b=port.b)
            if decode:
                ops.hyper_step(xs, S, conv_w=port.conv_w, conv_state=tail.conv, t_row=plan["t_row"], t_pos=plan["t_pos"], taps=taps,
                               x_out=x, **kw)
                return
            ops.hyper_step(xs, S, n_out=n, **kw)
            ops.canon_conv(n, port.conv_w, tail.conv, plan["t_row"], plan["t_pos"], plan["t_off"], x, taps)
            if taps > 1:
                ops.delta_conv_commit(n, tail.conv, plan["cu"], plan["rows"], plan["nb"], W, taps)

        step(None, None, 0, not stops)
        for k, (r, port, _, is_mixer) in enumerate(stops):
            if is_mixer:
                r.mixer(x, y, cache[r.slot].parts[0], plan, s, cache)
            else:
                r.mlp(x, y, s)
            closes_run = k + 1 == len(stops) or stops[k + 1][0] is not r
            tap = closes_run and self.residual_tap is not None
            step(y, port, k + 1, k + 1 == len(stops) or tap)
            if tap:
                self.residual_tap(r.layer, "run", h)

    def _advance_device(self, cache: List[RowState], a: dict, B: int, ids_i32: Optional[torch.Tensor] = None):
        """End of a step on the device: lengths += tokens brought, last token of every entry remembered."""
        ops.ragged_advance(cache[-1]._lengths, cache[-1].last_token, a["ids"] if ids_i32 is None else ids_i32, a["cu"], a["rows"], B)

    def _head(self, h_rows: torch.Tensor, a: dict, logits_out: Optional[torch.Tensor] = None, x_rows=None):
        """final norm + output projection of the given residual rows -> float32 logits."""
        n = h_rows.shape[0]
        xl = a["s"].get("xl", self.dtype, n, self.args.width)
        if self.final_tanh_norm is not None:
            ops.tanh_norm(h_rows, *self.final_tanh_norm, xl)
        else:
            ops.norm_add_norm(h_rows, self.eps, self.dtype, w_next=self.final_norm_w, x_out=xl)
        logits = self.lm_head(xl, GEMM_STORE_F32, out=logits_out)
        if self.logit_scale != 1.0:
            ops.scale_(logits, self.logit_scale)
        return logits

    def forward_ragged(self, seqs: Sequence[Sequence[int]], cache: List[RowState], rows: Optional[Sequence[int]] = None,
                       want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Feed entry i's tokens ``seqs[i]`` to cache row ``rows[i]`` (default i), continuing whatever the row holds.
        ``want[i]``: offsets into seqs[i] whose logits are returned (default: the last token of every non-empty entry), in
        entry order -> float32 [n_wanted, vocab]."""
        with self._lock:
            return self._forward_ragged_locked(seqs, cache, rows, want)

    def _forward_ragged_locked(self, seqs, cache, rows, want):
        from ._transformer import advance_rows, prepare_rows
        nb = len(seqs)
        rows = list(range(nb)) if rows is None else [int(r) for r in rows]
        if len(set(rows)) != nb or any(r < 0 or r >= cache[-1].batch_size for r in rows):
            raise ValueError("rows must be distinct rows of the cache")
        if want is None:
            want = [[len(q) - 1] if len(q) else [] for q in seqs]
        counts = [len(q) for q in seqs]
        dev = self.device
        outs = [[None] * len(w) for w in want]
        done = [0] * nb
        while True:
            # one pass: every entry brings its next tokens, the pass holds at most MAX_TOKENS_PER_FORWARD of them
            left = [counts[i] - done[i] for i in range(nb)]
            live = sum(1 for n in left if n > 0)
            if live == 0:
                break
            share = max(1, MAX_TOKENS_PER_FORWARD // live)
            take = [min(n, share) for n in left]
            M = sum(take)
            prepare_rows(cache, rows, take, self.dtype, dev)
            a = self._arena(_round_up_rows(M), nb, ragged=True)
            flat, cu = [], [0]
            for i in range(nb):
                flat.extend(seqs[i][done[i]:done[i] + take[i]])
                cu.append(cu[-1] + take[i])
            ids = a["ids"][:M]
            ids.copy_(torch.tensor(flat, dtype=torch.int32), non_blocking=False)
            a["cu"].copy_(torch.tensor(cu, dtype=torch.int32))
            a["rows"].copy_(torch.tensor(rows, dtype=torch.int32))
            self._layers_forward(ids, nb, 0, cache, a, M, max_n=max(take))
            self._advance_device(cache, a, nb, ids)
            advance_rows(cache, rows, take)
            pick, where = [], []
            for i in range(nb):
                for k, p in enumerate(want[i]):
                    if done[i] <= p < done[i] + take[i]:
                        pick.append(cu[i] + p - done[i])
                        where.append((i, k))
            if pick:
                hs = a["h"][:M].index_select(0, torch.tensor(pick, dtype=torch.int64, device=dev))
                lg = self._head(hs, a)
                for j, (i, k) in enumerate(where):
                    outs[i][k] = lg[j]
            for i in range(nb):
                done[i] += take[i]
        flat_out = [t for o in outs for t in o]
        if any(t is None for t in flat_out):
            raise ValueError("a wanted position lies outside its entry's tokens")
        V = self.lm_head.out_features
        return torch.stack(flat_out, 0) if flat_out else torch.empty((0, V), dtype=torch.float32, device=dev)

    def __call__(self, inputs, cache: Optional[List[RowState]] = None, last_only: bool = False, prompt_lengths=None):
        """inputs int [B, L] -> logits float32 [B, L, V] (or [B, 1, V] with last_only).  ``prompt_lengths[b]`` < L marks the
        first L - prompt_lengths[b] ids of row b as left padding: they are not fed to the model at all, and with
        last_only=False their logits are zero."""
        if not isinstance(inputs, torch.Tensor):
            inputs = torch.as_tensor(inputs)
        B, L = inputs.shape
        host = inputs.tolist()
        n = [L] * B if prompt_lengths is None else [int(v) for v in prompt_lengths]
        seqs = [host[b][L - n[b]:] for b in range(B)]
        if cache is None:
            cache = self.make_cache(B, step=max(L, 1))
        if last_only:
            return self.forward_ragged(seqs, cache).view(B, 1, -1)
        lg = self.forward_ragged(seqs, cache, want=[list(range(k)) for k in n])
        out = torch.zeros((B, L, lg.shape[-1]), dtype=torch.float32, device=lg.device)
        o = 0
        for b in range(B):
            out[b, L - n[b]:] = lg[o:o + n[b]]
            o += n[b]
        return out

    def release_rows(self, cache: List[RowState], rows: Sequence[int]):
        """Give rows back to the cache: the next sequence in them starts from nothing."""
        from ._transformer import release_rows
        with self._lock:
            release_rows(cache, [int(r) for r in rows])


def _round_up_rows(M: int) -> int:
    """Arena capacity for M packed tokens: powers of two from 64, so prompts of nearby sizes share scratch."""
    c = 64
    while c < M:
        c *= 2
    return c

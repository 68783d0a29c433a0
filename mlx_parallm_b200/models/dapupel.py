"""Dapupel: a decoder that keeps several copies of its residual stream, norms without statistics, and lets every sublayer read a
short convolution of its input.

config.json (``"architecture": "Dapupel"``) lists the layers one by one -- ``type``, the mixer's sizes, its feed-forward (or
null) -- and gives every size and constant; tensors are named ``l<i>.<part>``.

    stream        ``streams`` copies x_1 .. x_s, all equal to the embedding at the start.  A sublayer reads u = sum_s in[s] x_s and
                  writes x_r <- sum_s mix[s, r] x_s + out[r] y (``hc1`` for the mixer, ``hc2`` for the feed-forward); the output
                  reads the sum of the copies
    norm          tanh(alpha u) w + b with a scalar alpha: no mean, no variance
    input conv    every sublayer reads n + conv(n), a causal convolution of ``canon.taps`` taps over time on each channel of its
                  normed input n (``canon1`` / ``canon2``); the last taps - 1 inputs are state
    channel_delta    gated delta rule, one decay per head and key channel, decay and gate through low-rank pairs of matrices
    latent_attention queries and keys/values through rms-normed latents; every head's key has an unrotated part made from the
                  latent and a rotated part shared by all heads; interleaved pairs, frequencies stretched for long contexts
                  (the stretched part of the spectrum slowed by ``factor``, a linear ramp between ``fast`` and ``slow`` rotations
                  per ``original`` positions, cos and sin times 0.1 ln(factor) + 1); causal softmax
    attention     grouped heads without rotation, a short convolution on q and k, values = keys, scores capped by
                  softcap tanh(s / softcap), minus r1_h ln(1 + r2_h (i - j)), a sliding window, a sigmoid gate on the heads
    feed-forward  routed experts with the clamped unit g sigmoid(1.702 g) (u + 1); the ``top`` largest sigmoid scores are the
                  weights as they are, and multiply the experts' INPUT
    output        the model's norm, then the embedding table as the head

The reference has no such graph; the blocks are in models/_sequence.py and run on the ragged-batch kernels of the library.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from ._sequence import (GatedDeltaMixer, GatedFF, HashedBigramEmbedding, LatentAttention, LayerRun, Linear, RoutedExperts, SequenceModel,
                        StreamPort, WindowAttention)
from .base import BaseModelArgs

MIXER_TYPES = ("channel_delta", "latent_attention", "attention")
MAX_STREAMS = 8
MAX_CANON_TAPS = 16


def stretched_rates(dims: int, base: float, scaling: Optional[dict] = None) -> Tuple[List[float], float]:
    """(angle per position of the pairs (2i, 2i+1), i < dims / 2; factor on cos and sin).  f_i = base^(-2i / dims).  With
    ``scaling`` (factor, original, fast, slow): d(t) = dims ln(original / (2 pi t)) / (2 ln base) is the (fractional) pair that
    makes t turns in ``original`` positions; lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1); pairs below lo keep
    f_i, pairs above hi get f_i / factor, and between them r_i = (i - lo) / max(hi - lo, 0.001) blends the two linearly.  The
    magnitude is 0.1 ln(factor) + 1."""
    rates = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return rates, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(rates):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * r + f * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


@dataclass
class ModelArgs(BaseModelArgs):
    vocab: int
    width: int
    layers: List[Dict[str, Any]]
    norm: Dict[str, Any] = field(default_factory=dict)
    canon: Dict[str, Any] = field(default_factory=dict)
    streams: int = 1
    architecture: str = "Dapupel"
    model_type: str = "dapupel"

    def __post_init__(self):
        if not self.layers:
            raise ValueError("config 'layers' is empty")
        if not (1 <= int(self.streams) <= MAX_STREAMS):
            raise ValueError(f"streams must be in [1, {MAX_STREAMS}]")
        if not (1 <= int(self.canon.get("taps", 1)) <= MAX_CANON_TAPS):
            raise ValueError(f"canon.taps must be in [1, {MAX_CANON_TAPS}]")
        for i, L in enumerate(self.layers):
            if L.get("type") not in MIXER_TYPES:
                raise NotImplementedError(f"layer {i}: mixer type {L.get('type')!r} is not part of this design")
            m = L["mixer"]
            if L["type"] != "latent_attention" and m["heads"] % m.get("kv_heads", m["heads"]):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            if L["type"] == "latent_attention":
                rot = m.get("rot") or {}
                if int(m.get("rot_dim", 0)) and int(rot.get("dims", m["rot_dim"])) != int(m["rot_dim"]):
                    raise ValueError(f"layer {i}: the rotated part is rotated whole (rot.dims == rot_dim)")
                if int(m.get("rot_dim", 0)) % 2:
                    raise ValueError(f"layer {i}: rot_dim must be even")
            mlp = L.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "moe":
                    raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
                if not (1 <= int(mlp["router"]["top"]) <= int(mlp["router"]["experts"])):
                    raise ValueError(f"layer {i}: 1 <= top <= experts")

    @property
    def vocab_size(self) -> int:
        return self.vocab


class Model(SequenceModel):
    block_style = "hyper"
    kernel_units = "sequence_hyper"

    def __init__(self, args: ModelArgs):
        super().__init__(args)
        W = args.width
        self.eps = float(args.norm.get("eps", 1e-6))
        self.streams = int(args.streams)
        self.canon_taps = int(args.canon.get("taps", 1))
        self.embed = HashedBigramEmbedding(args.vocab, W, 1.0)
        for i, L in enumerate(args.layers):
            m = L["mixer"]
            if L["type"] == "channel_delta":
                mixer = GatedDeltaMixer(W, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], int(m.get("conv", 1)), self.eps,
                                        channel_decay=True, decay_rank=None, gate_rank=None, gate_act="sigmoid")
            elif L["type"] == "latent_attention":
                dr = int(m.get("rot_dim", 0))
                rot = m.get("rot") or {}
                rates, mag = stretched_rates(dr, float(rot["base"]), rot.get("scaling")) if dr else ([], 1.0)
                mixer = LatentAttention(W, m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"], float(m["scale"]), 0, self.eps,
                                        rot_dim=dr, rates=rates, mag=mag)
            else:
                if int(m.get("vdim", m["dim"])) != int(m["dim"]):
                    raise ValueError(f"layer {i}: the values are the keys, so vdim == dim")
                mixer = WindowAttention(W, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], float(m["scale"]), taps=int(m.get("conv", 1)),
                                        softcap=float(m.get("softcap", 0.0)), window=int((m.get("mask") or {}).get("size", 0)),
                                        distance_penalty=True, gated=True)
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                r = mlp["router"]
                ff = RoutedExperts(W, int(r["experts"]), int(r["top"]), int(mlp["expert"]["ff"]), "clamped", router_bias=False,
                                   scoring="scores", weight_on="input", limit=float(mlp["expert"]["limit"]))
            run = LayerRun(i, i, mixer, ff, f"l{i}.norm1", False, f"l{i}.norm2" if ff is not None else None)
            run.port1 = StreamPort(f"l{i}.norm1", f"l{i}.hc1", f"l{i}.canon1")
            run.port2 = StreamPort(f"l{i}.norm2", f"l{i}.hc2", f"l{i}.canon2") if ff is not None else None
            self.runs.append(run)
        self.mixers = [r.mixer for r in self.runs]
        self.lm_head = Linear(W, args.vocab)          # the embedding table

    # -- parameters ------------------------------------------------------------------------------------------
    def parameter_names(self) -> List[str]:
        names = ["embed", "final.norm", "final.norm.alpha", "final.norm.b"]
        for i, L in enumerate(self.args.layers):
            p = f"l{i}."
            subs = ("1", "2") if L.get("mlp") is not None else ("1",)
            for q in subs:
                names += [f"{p}norm{q}", f"{p}norm{q}.alpha", f"{p}norm{q}.b", f"{p}hc{q}.in", f"{p}hc{q}.out", f"{p}hc{q}.mix", f"{p}canon{q}"]
            if L["type"] == "channel_delta":
                names += [p + "mix." + n for n in ("q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "A_log", "norm", "a1", "a2",
                                                   "dt_bias", "g1", "g2", "o")]
            elif L["type"] == "latent_attention":
                names += [p + "mix." + n for n in ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "o")]
            else:
                names += [p + "mix." + n for n in ("q", "k", "q.conv", "k.conv", "r1", "r2", "g", "o")]
            mlp = L.get("mlp")
            if mlp is not None:
                for e in range(int(mlp["router"]["experts"])):
                    names += [f"{p}mlp.e{e}.{n}" for n in ("gate", "up", "down")]
                names.append(p + "mlp.router")
        return names

    def load_weights(self, weights: Dict[str, torch.Tensor], device="cuda", strict: bool = True, dtype=None):
        """Matrices go to the device in ``dtype`` (default: as stored); vectors and scalars (norms, stream weights, convolution
        taps, decay parameters, distance penalties) as float32.  Projections that read the same input are stacked into one
        matrix, gate / up rows interleaved for the fused epilogue, the experts stacked per layer, W_uk stored per head
        transposed; the rotation's rates are computed on the host in float64."""
        device = torch.device(device)
        missing = [n for n in self.parameter_names() if n not in weights]
        if missing:
            raise KeyError(f"missing parameters: {missing[:4]}{'...' if len(missing) > 4 else ''}")
        if dtype is None:
            dtype = weights["embed"].dtype
        if dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise TypeError(f"unsupported storage dtype {dtype}")
        self.dtype, self.device = dtype, device
        a, W, S, taps = self.args, self.args.width, self.streams, self.canon_taps

        def put(t):
            return t.to(device=device, dtype=dtype).contiguous()

        def check(name, shape):
            if tuple(weights[name].shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(weights[name].shape)} does not match the config ({tuple(shape)})")

        def vec(name, shape=None):
            if shape is not None:
                check(name, shape)
            return weights[name].float().reshape(-1 if weights[name].dim() == 0 else weights[name].shape).to(device).contiguous()

        def tanh_norm(name):
            if weights[name + ".alpha"].numel() != 1:
                raise ValueError(f"{name}.alpha: one number")
            return vec(name + ".alpha"), vec(name, (W,)), vec(name + ".b", (W,))

        def port(p: StreamPort):
            p.alpha, p.w, p.b = tanh_norm(p.norm_name)
            p.read, p.out, p.mix = vec(p.hc_name + ".in", (S,)), vec(p.hc_name + ".out", (S,)), vec(p.hc_name + ".mix", (S, S))
            p.conv_w = vec(p.conv_name, (W, taps)).t().contiguous()          # tap by tap: [taps, W]

        check("embed", (a.vocab, W))
        self.embed.weight = put(weights["embed"])
        self.lm_head.weight = self.embed.weight
        self.final_tanh_norm = tanh_norm("final.norm")
        for r, L in zip(self.runs, a.layers):
            i, m = r.layer, r.mixer
            p = f"l{i}.mix."
            port(r.port1)
            if isinstance(m, GatedDeltaMixer):
                check(p + "q", (m.c_qk, W))
                check(p + "k", (m.c_qk, W))
                check(p + "v", (m.c_v, W))
                check(p + "b", (m.heads, W))
                r_a, r_g = weights[p + "a1"].shape[0], weights[p + "g1"].shape[0]
                check(p + "a1", (r_a, W))
                check(p + "a2", (m.n_decay, r_a))
                check(p + "g1", (r_g, W))
                check(p + "g2", (m.c_v, r_g))
                check(p + "o", (W, m.c_v))
                m.set_ranks(r_a, r_g)
                m.in_proj.weight = put(m.stack_in_proj(*(weights[p + n] for n in ("q", "k", "v", "b", "g1", "a1"))))
                m.decay_up.weight, m.gate_up.weight = put(weights[p + "a2"]), put(weights[p + "g2"])
                m.o_proj.weight = put(weights[p + "o"])
                for n, rows in (("q.conv", m.c_qk), ("k.conv", m.c_qk), ("v.conv", m.c_v)):
                    check(p + n, (rows, m.taps))
                m.conv_w = torch.cat([weights[p + n].float() for n in ("q.conv", "k.conv", "v.conv")], 0).to(device).contiguous()
                m.A_log, m.dt_bias = vec(p + "A_log", (m.heads,)), vec(p + "dt_bias", (m.n_decay,))
                m.norm_w = vec(p + "norm", (m.vdim,))
            elif isinstance(m, LatentAttention):
                H, dk, dr, dv, R = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
                check(p + "dq", (m.q_rank, W))
                check(p + "dkv", (R + dr, W))
                check(p + "uq", (H * (dk + dr), m.q_rank))
                check(p + "uk", (H * dk, R))
                check(p + "uv", (H * dv, R))
                check(p + "o", (W, H * dv))
                m.down.weight = put(torch.cat([weights[p + "dq"], weights[p + "dkv"]], 0))
                m.uq.weight = put(weights[p + "uq"])
                m.uk_t = put(weights[p + "uk"].reshape(H, dk, R).transpose(1, 2))          # [H, R, dk]
                m.uv = put(weights[p + "uv"])
                m.o_proj.weight = put(weights[p + "o"])
                m.q_norm_w, m.kv_norm_w = vec(p + "dq.norm", (m.q_rank,)), vec(p + "dkv.norm", (R,))
                m.rates = torch.tensor(m.rate_values, dtype=torch.float32, device=device) if m.rate_values else None
            else:
                check(p + "q", (m.n_mix, W))
                check(p + "k", (m.kv_heads * m.dim, W))
                check(p + "g", (m.n_mix, W))
                check(p + "o", (W, m.n_mix))
                check(p + "q.conv", (m.n_mix, m.taps))
                check(p + "k.conv", (m.kv_heads * m.dim, m.taps))
                m.in_proj.weight = put(torch.cat([weights[p + n] for n in ("q", "k", "g")], 0))
                m.o_proj.weight = put(weights[p + "o"])
                m.conv_w = torch.cat([weights[p + "q.conv"].float(), weights[p + "k.conv"].float()], 0).t().to(device).contiguous()   # [taps, C]
                m.r1, m.r2 = vec(p + "r1", (m.heads,)), vec(p + "r2", (m.heads,))
            ff = r.mlp
            if ff is None:
                continue
            port(r.port2)
            q = f"l{i}.mlp."
            check(q + "router", (ff.experts, W))
            ff.router.weight = put(weights[q + "router"])
            for e in range(ff.experts):
                check(f"{q}e{e}.gate", (ff.ff, W))
                check(f"{q}e{e}.up", (ff.ff, W))
                check(f"{q}e{e}.down", (W, ff.ff))
            ff.gate_up = put(torch.stack([GatedFF.interleave(weights[f"{q}e{e}.gate"], weights[f"{q}e{e}.up"]) for e in range(ff.experts)], 0))
            ff.down = put(torch.stack([weights[f"{q}e{e}.down"] for e in range(ff.experts)], 0))
        self._arenas.clear()
        return self

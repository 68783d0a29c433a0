"""Nifalorn: a pre-norm decoder whose layers pick one of three mixers, with a span of layers that can run several times on the
same weights.

config.json (``"architecture": "Nifalorn"``) lists the layers one by one -- ``type``, the mixer's sizes, its feed-forward (or
null) -- and gives every size and constant; tensors are named ``l<i>.<part>``.

    layer         x <- x + mixer(n1(x)); x <- x + ff(n2(x)), n = rms_norm(x) * (1 + w)     (the stored norm weights are offsets from one)
    loop          layers start .. stop-1 run ``times`` times in a row; every pass has its own states; nothing else happens
                  between passes
    lightning     linear attention with a constant decay per head: silu on q, k, v, all heads normed as one vector, sigmoid gate
    mamba2        selective state-space layer: one projection [z | x | B | C | dt], a short convolution with bias on x, B, C,
                  a scalar decay per head and token, y * silu(z) normed in equal parts of the channels
    attention     two softmax maps per head over the same values, subtracted with one lambda per layer, the head's output
                  divided by its root mean square; pairwise rotation of the first rot.dims dimensions with slowed-down long
                  wavelengths; position i sees j <= i of its own chunk of mask.size positions
    feed-forward  dense W_down relu(W_up x)^2, or routed experts (silu gate) picked by sigmoid scores + a correction inside
                  the best expert groups, beside a shared expert gated by one sigmoid per token
    output        the model's norm, the head, times logit_scale; the embedding is multiplied by embedding.scale

The reference has no such graph; the blocks are in models/_sequence.py and run on the ragged-batch kernels of the library.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from ._sequence import (ActivatedFF, DecayLinearAttention, DifferentialAttention, GatedFF, HashedBigramEmbedding, LayerRun, Linear,
                        RoutedExperts, SequenceModel, SideBySideMixer, StateSpaceMixer, rotary_rates, unroll_layers)
from .base import BaseModelArgs

MIXER_TYPES = ("lightning", "mamba2", "attention")


@dataclass
class ModelArgs(BaseModelArgs):
    vocab: int
    width: int
    layers: List[Dict[str, Any]]
    norm: Dict[str, Any] = field(default_factory=dict)
    embedding: Dict[str, Any] = field(default_factory=dict)
    loop: Optional[Dict[str, Any]] = None
    logit_scale: float = 1.0
    architecture: str = "Nifalorn"
    model_type: str = "nifalorn"

    def __post_init__(self):
        if not self.layers:
            raise ValueError("config 'layers' is empty")
        for i, L in enumerate(self.layers):
            if L.get("type") not in MIXER_TYPES:
                raise NotImplementedError(f"layer {i}: mixer type {L.get('type')!r} is not part of this design")
            mlp = L.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
            m = L["mixer"]
            if L["type"] == "attention" and m["heads"] % m.get("kv_heads", m["heads"]):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            if L["type"] == "mamba2" and (m["heads"] % m.get("groups", 1) or (m["heads"] * m["vdim"]) % m.get("norm_groups", 1)):
                raise ValueError(f"layer {i}: heads must be a multiple of groups and the channels a multiple of norm_groups")
            if L["type"] == "lightning" and len(m["decay"]) != m["heads"]:
                raise ValueError(f"layer {i}: one decay per head")
            if mlp is not None and mlp["kind"] == "moe":
                r = mlp["router"]
                g = r.get("groups") or {}
                count = int(g.get("count", 1))
                keep = int(g.get("keep", count))
                if r["experts"] % count or not (1 <= keep <= count) or keep * (r["experts"] // count) < r["top"]:
                    raise ValueError(f"layer {i}: the expert groups must be equal and the kept ones hold at least 'top' experts")
        if self.loop:
            a, b, n = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
            if not (0 <= a <= b <= len(self.layers)) or n < 1:
                raise ValueError("loop: 0 <= start <= stop <= number of layers and times >= 1")

    @property
    def vocab_size(self) -> int:
        return self.vocab


class Model(SequenceModel):
    block_style = "prenorm"
    kernel_units = "sequence_ssm"

    def __init__(self, args: ModelArgs):
        super().__init__(args)
        W = args.width
        self.eps = float(args.norm.get("eps", 1e-6))
        self.logit_scale = float(args.logit_scale)
        self.embed = HashedBigramEmbedding(args.vocab, W, float(args.embedding.get("scale", 1.0)))
        blocks = []
        for L in args.layers:
            m = L["mixer"]
            if L["type"] == "lightning":
                mixer = SideBySideMixer(W, [DecayLinearAttention(m["heads"], m["dim"], m["vdim"], m["decay"], self.eps)], [1.0])
            elif L["type"] == "mamba2":
                mixer = StateSpaceMixer(W, m["heads"], m["vdim"], m["state"], int(m.get("groups", 1)), int(m.get("norm_groups", 1)),
                                        int(m.get("conv", 1)), self.eps)
            else:
                rot = m.get("rot") or {}
                rates = rotary_rates(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rot.get("dims") else []
                diff = float(m.get("diff", 0.0))
                mixer = DifferentialAttention(W, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], float(m["scale"]),
                                              self.eps, maps=2, rates=rates, chunk=int((m.get("mask") or {}).get("size", 0)),
                                              post=1.0 - diff, unit_norm=True)
            mlp = L.get("mlp")
            if mlp is None:
                ff = None
            elif mlp["kind"] == "dense":
                ff = ActivatedFF(W, int(mlp["ff"]), "relu_squared")
            else:
                r = mlp["router"]
                g = r.get("groups") or {}
                count = int(g.get("count", 1))
                shared = mlp.get("shared") or {}
                ff = RoutedExperts(W, int(r["experts"]), int(r["top"]), int(mlp["expert"]["ff"]), "silu",
                                   shared_ff=int(shared.get("ff", 0)), scoring="sigmoid", groups=(count, int(g.get("keep", count))),
                                   route_scale=float(r.get("scale", 1.0)), shared_gate=True)
            blocks.append((mixer, ff))
        self.mixers = [b[0] for b in blocks]
        loop = args.loop or {}
        order = unroll_layers(len(blocks), int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1)))
        for slot, (i, _) in enumerate(order):
            self.runs.append(LayerRun(i, slot, blocks[i][0], blocks[i][1], f"l{i}.norm1", False,
                                      f"l{i}.norm2" if blocks[i][1] is not None else None))
        self.lm_head = Linear(W, args.vocab)

    # -- parameters ------------------------------------------------------------------------------------------
    @staticmethod
    def _glu_names(prefix: str) -> List[str]:
        return [prefix + "gate", prefix + "up", prefix + "down"]

    def parameter_names(self) -> List[str]:
        names = ["embed", "final.norm", "head"]
        for i, L in enumerate(self.args.layers):
            p = f"l{i}."
            names.append(p + "norm1")
            if L["type"] == "lightning":
                names += [p + "mix." + n for n in ("q", "k", "v", "g", "o", "norm")]
            elif L["type"] == "mamba2":
                names += [p + "mix." + n for n in ("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")]
            else:
                names += [p + "mix." + n for n in ("q", "k", "v", "lq1", "lk1", "lq2", "lk2", "o")]
            mlp = L.get("mlp")
            if mlp is None:
                continue
            names.append(p + "norm2")
            if mlp["kind"] == "dense":
                names += [p + "mlp.up", p + "mlp.down"]
            else:
                for e in range(int(mlp["router"]["experts"])):
                    names += self._glu_names(f"{p}mlp.e{e}.")
                names += [p + "mlp.router", p + "mlp.correction"]
                if (mlp.get("shared") or {}).get("ff"):
                    names += self._glu_names(p + "mlp.shared.") + [p + "mlp.shared.sg"]
        return names

    def load_weights(self, weights: Dict[str, torch.Tensor], device="cuda", strict: bool = True, dtype=None):
        """Matrices go to the device in ``dtype`` (default: as stored); vectors (norm weights, convolution taps and biases,
        decay parameters, picking corrections) as float32, the layer norms' weights with their one added.  Projections that read
        the same input are stacked into one matrix, gate / up rows interleaved for the fused epilogue, the experts stacked per
        layer, the shared expert's gate row under the router's."""
        device = torch.device(device)
        missing = [n for n in self.parameter_names() if n not in weights]
        if missing:
            raise KeyError(f"missing parameters: {missing[:4]}{'...' if len(missing) > 4 else ''}")
        if dtype is None:
            dtype = weights["embed"].dtype
        if dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise TypeError(f"unsupported storage dtype {dtype}")
        self.dtype, self.device = dtype, device

        def put(t):
            return t.to(device=device, dtype=dtype).contiguous()

        def check(name, shape):
            if tuple(weights[name].shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(weights[name].shape)} does not match the config ({tuple(shape)})")

        def vec(name, shape=None, one_plus=False):
            t = weights[name].float()
            if shape is not None:
                check(name, shape)
            return ((1.0 + t) if one_plus else t).to(device).contiguous()

        def glu(ff: GatedFF, prefix: str):
            check(prefix + "gate", (ff.ff, W))
            check(prefix + "up", (ff.ff, W))
            check(prefix + "down", (W, ff.ff))
            ff.gate_up.weight = put(GatedFF.interleave(weights[prefix + "gate"], weights[prefix + "up"]))
            ff.down.weight = put(weights[prefix + "down"])

        a, W = self.args, self.args.width
        check("embed", (a.vocab, W))
        check("head", (a.vocab, W))
        self.embed.weight = put(weights["embed"])
        self.final_norm_w = vec("final.norm", (W,), one_plus=True)
        self.lm_head.weight = put(weights["head"])
        norm1, norm2 = {}, {}
        for i, (L, m) in enumerate(zip(a.layers, self.mixers)):
            p = f"l{i}.mix."
            norm1[i] = vec(f"l{i}.norm1", (W,), one_plus=True)
            if isinstance(m, SideBySideMixer):
                (b,) = m.branches
                check(p + "q", (b.c_qk, W))
                check(p + "k", (b.c_qk, W))
                check(p + "v", (b.c_v, W))
                check(p + "g", (b.c_v, W))
                check(p + "o", (W, b.c_v))
                m.in_proj.weight = put(m.stack_in_proj([torch.cat([weights[p + n] for n in ("q", "k", "v", "g")], 0)]))
                m.o_proj.weight = put(m.stack_o_proj([weights[p + "o"]]))
                b.norm_w = vec(p + "norm", (b.c_v,))
                b.decay = torch.tensor(b.decay_values, dtype=torch.float32, device=device)
            elif isinstance(m, StateSpaceMixer):
                check(p + "in", (m.n_proj, W))
                check(p + "conv", (m.conv_channels, m.taps))
                check(p + "o", (W, m.inner))
                m.in_proj.weight, m.o_proj.weight = put(weights[p + "in"]), put(weights[p + "o"])
                m.conv_w, m.conv_b = vec(p + "conv"), vec(p + "conv.b", (m.conv_channels,))
                m.A_log, m.dt_bias, m.D = vec(p + "A_log", (m.heads,)), vec(p + "dt_bias", (m.heads,)), vec(p + "D", (m.heads,))
                m.norm_w = vec(p + "norm", (m.inner,))
            else:
                check(p + "q", (m.col_k, W))
                check(p + "k", (m.col_v - m.col_k, W))
                check(p + "v", (m.kv_heads * m.vdim, W))
                check(p + "o", (W, m.n_mix))
                for n in ("lq1", "lk1", "lq2", "lk2"):
                    check(p + n, (m.dim,))
                m.in_proj.weight = put(torch.cat([weights[p + n] for n in ("q", "k", "v")], 0))
                m.o_proj.weight = put(weights[p + "o"])
                m.set_lambda(*(weights[p + n].float() for n in ("lq1", "lk1", "lq2", "lk2")), float(L["mixer"].get("diff", 0.0)))
                m.rates = torch.tensor(m.rate_values, dtype=torch.float32, device=device) if m.rate_values else None
        seen = set()
        for r in self.runs:
            r.norm_w = norm1[r.layer]
            ff = r.mlp
            if ff is None:
                continue
            if r.layer in seen:
                r.norm2_w = norm2[r.layer]
                continue
            seen.add(r.layer)
            r.norm2_w = norm2[r.layer] = vec(f"l{r.layer}.norm2", (W,), one_plus=True)
            q = f"l{r.layer}.mlp."
            if isinstance(ff, ActivatedFF):
                check(q + "up", (ff.ff, W))
                check(q + "down", (W, ff.ff))
                ff.up.weight, ff.down.weight = put(weights[q + "up"]), put(weights[q + "down"])
            else:
                check(q + "router", (ff.experts, W))
                has_shared = ff.shared is not None
                if has_shared:
                    if weights[q + "shared.sg"].numel() != W:
                        raise ValueError(f"{q}shared.sg: one row of the model's width")
                    glu(ff.shared, q + "shared.")
                ff.router.weight = put(ff.stack_router(weights[q + "router"], weights[q + "shared.sg"] if has_shared else None))
                ff.router_bias = vec(q + "correction", (ff.experts,))
                for e in range(ff.experts):
                    check(f"{q}e{e}.gate", (ff.ff, W))
                    check(f"{q}e{e}.up", (ff.ff, W))
                    check(f"{q}e{e}.down", (W, ff.ff))
                ff.gate_up = put(torch.stack([GatedFF.interleave(weights[f"{q}e{e}.gate"], weights[f"{q}e{e}.up"])
                                              for e in range(ff.experts)], 0))
                ff.down = put(torch.stack([weights[f"{q}e{e}.down"] for e in range(ff.experts)], 0))
        self._arenas.clear()
        return self

"""Deterministic synthetic checkpoints in the reference's on-disk format.

There is no network for real checkpoints and MLX's threefry PRNG is not reproducible outside MLX
(scripts/build_tiny_model.py:123 in the reference), so every BASELINE config is instantiated from
numpy / torch generators with fixed seeds, in MLX layout: ``*.weight`` uint32 packed codes,
``*.scales`` / ``*.biases`` [N, K/64], norm weights, ``config.json`` with a ``quantization`` block
(utils.py:679), ``model.safetensors`` with metadata {"format": "mlx"} (utils.py:870).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

import numpy as np
import torch

# HF-style configs of the five BASELINE.json configs (+ tiny variants for tests).  Dims: SURVEY 8.
CONFIGS: Dict[str, dict] = {
    # scripts/build_tiny_model.py:70-101 (hidden 64, 8 layers, 4 heads, inter 128, tied, 4-bit g64)
    "tiny": dict(model_type="llama", hidden_size=64, num_hidden_layers=8, intermediate_size=128,
                 num_attention_heads=4, num_key_value_heads=4, rms_norm_eps=1e-6, vocab_size=151936,
                 rope_theta=10000.0, tie_word_embeddings=True, quantization=dict(group_size=64, bits=4)),
    # same shape family with a small vocab so CPU tests stay fast
    "tiny-llama": dict(model_type="llama", hidden_size=128, num_hidden_layers=3, intermediate_size=256,
                       num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=512,
                       rope_theta=10000.0, tie_word_embeddings=False, quantization=dict(group_size=64, bits=4)),
    "tiny-qwen3": dict(model_type="qwen3", hidden_size=128, num_hidden_layers=3, intermediate_size=256,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
                       vocab_size=512, rope_theta=1000000.0, max_position_embeddings=4096,
                       tie_word_embeddings=False, quantization=dict(group_size=64, bits=4)),
    # D=128 / GQA-4 model small enough for the oracle, wide enough for the tensor paths
    "small-llama": dict(model_type="llama", hidden_size=512, num_hidden_layers=2, intermediate_size=1024,
                        num_attention_heads=4, num_key_value_heads=1, rms_norm_eps=1e-5, vocab_size=1024,
                        rope_theta=500000.0, tie_word_embeddings=False, quantization=dict(group_size=64, bits=4)),
    # Phi-3 graph (fused qkv_proj / gate_up_proj checkpoint keys, models/phi3.py); D=128, GQA-2
    "small-phi3": dict(model_type="phi3", hidden_size=512, num_hidden_layers=2, intermediate_size=1024,
                       num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=1024,
                       rope_theta=10000.0, tie_word_embeddings=False, quantization=dict(group_size=64, bits=4)),
    "mistral-7b": dict(model_type="mistral", hidden_size=4096, num_hidden_layers=32, intermediate_size=14336,
                       num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, vocab_size=32000,
                       rope_theta=10000.0, tie_word_embeddings=False, sliding_window=4096,
                       quantization=dict(group_size=64, bits=4)),
    "llama-3-8b": dict(model_type="llama", hidden_size=4096, num_hidden_layers=32, intermediate_size=14336,
                       num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, vocab_size=128256,
                       rope_theta=500000.0, tie_word_embeddings=False, quantization=dict(group_size=64, bits=4)),
    "qwen3-14b": dict(model_type="qwen3", hidden_size=5120, num_hidden_layers=40, intermediate_size=17408,
                      num_attention_heads=40, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                      vocab_size=151936, rope_theta=1000000.0, max_position_embeddings=40960,
                      tie_word_embeddings=False, quantization=dict(group_size=64, bits=4)),
    "llama-3-70b": dict(model_type="llama", hidden_size=8192, num_hidden_layers=80, intermediate_size=28672,
                        num_attention_heads=64, num_key_value_heads=8, rms_norm_eps=1e-5, vocab_size=128256,
                        rope_theta=500000.0, tie_word_embeddings=False, quantization=dict(group_size=64, bits=8)),
}


def get_config(name: str, **overrides) -> dict:
    cfg = json.loads(json.dumps(CONFIGS[name]))
    cfg.update(overrides)
    return cfg


def head_dim_of(cfg: dict) -> int:
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def linear_shapes(cfg: dict) -> Dict[str, tuple]:
    """(N, K) of every QuantizedLinear / QuantizedEmbedding by parameter prefix."""
    h, inter, D = cfg["hidden_size"], cfg["intermediate_size"], head_dim_of(cfg)
    Hq, Hkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    out = {"model.embed_tokens": (cfg["vocab_size"], h)}
    if not cfg.get("tie_word_embeddings", True):
        out["lm_head"] = (cfg["vocab_size"], h)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out[p + "self_attn.q_proj"] = (Hq * D, h)
        out[p + "self_attn.k_proj"] = (Hkv * D, h)
        out[p + "self_attn.v_proj"] = (Hkv * D, h)
        out[p + "self_attn.o_proj"] = (h, Hq * D)
        out[p + "mlp.gate_proj"] = (inter, h)
        out[p + "mlp.up_proj"] = (inter, h)
        out[p + "mlp.down_proj"] = (h, inter)
    return out


def norm_names(cfg: dict):
    names = ["model.norm.weight"]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        names += [p + "input_layernorm.weight", p + "post_attention_layernorm.weight"]
        if cfg["model_type"] == "qwen3":
            names += [p + "self_attn.q_norm.weight", p + "self_attn.k_norm.weight"]
    return names


def weight_bytes_per_step(cfg: dict, scale_bytes: int = 2) -> int:
    """Algorithmic weight bytes of one decode step (SURVEY 8d / BASELINE.md section 3): every linear
    except the embedding table (B gathered rows only) + norm weights."""
    q = cfg["quantization"]
    total = 0
    for name, (n, k) in linear_shapes(cfg).items():
        if name == "model.embed_tokens" and not cfg.get("tie_word_embeddings", True):
            continue
        total += n * k * q["bits"] // 8 + 2 * n * (k // q["group_size"]) * scale_bytes
    total += (2 * cfg["num_hidden_layers"] + 1) * cfg["hidden_size"] * scale_bytes
    return total


def kv_bytes_per_token(cfg: dict, kv_bytes: int = 2) -> int:
    Hkv = cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    return 2 * Hkv * head_dim_of(cfg) * cfg["num_hidden_layers"] * kv_bytes


_TORCH_DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def _stable_seed(seed: int, name: str) -> int:
    h = 1469598103934665603
    for ch in name.encode():
        h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return (h ^ (seed * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF


def random_weights(cfg: dict, seed: int = 1234, dtype: str = "float16", device="cpu",
                   only: Optional[callable] = None) -> Dict[str, torch.Tensor]:
    """Config-2 style generator: uniform random codes, scales = +-U(0.5,1.5)*(2/(2^bits-1))/sqrt(K)
    (random sign exercises MLX's signed scales), biases = -scale*(2^bits-1)/2 + N(0, 0.01/sqrt(K)),
    norm weights 1 + N(0, 0.02).  One torch.Generator per tensor, seeded from (seed, name), so any subset or
    any TP shard of the same model can be regenerated independently on any device type... but NOT across
    device types (CPU and CUDA generators differ): parity tests generate on CPU and copy."""
    q = cfg["quantization"]
    bits, gs = q["bits"], q["group_size"]
    nb = float((1 << bits) - 1)
    tdt = _TORCH_DT[dtype]
    dev = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for name, (n, k) in linear_shapes(cfg).items():
        if only is not None and not only(name):
            continue
        g = torch.Generator(device=dev)
        g.manual_seed(_stable_seed(seed, name))
        words = k * bits // 32
        w = torch.randint(-(2 ** 31), 2 ** 31, (n, words), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
        mag = (torch.rand((n, k // gs), generator=g, device=dev) + 0.5) * (2.0 / nb) / math.sqrt(k)
        sign = torch.where(torch.rand((n, k // gs), generator=g, device=dev) < 0.5, -1.0, 1.0)
        s = (mag * sign).to(tdt)
        b = (-s.float() * (nb / 2) + torch.randn((n, k // gs), generator=g, device=dev) * (0.01 / math.sqrt(k))).to(tdt)
        if name == "model.embed_tokens":                   # embeddings ~ N(0, 1/sqrt(h))-ish spread
            s = (s.float() * math.sqrt(k) * 0.5).to(tdt)
            b = (-s.float() * (nb / 2)).to(tdt)
        out[name + ".weight"], out[name + ".scales"], out[name + ".biases"] = w, s, b
    for name in norm_names(cfg):
        if only is not None and not only(name):
            continue
        g = torch.Generator(device=dev)
        g.manual_seed(_stable_seed(seed, name))
        dim = head_dim_of(cfg) if ("q_norm" in name or "k_norm" in name) else cfg["hidden_size"]
        out[name] = (1.0 + 0.02 * torch.randn((dim,), generator=g, device=dev)).to(tdt)
    return out


def to_phi3_checkpoint(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Per-projection tensors -> the key layout of a Phi-3 checkpoint: rows [q | k | v] as ``self_attn.qkv_proj`` and
    [gate | up] as ``mlp.gate_up_proj`` (reference phi3.py:56-57, 92-96, 117-126)."""
    out = {}
    for name, t in weights.items():
        mod, _, leaf = name.rpartition(".")
        if mod.endswith(("self_attn.k_proj", "self_attn.v_proj", "mlp.up_proj")):
            continue
        if mod.endswith("self_attn.q_proj"):
            base = mod[:-len("q_proj")]
            out[f"{base}qkv_proj.{leaf}"] = torch.cat([weights[f"{base}{p}_proj.{leaf}"] for p in "qkv"], 0)
        elif mod.endswith("mlp.gate_proj"):
            base = mod[:-len("gate_proj")]
            out[f"{base}gate_up_proj.{leaf}"] = torch.cat([t, weights[f"{base}up_proj.{leaf}"]], 0)
        else:
            out[name] = t
    return out


def to_numpy_weights(weights: Dict[str, torch.Tensor]) -> Dict[str, np.ndarray]:
    """torch -> numpy for the oracle: packed int32 -> uint32, bf16/f16 -> float32 (exact)."""
    out = {}
    for k, v in weights.items():
        v = v.detach().cpu()
        if v.dtype == torch.int32:
            out[k] = v.numpy().view(np.uint32)
        else:
            out[k] = v.float().numpy()
    return out


def save_checkpoint(path: str, cfg: dict, weights: Dict[str, torch.Tensor]):
    """Write config.json + model.safetensors the way the reference's save_weights does (utils.py:836-885)."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    tensors = {}
    for k, v in weights.items():
        v = v.detach().cpu().contiguous()
        tensors[k] = v.view(torch.uint32) if v.dtype == torch.int32 else v
    save_file(tensors, os.path.join(path, "model.safetensors"), metadata={"format": "mlx"})


# ---- Dogulorn (models/dogulorn.py): dense bfloat16 checkpoints, tensors l<i>.<part> ---------------------------------------
def dogulorn_config(width: int, ff: int, n_layers: int, heads: int, head_dim: int, q_rank: int, kv_rank: int, window: int,
                    delta_heads: int, delta_kv_heads: int, delta_dim: int, delta_vdim: int, vocab: int = 32000, taps: int = 4,
                    side_dim: int = 64, buckets: int = 65521) -> dict:
    """A config of the design at the sizes of a real model: layers cycle (delta, attention, attention reading the previous
    attention layer's latents); every layer has the feed-forward."""
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    layers, last_own = [], None
    for i in range(n_layers):
        kind = i % 3
        if kind == 0:
            layers.append({"type": "delta", "mlp": dict(mlp), "mixer": {"heads": delta_heads, "kv_heads": delta_kv_heads,
                                                                      "dim": delta_dim, "vdim": delta_vdim, "conv": taps}})
            continue
        m = {"heads": heads, "dim": head_dim, "vdim": head_dim, "q_rank": q_rank, "kv_rank": kv_rank, "mask": {"size": window},
             "scale": head_dim ** -0.5}
        if kind == 2 and last_own is not None:
            m["kv_from"] = last_own
        else:
            last_own = i
        layers.append({"type": "latent_attention", "mlp": dict(mlp), "mixer": m})
    return {"architecture": "Dogulorn", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0, "bigram": {"buckets": buckets, "mul_prev": 1009, "mul_cur": 13}},
            "token_side": {"dim": side_dim}}


def dogulorn_shapes(cfg: dict) -> Dict[str, tuple]:
    """Shape of every tensor of a Dogulorn checkpoint (matrices [out, in])."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        out["bigram"] = (big["buckets"] + 1, W)
    side = cfg.get("token_side")
    if side:
        out["side.embed"] = (V, len(cfg["layers"]) * side["dim"])
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = out[p + "norm1b"] = (W,)
        if L["type"] == "delta":
            H, G, dk, dv, n = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m.get("conv", 1)
            for nm, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + "mix." + nm] = (rows, W)
                out[p + f"mix.{nm}.conv"] = (rows, n)
            out[p + "mix.b"] = out[p + "mix.a"] = (H, W)
            out[p + "mix.g"] = (H * dv, W)
            out[p + "mix.o"] = (W, H * dv)
            out[p + "mix.A_log"] = out[p + "mix.dt_bias"] = (H,)
            out[p + "mix.norm"] = (dv,)
        else:
            H, dk, dv, rq, rk = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            out[p + "mix.dq"], out[p + "mix.dq.norm"], out[p + "mix.uq"] = (rq, W), (rq,), (H * dk, rq)
            if m.get("kv_from") is None:
                out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = (rk, W), (rk,)
            out[p + "mix.uk"], out[p + "mix.uv"], out[p + "mix.o"] = (H * dk, rk), (H * dv, rk), (W, H * dv)
        if L.get("mlp") is not None:
            ff = L["mlp"]["ff"]
            out[p + "norm2"] = out[p + "norm2b"] = (W,)
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (ff, W)
            out[p + "mlp.down"] = (W, ff)
        if side:
            out[p + "side.gate"], out[p + "side.proj"], out[p + "side.norm"] = (side["dim"], W), (W, side["dim"]), (W,)
    return out


def dogulorn_random_weights(cfg: dict, seed: int = 1234, device="cpu") -> Dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, 1/in), norm weights 1 + N(0, 0.02), decay parameters spread so that heads forget at
    different speeds.  One generator per tensor, seeded from (seed, name)."""
    dev = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in dogulorn_shapes(cfg).items():
        g = torch.Generator(device=dev)
        g.manual_seed(_stable_seed(seed, name))
        if len(shape) == 2 and not name.endswith(".conv"):
            t = torch.randn(shape, generator=g, device=dev) / math.sqrt(shape[1])
            if name in ("embed", "bigram", "side.embed"):
                t = t * math.sqrt(shape[1]) * 0.5
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=g, device=dev) * 0.5
        elif name.endswith("A_log"):
            t = torch.rand(shape, generator=g, device=dev) * 3.0 - 2.0
        elif name.endswith("dt_bias"):
            t = torch.randn(shape, generator=g, device=dev)
        else:
            t = 1.0 + 0.02 * torch.randn(shape, generator=g, device=dev)
        out[name] = t.to(torch.bfloat16)
    return out


# ---- Pupopel ----------------------------------------------------------------------------------------------------------------
def pupopel_config(width: int, ff: int, n_layers: int, heads: int, head_dim: int, delta_heads: int, delta_kv_heads: int,
                   delta_dim: int, delta_vdim: int, kv_heads: Optional[int] = None, linear_heads: Optional[int] = None,
                   experts: int = 16, top: int = 2, vocab: int = 32000, taps: int = 4, loop_times: int = 1, **unused) -> dict:
    """A config of the design at the sizes of a real model: layers cycle (channel-delta + dense feed-forward, attention beside
    linear attention + routed experts, the same + dense); the routed layer's active experts and its shared expert together
    have the dense layer's hidden size.  All layers form one span that runs ``loop_times`` times."""
    kv_heads = kv_heads or max(1, heads // 4)
    linear_heads = linear_heads or heads
    layers = []
    for i in range(n_layers):
        kind = i % 3
        if kind == 0:
            mixer = {"heads": delta_heads, "kv_heads": delta_kv_heads, "dim": delta_dim, "vdim": delta_vdim, "conv": taps}
            layers.append({"type": "channel_delta", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}})
            continue
        left = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
                "q_temp": {"coef": 0.1, "every": 512}}
        right = {"heads": linear_heads, "dim": head_dim, "vdim": head_dim,
                 "decay": [1.0 - 2.0 ** (-4.0 - 6.0 * h / max(1, linear_heads - 1)) for h in range(linear_heads)]}
        mixer = {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0}
        if kind == 1:
            mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff // (2 * top)}, "shared": {"ff": ff // 2}}
        else:
            mlp = {"kind": "dense", "ff": ff}
        layers.append({"type": "parallel", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Pupopel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6},
            "loop": {"start": 0, "stop": n_layers, "times": loop_times}}


def pupopel_shapes(cfg: dict, rank: Optional[int] = None) -> Dict[str, tuple]:
    """Shape of every tensor of a Pupopel checkpoint (matrices [out, in]); ``rank``: inner size of the low-rank decay and gate
    projections (default width / 16, at least 8)."""
    W, V = cfg["width"], cfg["vocab"]
    r = rank or max(8, W // 16)
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    loop = cfg.get("loop")
    if loop and loop["stop"] > loop["start"]:
        out["loop.in"] = (W, 2 * W)

    def glu(p, ff):
        out[p + "gate"] = out[p + "up"] = (ff, W)
        out[p + "down"] = (W, ff)

    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        out[f"l{i}.norm1"] = (W,)
        if L["type"] == "channel_delta":
            H, G, dk, dv, n = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m.get("conv", 1)
            for nm, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + nm] = (rows, W)
                out[p + nm + ".conv"] = (rows, n)
            out[p + "b"] = (H, W)
            out[p + "a1"], out[p + "a2"] = (r, W), (H * dk, r)
            out[p + "g1"], out[p + "g2"] = (r, W), (H * dv, r)
            out[p + "A_log"], out[p + "dt_bias"], out[p + "norm"] = (H,), (H * dk,), (dv,)
            out[p + "o"] = (W, H * dv)
        else:
            a, b = m["left"], m["right"]
            G = a.get("kv_heads", a["heads"])
            out[p + "left.q"], out[p + "left.k"], out[p + "left.v"] = (a["heads"] * a["dim"], W), (G * a["dim"], W), (G * a["vdim"], W)
            out[p + "left.q.norm"] = out[p + "left.k.norm"] = (a["dim"],)
            out[p + "left.sink"] = (a["heads"],)
            out[p + "left.o"] = (W, a["heads"] * a["vdim"])
            cq, cv = b["heads"] * b["dim"], b["heads"] * b["vdim"]
            out[p + "right.q"] = out[p + "right.k"] = (cq, W)
            out[p + "right.v"] = out[p + "right.g"] = (cv, W)
            out[p + "right.norm"], out[p + "right.o"] = (cv,), (W, cv)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        q = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            glu(q, mlp["ff"])
        else:
            for e in range(mlp["router"]["experts"]):
                glu(f"{q}e{e}.", mlp["expert"]["ff"])
            out[q + "router"], out[q + "router.b"] = (mlp["router"]["experts"], W), (mlp["router"]["experts"],)
            if (mlp.get("shared") or {}).get("ff"):
                glu(q + "shared.", mlp["shared"]["ff"])
    return out


def pupopel_random_weights(cfg: dict, seed: int = 1234, device="cpu", rank: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, 1/in), norm offsets N(0, 0.02) (weights that multiply directly: 1 + that), sinks and
    router biases N(0, 1) / N(0, 0.1), decay parameters spread so that channels forget at different speeds."""
    dev = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in pupopel_shapes(cfg, rank).items():
        g = torch.Generator(device=dev)
        g.manual_seed(_stable_seed(seed, name))
        if len(shape) == 2 and not name.endswith(".conv"):
            t = torch.randn(shape, generator=g, device=dev) / math.sqrt(shape[1])
            if name == "embed":
                t = t * math.sqrt(shape[1]) * 0.5
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=g, device=dev) * 0.5
        elif name.endswith("A_log"):
            t = torch.rand(shape, generator=g, device=dev) * 3.0 - 2.0
        elif name.endswith("dt_bias") or name.endswith("sink"):
            t = torch.randn(shape, generator=g, device=dev)
        elif name.endswith("router.b"):
            t = 0.1 * torch.randn(shape, generator=g, device=dev)
        elif name.endswith("norm1") or name == "final.norm":
            t = 0.02 * torch.randn(shape, generator=g, device=dev)
        else:
            t = 1.0 + 0.02 * torch.randn(shape, generator=g, device=dev)
        out[name] = t.to(torch.bfloat16)
    return out


# ---- Nifalorn ---------------------------------------------------------------------------------------------------------------
def nifalorn_config(width: int, ff: int, n_layers: int, heads: int, head_dim: int, kv_heads: Optional[int] = None,
                    ssm_head_dim: int = 64, ssm_state: int = 128, ssm_groups: int = 8, experts: int = 16, top: int = 2,
                    expert_groups: int = 4, keep_groups: int = 2, chunk: int = 8192, vocab: int = 32000, taps: int = 4,
                    loop_times: int = 1, **unused) -> dict:
    """A config of the design at the sizes of a real model: layers cycle (state-space mixer of twice the width + dense
    feed-forward, two-map attention + routed experts, constant-decay linear attention + dense); each score map has half the
    head size, the values the whole; the routed layer's active experts and its shared expert together have the dense layer's
    hidden size.  All layers form one span that runs ``loop_times`` times."""
    kv_heads = kv_heads or max(1, heads // 4)
    moe = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": expert_groups, "keep": keep_groups}},
           "expert": {"ff": ff // (2 * top)}, "shared": {"ff": ff // 2}}
    layers = []
    for i in range(n_layers):
        kind = i % 3
        if kind == 0:
            ssm_heads = 2 * width // ssm_head_dim
            mixer = {"heads": ssm_heads, "vdim": ssm_head_dim, "state": ssm_state, "groups": ssm_groups, "norm_groups": ssm_groups, "conv": taps}
            layers.append({"type": "mamba2", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}})
        elif kind == 1:
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim // 2, "vdim": head_dim, "scale": (head_dim // 2) ** -0.5, "diff": 0.6,
                     "mask": {"size": chunk},
                     "rot": {"dims": head_dim // 2, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
            layers.append({"type": "attention", "mixer": mixer, "mlp": moe})
        else:
            mixer = {"heads": heads, "dim": head_dim, "vdim": head_dim,
                     "decay": [1.0 - 2.0 ** (-4.0 - 6.0 * h / max(1, heads - 1)) for h in range(heads)]}
            layers.append({"type": "lightning", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Nifalorn", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "logit_scale": 1.0, "loop": {"start": 0, "stop": n_layers, "times": loop_times}}


def nifalorn_shapes(cfg: dict) -> Dict[str, tuple]:
    """Shape of every tensor of a Nifalorn checkpoint (matrices [out, in])."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}

    def glu(p, ff):
        out[p + "gate"] = out[p + "up"] = (ff, W)
        out[p + "down"] = (W, ff)

    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        out[f"l{i}.norm1"] = (W,)
        if L["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out[p + "in"] = (2 * inner + 2 * gn + m["heads"], W)
            out[p + "conv"], out[p + "conv.b"] = (inner + 2 * gn, m.get("conv", 1)), (inner + 2 * gn,)
            out[p + "dt_bias"] = out[p + "A_log"] = out[p + "D"] = (m["heads"],)
            out[p + "norm"], out[p + "o"] = (inner,), (W, inner)
        elif L["type"] == "attention":
            G = m.get("kv_heads", m["heads"])
            out[p + "q"], out[p + "k"], out[p + "v"] = (m["heads"] * 2 * m["dim"], W), (G * 2 * m["dim"], W), (G * m["vdim"], W)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[p + n] = (m["dim"],)
            out[p + "o"] = (W, m["heads"] * m["vdim"])
        else:
            cq, cv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out[p + "q"] = out[p + "k"] = (cq, W)
            out[p + "v"] = out[p + "g"] = (cv, W)
            out[p + "norm"], out[p + "o"] = (cv,), (W, cv)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        q = f"l{i}.mlp."
        out[f"l{i}.norm2"] = (W,)
        if mlp["kind"] == "dense":
            out[q + "up"], out[q + "down"] = (mlp["ff"], W), (W, mlp["ff"])
        else:
            for e in range(mlp["router"]["experts"]):
                glu(f"{q}e{e}.", mlp["expert"]["ff"])
            out[q + "router"], out[q + "correction"] = (mlp["router"]["experts"], W), (mlp["router"]["experts"],)
            if (mlp.get("shared") or {}).get("ff"):
                glu(q + "shared.", mlp["shared"]["ff"])
                out[q + "shared.sg"] = (1, W)
    return out


def nifalorn_random_weights(cfg: dict, seed: int = 1234, device="cpu") -> Dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, 1/in), norm offsets N(0, 0.02) (weights that multiply directly: 1 + that), convolution
    taps N(0, 0.25), decay parameters spread so that heads forget at different speeds, small picking corrections."""
    dev = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in nifalorn_shapes(cfg).items():
        g = torch.Generator(device=dev)
        g.manual_seed(_stable_seed(seed, name))
        leaf = name.rsplit(".", 1)[-1]
        if len(shape) == 2 and leaf != "conv":
            t = torch.randn(shape, generator=g, device=dev) / math.sqrt(shape[1])
            if name == "embed":
                t = t * math.sqrt(shape[1]) * 0.5
        elif leaf == "conv":
            t = torch.randn(shape, generator=g, device=dev) * 0.5
        elif leaf == "A_log":
            t = torch.rand(shape, generator=g, device=dev) * 3.0 - 2.0
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g, device=dev) - 1.0
        elif leaf in ("correction", "b", "lq1", "lk1", "lq2", "lk2"):
            t = 0.1 * torch.randn(shape, generator=g, device=dev)
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            t = 0.02 * torch.randn(shape, generator=g, device=dev)
        else:                                   # mix.norm, D
            t = 1.0 + 0.02 * torch.randn(shape, generator=g, device=dev)
        out[name] = t.to(torch.bfloat16)
    return out


# ---- Dapupel ----------------------------------------------------------------------------------------------------------------
def dapupel_config(width: int, ff: int, n_layers: int, heads: int, head_dim: int, q_rank: int, kv_rank: int, window: int,
                   delta_heads: int, delta_kv_heads: int, delta_dim: int, delta_vdim: int, kv_heads: Optional[int] = None,
                   rot_dim: int = 64, experts: int = 16, top: int = 2, streams: int = 4, canon_taps: int = 4, vocab: int = 32000,
                   taps: int = 4, **unused) -> dict:
    """A config of the design at the sizes of a real model: layers cycle (channel-delta, latent attention with a rotated key
    part, windowed attention over its keys), every one with routed experts whose active ones together have the hidden size
    ``ff``; ``streams`` copies of the residual stream and an input convolution of ``canon_taps`` taps."""
    kv_heads = kv_heads or max(1, heads // 4)
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff // top, "limit": 7.0}}
    layers = []
    for i in range(n_layers):
        kind = i % 3
        if kind == 0:
            mixer = {"heads": delta_heads, "kv_heads": delta_kv_heads, "dim": delta_dim, "vdim": delta_vdim, "conv": taps}
            layers.append({"type": "channel_delta", "mixer": mixer, "mlp": moe})
        elif kind == 1:
            mixer = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "q_rank": q_rank, "kv_rank": kv_rank,
                     "scale": (head_dim + rot_dim) ** -0.5,
                     "rot": {"dims": rot_dim, "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
            layers.append({"type": "latent_attention", "mixer": mixer, "mlp": moe})
        else:
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "softcap": 50.0,
                     "mask": {"size": window}, "conv": taps}
            layers.append({"type": "attention", "mixer": mixer, "mlp": moe})
    return {"architecture": "Dapupel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6}, "streams": streams,
            "canon": {"taps": canon_taps}}


def dapupel_shapes(cfg: dict, rank: Optional[int] = None) -> Dict[str, tuple]:
    """Shape of every tensor of a Dapupel checkpoint (matrices [out, in]); ``rank``: inner size of the low-rank decay and gate
    projections (default width / 16, at least 8)."""
    W, V, S, ct = cfg["width"], cfg["vocab"], cfg["streams"], cfg["canon"]["taps"]
    r = rank or max(8, W // 16)
    out = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,), "final.norm.alpha": ()}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        for q in ("1", "2") if L.get("mlp") is not None else ("1",):
            out[f"l{i}.norm{q}"] = out[f"l{i}.norm{q}.b"] = (W,)
            out[f"l{i}.norm{q}.alpha"] = ()
            out[f"l{i}.hc{q}.in"] = out[f"l{i}.hc{q}.out"] = (S,)
            out[f"l{i}.hc{q}.mix"] = (S, S)
            out[f"l{i}.canon{q}"] = (W, ct)
        if L["type"] == "channel_delta":
            ck, cv, n = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m.get("conv", 1)
            out[p + "q"] = out[p + "k"] = (ck, W)
            out[p + "q.conv"] = out[p + "k.conv"] = (ck, n)
            out[p + "v"], out[p + "v.conv"] = (cv, W), (cv, n)
            out[p + "b"], out[p + "A_log"], out[p + "norm"] = (m["heads"], W), (m["heads"],), (m["vdim"],)
            out[p + "a1"], out[p + "a2"], out[p + "dt_bias"] = (r, W), (m["heads"] * m["dim"], r), (m["heads"] * m["dim"],)
            out[p + "g1"], out[p + "g2"], out[p + "o"] = (r, W), (cv, r), (W, cv)
        elif L["type"] == "latent_attention":
            H = m["heads"]
            out[p + "dq"], out[p + "dq.norm"], out[p + "uq"] = (m["q_rank"], W), (m["q_rank"],), (H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            out[p + "dkv"], out[p + "dkv.norm"] = (m["kv_rank"] + m["rot_dim"], W), (m["kv_rank"],)
            out[p + "uk"], out[p + "uv"], out[p + "o"] = (H * m["dim"], m["kv_rank"]), (H * m["vdim"], m["kv_rank"]), (W, H * m["vdim"])
        else:
            cq, ck, n = m["heads"] * m["dim"], m.get("kv_heads", m["heads"]) * m["dim"], m.get("conv", 1)
            out[p + "q"], out[p + "k"], out[p + "g"], out[p + "o"] = (cq, W), (ck, W), (cq, W), (W, cq)
            out[p + "q.conv"], out[p + "k.conv"] = (cq, n), (ck, n)
            out[p + "r1"] = out[p + "r2"] = (m["heads"],)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        q = f"l{i}.mlp."
        for e in range(mlp["router"]["experts"]):
            out[f"{q}e{e}.gate"] = out[f"{q}e{e}.up"] = (mlp["expert"]["ff"], W)
            out[f"{q}e{e}.down"] = (W, mlp["expert"]["ff"])
        out[q + "router"] = (mlp["router"]["experts"], W)
    return out


def dapupel_random_weights(cfg: dict, seed: int = 1234, device="cpu", rank: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, 1/in), norm weights near one with small offsets, stream weights near an even read and an
    identity write, convolution taps N(0, 0.25) (the mixers' own with a one on the current token), decay parameters spread so that
    channels forget at different speeds."""
    dev = torch.device(device)
    S = cfg["streams"]
    out: Dict[str, torch.Tensor] = {}
    for name, shape in dapupel_shapes(cfg, rank).items():
        g = torch.Generator(device=dev)
        g.manual_seed(_stable_seed(seed, name))
        parts = name.split(".")
        leaf = parts[-1]
        if leaf == "alpha":
            t = torch.full(shape, 0.5, device=dev)
        elif len(parts) >= 2 and parts[-2].startswith("hc"):
            if leaf == "mix":
                t = torch.eye(S, device=dev) + 0.05 * torch.randn(shape, generator=g, device=dev)
            elif leaf == "in":
                t = torch.full(shape, 1.0 / S, device=dev) + 0.02 * torch.randn(shape, generator=g, device=dev)
            else:
                t = 1.0 + 0.05 * torch.randn(shape, generator=g, device=dev)
        elif leaf.startswith("canon"):
            t = torch.randn(shape, generator=g, device=dev) * 0.25
        elif leaf == "conv":
            t = torch.randn(shape, generator=g, device=dev) * 0.5
            if "q" in parts or "k" in parts:
                t[:, -1] += 1.0
        elif leaf in ("r1", "r2"):
            t = torch.rand(shape, generator=g, device=dev) * 0.5 + 0.05
        elif leaf == "A_log":
            t = torch.rand(shape, generator=g, device=dev) * 3.0 - 2.0
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g, device=dev)
        elif leaf == "b" and parts[-2].startswith("norm"):
            t = 0.02 * torch.randn(shape, generator=g, device=dev)
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g, device=dev) / math.sqrt(shape[1])
            if name == "embed":
                t = t * math.sqrt(shape[1]) * 0.5
        else:                                   # norm weights
            t = 1.0 + 0.02 * torch.randn(shape, generator=g, device=dev)
        out[name] = t.to(torch.bfloat16)
    return out

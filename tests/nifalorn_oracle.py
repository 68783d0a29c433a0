"""Slow float64 statement of the Nifalorn design, one function per mechanism, whole sequences on the CPU.

Written from the design's equations; shares no code with mlx_parallm_b200 (it does not import it).  Notation: T tokens,
W width, x the residual stream [T, W], weights ``P[name]`` stored [out, in] and applied as a @ P.T.

The design: pre-norm layers x <- x + mixer(n1(x)); x <- x + ff(n2(x)) whose norm weights are stored as offsets from one; a
span of layers that may run several times on the same weights (a state per pass); three mixers -- a constant-decay linear
attention, a selective state-space layer with a short convolution, and a two-map ("differential") softmax attention over
position chunks with a partial interleaved rotation; feed-forwards that are dense (squared relu) or a routed mixture whose
experts are picked by sigmoid scores inside the best expert groups, beside a gated shared expert.
"""
import math

import torch

F64 = torch.float64


# ---- elementwise --------------------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    return torch.clamp(z, min=0.0).pow(2)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u, taps_w, bias):
    """out[t, c] = bias[c] + sum_j taps_w[c, j] u[t - (n - 1 - j), c], zeros before the start; u [T, C], taps_w [C, n]."""
    T, C = u.shape
    n = taps_w.shape[1]
    out = bias.unsqueeze(0).repeat(T, 1).to(F64)
    for t in range(T):
        for j in range(n):
            s = t - (n - 1 - j)
            if s >= 0:
                out[t] += taps_w[:, j] * u[s]
    return out


# ---- mixers -------------------------------------------------------------------------------------------------------------
def lightning(h, P, pre, m, eps):
    """Per head S_t = lambda S_{t-1} + k_t v_t^T, o_t = S_t^T q_t with q, k, v = silu of their projections; all heads
    rms-normed as one vector (plain weight), gated by a sigmoid, projected."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ P[pre + "q"].T).view(T, H, dk)
    k = silu(h @ P[pre + "k"].T).view(T, H, dk)
    v = silu(h @ P[pre + "v"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    o = rms_unit(out.reshape(T, H * dv), eps) * P[pre + "norm"] * torch.sigmoid(h @ P[pre + "g"].T)
    return o @ P[pre + "o"].T


def state_space(h, P, pre, m, eps):
    """Selective state-space layer.  One projection gives [z | x | B | C | dt]; x, B, C pass a short causal convolution with
    bias and silu; dt = softplus(dt + dt_bias).  Per head (reading the B / C of its group), state S [N, dv] from zero:
    S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T;  y_t = S_t^T C_t + D x_t.  Then y * silu(z), rms norm in equal
    parts of the channels, a weight, the output projection."""
    T = h.shape[0]
    H, dv, N, G, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * dv
    u = h @ P[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P[pre + "conv"], P[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + P[pre + "dt_bias"])                                         # [T, H]
    y = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        rate = torch.exp(P[pre + "A_log"][head])
        S = torch.zeros(N, dv, dtype=F64)
        for t in range(T):
            S = torch.exp(-rate * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + P[pre + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * P[pre + "norm"]
    return y @ P[pre + "o"].T


def rotation_rates(rot):
    """f_i = base^(-2i/n), i < n/2, with long wavelengths slowed down: wavelength l = 2 pi / f; f kept where l < L/high,
    f / factor where l > L/low, a straight blend of the two in between (L the original context length)."""
    n = int(rot["dims"])
    f = [float(rot["base"]) ** (-2.0 * i / n) for i in range(n // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            l = 2.0 * math.pi / fi
            if l < sc["original"] / sc["high"]:
                out.append(fi)
            elif l > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / l - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate_pairs(u, rates, start=0):
    """u [T, heads, d]: dimensions (2i, 2i+1), i < len(rates), of the token at position p turn by the angle p * rates[i]."""
    T = u.shape[0]
    n = 2 * rates.numel()
    ang = (torch.arange(T, dtype=F64) + start).view(T, 1, 1) * rates.view(1, 1, -1)
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = u[..., 0:n:2], u[..., 1:n:2]
    out = u.clone()
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


def differential_attention(h, P, pre, m, eps):
    """Two softmax attentions ("maps") per head over the same values, o = a1 - lambda a2 with one lambda per layer,
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff; o is divided by its root mean square and scaled by 1 - diff.  Position i
    sees j <= i of its own chunk of ``mask.size`` positions.  The first rot.dims dimensions of every map of q and k are rotated."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ P[pre + "q"].T).view(T, H, 2, d)
    k = (h @ P[pre + "k"].T).view(T, G, 2, d)
    v = (h @ P[pre + "v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        rates = rotation_rates(rot)
        q = rotate_pairs(q.reshape(T, H * 2, d), rates).view(T, H, 2, d)
        k = rotate_pairs(k.reshape(T, G * 2, d), rates).view(T, G, 2, d)
    lam = (torch.exp((P[pre + "lq1"] * P[pre + "lk1"]).sum()) - torch.exp((P[pre + "lq2"] * P[pre + "lk2"]).sum()) + m["diff"])
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    hidden = j > i
    size = (m.get("mask") or {}).get("size")
    if size:
        hidden = hidden | ((i // size) != (j // size))
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        kv = head // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, head, mp] @ k[:, kv, mp].T) * m["scale"]
            s = s.masked_fill(hidden, -math.inf)
            a.append(torch.softmax(s, -1) @ v[:, kv])
        out[:, head] = rms_unit(a[0] - lam * a[1], eps) * (1.0 - m["diff"])
    return out.reshape(T, H * dv) @ P[pre + "o"].T


# ---- feed-forwards --------------------------------------------------------------------------------------------------------
def dense_ff(h, P, pre):
    return relu_squared(h @ P[pre + "up"].T) @ P[pre + "down"].T


def gated_expert(h, P, pre):
    return (silu(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def route(h, P, pre, r):
    """-> (chosen experts [T, top], weights [T, top]).  s = sigmoid(router logits); picks by s + correction among the experts
    of the ``keep`` groups whose two best picking scores sum highest; weights s / sum(s of the chosen) * scale."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ P[pre + "router"].T)
    pick = s + P[pre + "correction"]
    grp = r.get("groups") or {}
    count, keep = int(grp.get("count", 1)), int(grp.get("keep", grp.get("count", 1)))
    if count > 1:
        T = h.shape[0]
        per = E // count
        gs = pick.view(T, count, per).topk(min(2, per), -1).values.sum(-1)
        kept = torch.zeros(T, count, dtype=torch.bool)
        kept.scatter_(1, gs.topk(keep, -1).indices, True)
        pick = pick.masked_fill(~kept.repeat_interleave(per, 1), -math.inf)
    ids = pick.topk(top, -1).indices
    w = s.gather(1, ids)
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20) * r["scale"]


def routed_ff(h, P, pre, mlp):
    ids, w = route(h, P, pre, mlp["router"])
    out = torch.zeros(h.shape[0], P[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for c in range(ids.shape[1]):
            out[t] += w[t, c] * gated_expert(h[t:t + 1], P, f"{pre}e{int(ids[t, c])}.")[0]
    if (mlp.get("shared") or {}).get("ff"):
        out = out + torch.sigmoid(h @ P[pre + "shared.sg"].T) * gated_expert(h, P, pre + "shared.")
    return out


# ---- the model ------------------------------------------------------------------------------------------------------------
MIXERS = {"lightning": lightning, "mamba2": state_space, "attention": differential_attention}


def layer_runs(cfg):
    """Layer indices in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return list(range(n))
    a, b = loop["start"], loop["stop"]
    return list(range(a)) + list(range(a, b)) * loop["times"] + list(range(b, n))


def forward(cfg, P, tokens, tap=None):
    """Logits [T, vocab] of one sequence from its first token; ``tap(run, x)`` sees the residual stream after every layer run."""
    P = {k: v.to(F64) for k, v in P.items()}
    eps = cfg["norm"]["eps"]
    x = P["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for run, i in enumerate(layer_runs(cfg)):
        L = cfg["layers"][i]
        p = f"l{i}."
        x = x + MIXERS[L["type"]](norm_one_plus(x, P[p + "norm1"], eps), P, p + "mix.", L["mixer"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            hn = norm_one_plus(x, P[p + "norm2"], eps)
            x = x + (dense_ff(hn, P, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(hn, P, p + "mlp.", mlp))
        if tap is not None:
            tap(run, x)
    return (norm_one_plus(x, P["final.norm"], eps) @ P["head"].T) * cfg["logit_scale"]


# ---- small configurations and random weights for the tests ------------------------------------------------------------------
def dense_mlp(ff):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts, top, ff, groups=(1, 1), scale=1.0, shared_ff=0):
    mlp = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared_ff:
        mlp["shared"] = {"ff": shared_ff}
    return mlp


def lightning_layer(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def ssm_layer(heads, vdim, state, groups, norm_groups, conv, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups,
                                        "conv": conv}, "mlp": mlp}


def attention_layer(heads, kv_heads, dim, vdim, scale, diff, chunk, rot_dims, base=10000.0, scaling=None, mlp=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
                                           "mask": {"size": chunk}, "rot": rot}, "mlp": mlp}


def make_config(layers, vocab=40, width=32, eps=1e-5, loop=None, embed_scale=1.0, logit_scale=1.0):
    cfg = {"architecture": "Nifalorn", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "embedding": {"scale": embed_scale}, "logit_scale": logit_scale}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = (W,)
        if L["type"] == "lightning":
            ck, cv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            s.update({p + "mix.q": (ck, W), p + "mix.k": (ck, W), p + "mix.v": (cv, W), p + "mix.g": (cv, W), p + "mix.o": (W, cv),
                      p + "mix.norm": (cv,)})
        elif L["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            s.update({p + "mix.in": (2 * inner + 2 * gn + m["heads"], W), p + "mix.conv": (inner + 2 * gn, m["conv"]),
                      p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (m["heads"],), p + "mix.A_log": (m["heads"],),
                      p + "mix.D": (m["heads"],), p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
        else:
            s.update({p + "mix.q": (m["heads"] * 2 * m["dim"], W), p + "mix.k": (m["kv_heads"] * 2 * m["dim"], W),
                      p + "mix.v": (m["kv_heads"] * m["vdim"], W), p + "mix.o": (W, m["heads"] * m["vdim"])})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                s[p + "mix." + n] = (m["dim"],)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        s[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            s.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            continue
        E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        for e in range(E):
            s.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
        s.update({p + "mlp.router": (E, W), p + "mlp.correction": (E,)})
        sf = (mlp.get("shared") or {}).get("ff")
        if sf:
            s.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf),
                      p + "mlp.shared.sg": (1, W)})
    return s


def random_weights(cfg, seed=0, dtype=torch.float32):
    """Random tensors of every shape, scaled so that each branch moves the stream visibly; values are rounded to bfloat16
    (kept in ``dtype``) so that a bfloat16 model holds the same numbers."""
    g = torch.Generator().manual_seed(seed)
    P = {}
    for name, shape in shapes(cfg).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2 and leaf not in ("conv",):
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[1]))
            if leaf == "router":
                t = t * 2.0
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            t = torch.randn(shape, generator=g) * 0.2
        elif leaf == "norm":
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif leaf == "A_log":
            t = torch.rand(shape, generator=g) * 1.5 - 1.0
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) * 0.7 - 0.5
        elif leaf == "D":
            t = torch.randn(shape, generator=g) * 0.5 + 0.5
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = torch.randn(shape, generator=g) * 0.3
        elif leaf == "correction":
            t = torch.randn(shape, generator=g) * 0.3
        else:                                   # conv.b
            t = torch.randn(shape, generator=g) * 0.2
        P[name] = t.to(torch.bfloat16).to(dtype)
    return P


def logits_error(got, want):
    """Worst position: rms over the vocabulary of the centred difference, relative to the rms of the centred expected row."""
    got, want = got.to(F64).cpu(), want.to(F64).cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())

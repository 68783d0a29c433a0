"""Slow float64 statement of the Dapupel design, one function per mechanism, whole sequences on the CPU.

Written from the design's equations; shares no code with mlx_parallm_b200 (it does not import it).  Notation: T tokens,
W width, weights ``P[name]`` stored [out, in] and applied as a @ P.T.

The design: ``streams`` copies of the residual stream ("hyper-connections": every sublayer reads a weighted sum of the copies
and writes back through a mixing matrix and an output vector); a tanh norm without statistics; a short causal convolution
added to what every sublayer reads; three mixers -- a delta rule whose decay is a vector over the key channels, latent
attention with a rotated key part shared by the heads (frequencies stretched for long contexts), and windowed grouped
attention without rotation whose values are its keys, with capped scores and a logarithmic distance penalty; a routed
feed-forward whose sigmoid scores multiply the experts' inputs; the output reads the embedding table.
"""
import math

import torch

F64 = torch.float64


# ---- elementwise --------------------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def tanh_norm(x, P, name):
    """tanh(alpha x) w + b: no mean, no variance."""
    return torch.tanh(P[name + ".alpha"] * x) * P[name] + P[name + ".b"]


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u, taps_w):
    """out[t, c] = sum_j taps_w[c, j] u[t - (n - 1 - j), c], zeros before the start; u [T, C], taps_w [C, n]."""
    T, C = u.shape
    n = taps_w.shape[1]
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(n):
            s = t - (n - 1 - j)
            if s >= 0:
                out[t] += taps_w[:, j] * u[s]
    return out


def with_input_conv(n, taps_w):
    """What a sublayer reads: its normed input plus the convolution of it."""
    return n + causal_conv(n, taps_w)


# ---- mixers -------------------------------------------------------------------------------------------------------------
def channel_delta(h, P, pre, m, eps):
    """q, k (kv_heads x dim) and v (heads x vdim) pass a short convolution and silu; q, k become unit vectors per head
    (1e-6 inside the root), q times dim^-1/2.  Per head, state S [dim, vdim] from zero:
    S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ P[pre + "q"].T, P[pre + "q.conv"])).view(T, G, dk)
    k = silu(causal_conv(h @ P[pre + "k"].T, P[pre + "k.conv"])).view(T, G, dk)
    v = silu(causal_conv(h @ P[pre + "v"].T, P[pre + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ P[pre + "b"].T)                                     # [T, H]
    step = softplus((h @ P[pre + "a1"].T) @ P[pre + "a2"].T + P[pre + "dt_bias"]).view(T, H, dk)
    g = torch.exp(-torch.exp(P[pre + "A_log"]).view(1, H, 1) * step)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        kh = head // (H // G)
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = g[t, head].unsqueeze(1) * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, head] = S.T @ q[t, kh]
    gate = torch.sigmoid((h @ P[pre + "g1"].T) @ P[pre + "g2"].T).view(T, H, dv)
    o = rms_unit(out, eps) * P[pre + "norm"] * gate
    return o.reshape(T, H * dv) @ P[pre + "o"].T


def stretched_rates(rot):
    """Angle per position of pair i < dims / 2, and the factor on cos and sin.  f_i = base^(-2i/dims); with
    d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1): rate_i = r_i f_i / factor + (1 - r_i) f_i; magnitude 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def d(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(sc["fast"]))), 0)
    hi = min(math.ceil(d(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * r + fi * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(u, rates, mag):
    """u [T, ..., 2 n]: dimensions (2i, 2i+1) of position p turn by p rates[i]; cos and sin carry the factor ``mag``."""
    T = u.shape[0]
    n = len(rates)
    ang = torch.arange(T, dtype=F64).unsqueeze(1) * torch.tensor(rates, dtype=F64).unsqueeze(0)       # [T, n]
    shape = [T] + [1] * (u.dim() - 2) + [n]
    c, s = (torch.cos(ang) * mag).view(shape), (torch.sin(ang) * mag).view(shape)
    a, b = u[..., 0:2 * n:2], u[..., 1:2 * n:2]
    out = u.clone()
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


def latent_attention(h, P, pre, m, eps):
    """Queries through a normed latent; keys and values from one normed latent per position, plus one rotated key part that
    all heads share.  Every head: [dim unrotated | rot_dim rotated]; causal softmax."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_unit(h @ P[pre + "dq"].T, eps) * P[pre + "dq.norm"]
    q = (cq @ P[pre + "uq"].T).view(T, H, dn + dr)
    dkv = h @ P[pre + "dkv"].T
    c = rms_unit(dkv[:, :R], eps) * P[pre + "dkv.norm"]
    rates, mag = stretched_rates(m["rot"])
    k_rot = rotate_pairs(dkv[:, R:], rates, mag)                                  # [T, dr]
    q_rot = rotate_pairs(q[..., dn:], rates, mag)                                 # [T, H, dr]
    k = (c @ P[pre + "uk"].T).view(T, H, dn)
    v = (c @ P[pre + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        s = (q[:, head, :dn] @ k[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        s = s.masked_fill(torch.ones(T, T).triu(1).bool(), -math.inf)
        out[:, head] = torch.softmax(s, -1) @ v[:, head]
    return out.reshape(T, H * dv) @ P[pre + "o"].T


def capped_window_attention(h, P, pre, m, eps):
    """Grouped heads, a short convolution on q and k, values = convolved keys.  score = cap tanh(q . k scale / cap)
    - r1 ln(1 + r2 (i - j)); position i sees 0 <= i - j < mask.size; the heads are gated by a sigmoid of the input."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = causal_conv(h @ P[pre + "q"].T, P[pre + "q.conv"]).view(T, H, d)
    k = causal_conv(h @ P[pre + "k"].T, P[pre + "k.conv"]).view(T, G, d)
    cap, win = float(m["softcap"]), int(m["mask"]["size"])
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    dist = (i - j).to(F64)
    hidden = (j > i) | (i - j >= win)
    out = torch.zeros(T, H, d, dtype=F64)
    for head in range(H):
        kh = head // (H // G)
        s = q[:, head] @ k[:, kh].T * m["scale"]
        s = cap * torch.tanh(s / cap)
        s = s - P[pre + "r1"][head] * torch.log1p(P[pre + "r2"][head] * dist.clamp(min=0.0))
        s = s.masked_fill(hidden, -math.inf)
        out[:, head] = torch.softmax(s, -1) @ k[:, kh]
    o = out.reshape(T, H * d) * torch.sigmoid(h @ P[pre + "g"].T)
    return o @ P[pre + "o"].T


MIXERS = {"channel_delta": channel_delta, "latent_attention": latent_attention, "attention": capped_window_attention}


# ---- feed-forward -------------------------------------------------------------------------------------------------------
def clamped_expert(h, P, pre, limit):
    g = torch.clamp(h @ P[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ P[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ P[pre + "down"].T


def route(h, P, pre, r):
    """(chosen experts [T, top], their weights): the largest sigmoid scores, used as they are."""
    s = torch.sigmoid(h @ P[pre + "router"].T)
    w, ids = torch.topk(s, int(r["top"]), dim=-1)
    return ids, w


def routed_ff(h, P, pre, mlp, chosen=None):
    """sum over the chosen experts of expert(w h): the weight goes on the expert's input."""
    ids, w = route(h, P, pre, mlp["router"]) if chosen is None else chosen
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros(h.shape[0], P[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t].tolist(), w[t]):
            out[t] += clamped_expert(wt * h[t:t + 1], P, f"{pre}e{e}.", limit)[0]
    return out


# ---- the model ----------------------------------------------------------------------------------------------------------
def hyper_read(xs, P, name):
    """u = sum_s in[s] x_s; xs [S, T, W]."""
    return torch.einsum("s,stw->tw", P[name + ".in"], xs)


def hyper_write(xs, y, P, name):
    """x_t <- sum_s mix[s, t] x_s + out[t] y, every copy from the old ones."""
    return torch.einsum("sr,stw->rtw", P[name + ".mix"], xs) + P[name + ".out"].view(-1, 1, 1) * y.unsqueeze(0)


def forward(cfg, P, tokens, tap=None, chosen=None):
    """Logits [T, vocab] of one sequence.  ``tap(layer, sum of the copies)`` after every layer.  ``chosen``: per layer the
    (experts, weights) to use instead of routing (to compare past a close call)."""
    P = {k: v.to(F64) if v.is_floating_point() else v for k, v in P.items()}
    eps = float(cfg["norm"]["eps"])
    x0 = P["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    xs = x0.unsqueeze(0).repeat(int(cfg["streams"]), 1, 1)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = with_input_conv(tanh_norm(hyper_read(xs, P, p + "hc1"), P, p + "norm1"), P[p + "canon1"])
        xs = hyper_write(xs, MIXERS[L["type"]](n, P, p + "mix.", L["mixer"], eps), P, p + "hc1")
        if L.get("mlp") is not None:
            n = with_input_conv(tanh_norm(hyper_read(xs, P, p + "hc2"), P, p + "norm2"), P[p + "canon2"])
            xs = hyper_write(xs, routed_ff(n, P, p + "mlp.", L["mlp"], None if chosen is None else chosen[i]), P, p + "hc2")
        if tap is not None:
            tap(i, xs.sum(0))
    return tanh_norm(xs.sum(0), P, "final.norm") @ P["embed"].T


# ---- small configurations and random weights for the tests ------------------------------------------------------------------
def moe_mlp(experts, top, ff, limit=1.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def delta_layer(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def latent_layer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None, mlp=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                                                  "kv_rank": kv_rank, "scale": scale, "rot": rot}, "mlp": mlp}


def window_layer(heads, kv_heads, dim, scale, window, softcap, conv, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "softcap": softcap,
                                           "mask": {"size": window}, "conv": conv}, "mlp": mlp}


def make_config(layers, vocab=40, width=32, eps=1e-5, streams=2, taps=3):
    return {"architecture": "Dapupel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}, "streams": streams,
            "canon": {"taps": taps}}


def low_rank(width):
    """inner sizes of the decay's and the gate's pairs of matrices (the config does not give them: the tensors do)"""
    return max(4, width // 8), max(4, width // 8 + 3)


def shapes(cfg):
    W, V, S, taps = cfg["width"], cfg["vocab"], cfg["streams"], cfg["canon"]["taps"]
    s = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,), "final.norm.alpha": ()}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for q in ("1", "2") if L.get("mlp") is not None else ("1",):
            s.update({f"{p}norm{q}": (W,), f"{p}norm{q}.b": (W,), f"{p}norm{q}.alpha": (), f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,),
                      f"{p}hc{q}.mix": (S, S), f"{p}canon{q}": (W, taps)})
        if L["type"] == "channel_delta":
            ck, cv, n = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["conv"]
            ra, rg = low_rank(W)
            s.update({p + "mix.q": (ck, W), p + "mix.q.conv": (ck, n), p + "mix.k": (ck, W), p + "mix.k.conv": (ck, n), p + "mix.v": (cv, W),
                      p + "mix.v.conv": (cv, n), p + "mix.b": (m["heads"], W), p + "mix.A_log": (m["heads"],), p + "mix.norm": (m["vdim"],),
                      p + "mix.a1": (ra, W), p + "mix.a2": (m["heads"] * m["dim"], ra), p + "mix.dt_bias": (m["heads"] * m["dim"],),
                      p + "mix.g1": (rg, W), p + "mix.g2": (cv, rg), p + "mix.o": (W, cv)})
        elif L["type"] == "latent_attention":
            H = m["heads"]
            s.update({p + "mix.dq": (m["q_rank"], W), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                      p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], W), p + "mix.dkv.norm": (m["kv_rank"],),
                      p + "mix.uk": (H * m["dim"], m["kv_rank"]), p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.o": (W, H * m["vdim"])})
        else:
            cq, ck, n = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["conv"]
            s.update({p + "mix.q": (cq, W), p + "mix.k": (ck, W), p + "mix.q.conv": (cq, n), p + "mix.k.conv": (ck, n), p + "mix.r1": (m["heads"],),
                      p + "mix.r2": (m["heads"],), p + "mix.g": (cq, W), p + "mix.o": (W, cq)})
        mlp = L.get("mlp")
        if mlp is None:
            continue
        E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        for e in range(E):
            s.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
        s[p + "mlp.router"] = (E, W)
    return s


def random_weights(cfg, seed=0, dtype=torch.float32, gain=1.0):
    """Random tensors of every shape, scaled so that each branch moves the stream visibly (``gain`` multiplies the projection
    matrices: below one, a rounding error early in the model grows less on its way to the logits); values are rounded to
    bfloat16 (kept in ``dtype``) so that a bfloat16 model holds the same numbers."""
    g = torch.Generator().manual_seed(seed)
    S = cfg["streams"]
    P = {}
    for name, shape in shapes(cfg).items():
        parts = name.split(".")
        leaf = parts[-1]
        if leaf == "alpha":
            t = torch.rand(shape, generator=g) * 0.6 + 0.5
        elif len(parts) >= 2 and parts[-2].startswith("hc"):
            if leaf == "mix":
                t = torch.eye(S) * 0.8 + torch.randn(shape, generator=g) * 0.25
            elif leaf == "in":
                t = torch.rand(shape, generator=g) * 0.8 + 0.3
            else:
                t = torch.randn(shape, generator=g) * 0.4 + 0.8
        elif leaf.startswith("canon"):
            t = torch.randn(shape, generator=g) * 0.4
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.5
            if "q" in parts or "k" in parts:
                t[:, -1] += 1.0
        elif leaf in ("r1", "r2"):
            t = torch.rand(shape, generator=g) * 0.8 + 0.1
        elif leaf == "b" and parts[-2].startswith("norm"):
            t = torch.randn(shape, generator=g) * 0.2
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + torch.randn(shape, generator=g) * 0.3
        elif leaf == "norm":
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif leaf == "A_log":
            t = torch.rand(shape, generator=g) * 1.5 - 1.0
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) * 0.7 - 0.5
        elif name == "embed":
            t = torch.randn(shape, generator=g) * 0.8
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * (1.5 * gain / math.sqrt(shape[1]))
            if leaf == "router":
                t = t * 2.0
        else:
            raise KeyError(name)
        P[name] = t.to(torch.bfloat16).to(dtype)
    return P


def logits_error(got, want):
    """Worst position: rms over the vocabulary of the centred difference, relative to the rms of the centred expected row."""
    got, want = got.to(F64).cpu(), want.to(F64).cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())

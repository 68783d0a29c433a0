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

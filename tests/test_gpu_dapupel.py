"""Dapupel on the GPU against the slow float64 oracle (tests/dapupel_oracle.py): each mechanism alone, prompts against
token-by-token decoding, portions, ragged batches, rows given back and used again, far keys and window edges in prompts and in
decoding, the rotation, the stream copies and the input convolution, other sizes, greedy generation through generate_step."""
import math

import numpy as np
import pytest
import torch

import dapupel_oracle as O

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4        # float32 model against the float64 oracle (centred rms over the vocabulary, relative)
BF16_TOL = 6e-2       # bfloat16 matrix products


def build(cfg, seed=0, dtype=torch.float32, weights=None, gain=1.0):
    from mlx_parallm_b200.utils import _get_classes
    Model, Args = _get_classes(cfg)
    w = O.random_weights(cfg, seed, gain=gain) if weights is None else weights
    return Model(Args.from_dict(cfg)).load_weights(w, device="cuda", dtype=dtype), w


def toks(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def residuals(cfg, w, t):
    res = []
    logits = O.forward(cfg, w, t, tap=lambda run, x: res.append(x.clone()))
    return logits, res


CONFIGS = {
    # every branch: the three mixers, with and without a feed-forward, several experts per token, grouped key heads
    "mixed": lambda: O.make_config([
        O.delta_layer(4, 2, 8, 12, 4, mlp=O.moe_mlp(6, 2, 24, limit=0.8)),
        O.latent_layer(4, 8, 4, 12, 12, 16, 0.3, base=100.0, scaling=(4.0, 24, 6.0, 0.5), mlp=O.moe_mlp(8, 3, 16)),
        O.window_layer(6, 2, 8, 0.35, 11, 3.0, 3, mlp=O.moe_mlp(5, 1, 20, limit=2.5)),
        O.latent_layer(2, 16, 8, 8, 8, 24, 0.2),
        O.window_layer(2, 2, 16, 0.25, 7, 30.0, 2),
    ], streams=3, taps=3),
    # sizes off the fast paths (odd width, heads, vector sizes), one key head for three heads, four copies of the stream, two
    # taps, every expert chosen, a window of one position, a rotated part of two dimensions
    "odd": lambda: O.make_config([
        O.window_layer(3, 1, 6, 0.4, 1, 1.5, 4, mlp=O.moe_mlp(4, 4, 13, limit=0.5)),
        O.latent_layer(3, 5, 2, 7, 9, 11, 0.45, base=7.0, scaling=(2.0, 8, 4.0, 1.0), mlp=O.moe_mlp(7, 2, 9)),
        O.delta_layer(3, 1, 6, 11, 2, mlp=O.moe_mlp(3, 1, 11)),
    ], vocab=31, width=27, eps=1e-3, streams=4, taps=2),
    # wider heads: sizes of the tile kernels, a latent row that fills its 32-value padding exactly and one that does not, a
    # window longer than any test prompt, as many key heads as heads
    "wide": lambda: O.make_config([
        O.latent_layer(8, 32, 32, 32, 48, 96, 0.12, base=1e5, scaling=(8.0, 64, 16.0, 1.0), mlp=O.moe_mlp(3, 1, 24)),
        O.window_layer(2, 2, 64, 0.12, 4096, 50.0, 3),
        O.delta_layer(2, 2, 128, 64, 3),
        O.latent_layer(8, 16, 8, 16, 24, 40, 0.2, mlp=O.moe_mlp(4, 2, 16)),
    ], vocab=130, width=64, streams=2, taps=4),
    # one copy of the stream, no convolutions anywhere (one tap), one head, one expert
    "plain": lambda: O.make_config([
        O.delta_layer(1, 1, 8, 8, 1, mlp=O.moe_mlp(1, 1, 24)),
        O.window_layer(1, 1, 8, 0.35, 16, 20.0, 1, mlp=O.moe_mlp(2, 1, 24)),
        O.latent_layer(1, 8, 8, 8, 8, 8, 0.3),
    ], vocab=50, width=32, streams=1, taps=1),
}


@pytest.fixture(scope="module")
def models():
    out = {}
    for name, mk in CONFIGS.items():
        cfg = mk()
        m, w = build(cfg, seed=len(name))
        out[name] = (cfg, m, w)
    return out


I32 = dict(dtype=torch.int32, device="cuda")


# ---- the copies of the stream, the tanh norm, the input convolution ---------------------------------------------------------
@pytest.mark.parametrize("S,W,taps", [(1, 32, 1), (2, 48, 3), (3, 27, 2), (5, 1024, 4), (8, 64, 16)])
def test_stream_step_prompt_and_decode(S, W, taps):
    """One launch writes a sublayer's output into the copies, reads them for the next sublayer and norms; the convolution over
    three portions (7, 2 and 1 tokens, the last through the fused decode path) of two rows equals the whole sequence's."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(S * 100 + W)
    T = 10
    xs0 = torch.randn(2, T, S, W, generator=g)
    y = torch.randn(2, T, W, generator=g)
    mix, out, read = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    alpha, w, b = torch.tensor([0.7]), torch.randn(W, generator=g), torch.randn(W, generator=g)
    cw = torch.randn(W, taps, generator=g) * 0.5
    new = torch.einsum("sr,btsw->btrw", mix.double(), xs0.double()) + out.double().view(1, 1, S, 1) * y.double().unsqueeze(2)
    n = torch.tanh(0.7 * torch.einsum("r,btrw->btw", read.double(), new)) * w.double() + b.double()
    want_x = torch.stack([O.with_input_conv(n[r], cw.double()) for r in range(2)])
    dev = lambda t: t.cuda().contiguous()
    state = torch.full((3, max(taps - 1, 1), W), 7.0, device="cuda")          # stale values: position 0 must not read them
    got_x = torch.zeros(2, T, W)
    got_new = torch.zeros(2, T, S, W)
    got_sum = torch.zeros(2, T, W)
    lo = 0
    for cnt in (7, 2, 1):
        M = 2 * cnt
        xs = dev(xs0[:, lo:lo + cnt].reshape(M, S * W))
        yy = dev(y[:, lo:lo + cnt].reshape(M, W))
        t_row = torch.tensor([2] * cnt + [0] * cnt, **I32)
        t_pos = torch.tensor(list(range(lo, lo + cnt)) * 2, **I32)
        t_off = torch.tensor(list(range(cnt)) * 2, **I32)
        x_out = torch.zeros(M, W, device="cuda")
        sums = torch.zeros(M, W, device="cuda")
        kw = dict(y=yy, mix=dev(mix), out=dev(out), read=dev(read), alpha=dev(alpha), w=dev(w), b=dev(b), sum_out=sums)
        if cnt == 1:
            ops.hyper_step(xs, S, conv_w=dev(cw.t()), conv_state=state, t_row=t_row, t_pos=t_pos, taps=taps, x_out=x_out, **kw)
        else:
            nn = torch.zeros(M, W, device="cuda")
            ops.hyper_step(xs, S, n_out=nn, **kw)
            ops.canon_conv(nn, dev(cw.t()), state, t_row, t_pos, t_off, x_out, taps)
            if taps > 1:
                ops.delta_conv_commit(nn, state, torch.tensor([0, cnt, 2 * cnt], **I32), torch.tensor([2, 0], **I32), 2, W, taps)
        got_x[:, lo:lo + cnt] = x_out.cpu().view(2, cnt, W)
        got_new[:, lo:lo + cnt] = xs.cpu().view(2, cnt, S, W)
        got_sum[:, lo:lo + cnt] = sums.cpu().view(2, cnt, W)
        lo += cnt
    assert (got_new.double() - new).abs().max() < 1e-5 * max(1.0, float(new.abs().max()))
    assert (got_sum.double() - new.sum(2)).abs().max() < 1e-5 * max(1.0, float(new.abs().max()) * S)
    assert (got_x.double() - want_x).abs().max() < 2e-5 * max(1.0, float(want_x.abs().max()))


def test_stream_start_and_final_norm():
    """Every copy starts as the embedding; the last norm is the same tanh norm on given rows."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(5)
    S, W, M = 3, 40, 6
    e = torch.randn(M, W, generator=g)
    read, alpha, w, b = torch.randn(S, generator=g), torch.tensor([1.3]), torch.randn(W, generator=g), torch.randn(W, generator=g)
    xs = torch.full((M, S * W), 9.0, device="cuda")
    n = torch.zeros(M, W, device="cuda")
    ops.hyper_step(xs, S, src=e.cuda(), read=read.cuda(), alpha=alpha.cuda(), w=w.cuda(), b=b.cuda(), n_out=n)
    assert torch.equal(xs.cpu().view(M, S, W), e.unsqueeze(1).expand(M, S, W))
    want = torch.tanh(1.3 * read.double().sum() * e.double()) * w.double() + b.double()
    assert (n.cpu().double() - want).abs().max() < 1e-5
    for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        x = torch.zeros(M, W, dtype=dt, device="cuda")
        ops.tanh_norm(e.cuda(), alpha.cuda(), w.cuda(), b.cuda(), x)
        ref = torch.tanh(1.3 * e.double()) * w.double() + b.double()
        assert (x.cpu().double() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))


# ---- routing ------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top,M,W", [(6, 2, 9, 16), (12, 1, 40, 24), (5, 5, 3, 8), (40, 7, 33, 64), (1, 1, 4, 8)])
def test_routing_by_scores_and_weights_on_the_input(E, top, M, W):
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    logits = torch.randn(M, E, generator=g) * 2.0
    x = torch.randn(M, W, generator=g)
    ids = torch.zeros(M, top, **I32)
    wts = torch.zeros(M, top, device="cuda")
    seg, slot_of, token_of = torch.zeros(E + 1, **I32), torch.zeros(M, top, **I32), torch.zeros(M, top, **I32)
    ops.moe_route_scores(logits.cuda(), ids, wts, seg, slot_of, token_of, top)
    s = torch.sigmoid(logits.double())
    want_w, want_ids = torch.topk(s, top, dim=-1)
    assert ids.cpu().tolist() == want_ids.tolist()
    assert (wts.cpu().double() - want_w).abs().max() < 1e-6
    counts = torch.bincount(want_ids.flatten(), minlength=E)
    assert seg.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()
    for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        xs = torch.zeros(M * top, W, dtype=dt, device="cuda")
        ops.moe_scatter_scaled(x.to(dt).cuda(), slot_of, wts, xs, top)
        so, sg = slot_of.cpu(), seg.cpu()
        for t in range(M):
            for k in range(top):
                slot = int(so[t, k])
                e = int(want_ids[t, k])
                assert sg[e] <= slot < sg[e + 1]
                ref = want_w[t, k] * x[t].to(dt).double()
                assert (xs[slot].cpu().double() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))


# ---- mixers alone -----------------------------------------------------------------------------------------------------------
def one_layer(layer, **kw):
    return O.make_config([layer], **kw)


def mixer_alone(cfg, w, T, seed, dtype=torch.float32, cuts=None):
    """Residual stream after the single layer of cfg for T random tokens: framework (optionally fed in portions), oracle."""
    m, _ = build(cfg, dtype=dtype, weights=w)
    t = toks(cfg, T, seed)
    _, res = residuals(cfg, w, t)
    got = []
    m.residual_tap = lambda layer, kind, h: got.append(h.clone())
    cache = m.make_cache(1)
    lo = 0
    for n in (cuts or [T]):
        m.forward_ragged([t[lo:lo + n]], cache)
        lo += n
    m.residual_tap = None
    return torch.cat(got).double().cpu(), res[0]


@pytest.mark.parametrize("H,G,dk,dv,conv", [(4, 2, 8, 12, 4), (3, 1, 6, 11, 2), (2, 2, 128, 64, 3), (1, 1, 40, 160, 1)])
def test_channel_delta_alone(H, G, dk, dv, conv):
    cfg = one_layer(O.delta_layer(H, G, dk, dv, conv), width=32)
    w = O.random_weights(cfg, H + dk)
    for cuts in (None, [9, 1, 1, 2, 17]):
        got, want = mixer_alone(cfg, w, 30, 1, cuts=cuts)
        assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("H,dn,dr,dv,qr,kr,scaling", [(4, 8, 4, 12, 12, 16, None), (3, 5, 2, 7, 9, 11, (2.0, 8, 4.0, 1.0)),
                                                      (8, 32, 32, 32, 48, 96, (8.0, 64, 16.0, 1.0)), (2, 64, 16, 64, 16, 48, (40.0, 32, 32.0, 1.0)),
                                                      (1, 8, 8, 8, 8, 8, None), (9, 8, 6, 8, 8, 600, None)])
def test_latent_attention_alone(H, dn, dr, dv, qr, kr, scaling):
    cfg = one_layer(O.latent_layer(H, dn, dr, dv, qr, kr, 0.3 / math.sqrt(dn + dr) * 4, base=50.0, scaling=scaling), width=32)
    w = O.random_weights(cfg, H + kr)
    for cuts in (None, [9, 1, 1, 2, 27]):
        got, want = mixer_alone(cfg, w, 40, 2, cuts=cuts)
        assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    got, want = mixer_alone(cfg, w, 40, 2, dtype=torch.bfloat16)
    assert (got - want).abs().max() < 6e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("H,G,d,win,cap,conv", [(4, 2, 8, 5, 3.0, 3), (3, 1, 6, 1, 1.5, 4), (2, 2, 64, 4096, 50.0, 3), (6, 3, 48, 9, 10.0, 2),
                                                (1, 1, 128, 20, 5.0, 1), (2, 1, 10, 40, 2.0, 5)])
def test_window_attention_alone(H, G, d, win, cap, conv):
    cfg = one_layer(O.window_layer(H, G, d, 1.0 / math.sqrt(d), win, cap, conv), width=32)
    w = O.random_weights(cfg, H + d)
    for cuts in (None, [9, 1, 1, 2, 27]):
        got, want = mixer_alone(cfg, w, 40, 3, cuts=cuts)
        assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    got, want = mixer_alone(cfg, w, 40, 3, dtype=torch.bfloat16)
    assert (got - want).abs().max() < 6e-2 * max(1.0, float(want.abs().max()))


def test_rotation_kernels():
    """Both rotation kernels against the oracle's rotation at positions up to 5000: interleaved pairs, stretched rates, the
    magnitude on cos and sin; the latent part normed, the padding zero."""
    from mlx_parallm_b200 import ops
    from mlx_parallm_b200.models.dapupel import stretched_rates
    g = torch.Generator().manual_seed(3)
    H, dn, dr, R, qr, M = 3, 6, 8, 10, 5, 7
    rot = {"dims": dr, "base": 300.0, "scaling": {"factor": 6.0, "original": 40, "fast": 8.0, "slow": 0.5}}
    rates, mag = stretched_rates(dr, 300.0, rot["scaling"])
    want_rates, want_mag = O.stretched_rates(rot)
    assert rates == pytest.approx(want_rates, rel=1e-12) and mag == pytest.approx(want_mag)
    assert any(abs(a - b) > 1e-6 for a, b in zip(rates, [300.0 ** (-2.0 * i / dr) for i in range(dr // 2)]))
    pos = [0, 1, 2, 17, 600, 4999, 5000]
    proj = torch.randn(M, qr + R + dr, generator=g)
    wq, wkv = torch.rand(qr, generator=g) + 0.5, torch.rand(R, generator=g) + 0.5
    row = 32
    cache = torch.full((2, 5001, row), 5.0, device="cuda")
    cq = torch.zeros(M, qr, device="cuda")
    rd = torch.tensor(rates, dtype=torch.float32, device="cuda")
    ops.latent_rope_prep(proj.cuda(), qr, R, dr, wq.cuda(), wkv.cuda(), 1e-3, rd, mag, cq, cache, torch.ones(M, **I32), torch.tensor(pos, **I32))
    full = torch.zeros(5001, dr, dtype=torch.float64)
    full[pos] = proj[:, qr + R:].double()
    want_rot = O.rotate_pairs(full, want_rates, want_mag)[pos]
    got = cache[1, pos].cpu().double()
    assert (got[:, R:R + dr] - want_rot).abs().max() < 5e-4           # the angle is a float32 product: 5000 * rate
    assert (got[:, :R] - O.rms_unit(proj[:, qr:qr + R].double(), 1e-3) * wkv.double()).abs().max() < 1e-5
    assert float(got[:, R + dr:].abs().max()) == 0.0 and float(cache[0].min()) == 5.0
    assert (cq.cpu().double() - O.rms_unit(proj[:, :qr].double(), 1e-3) * wq.double()).abs().max() < 1e-5
    q = torch.randn(M, H, dn + dr, generator=g)
    qlat = torch.full((M, H * row), 3.0, device="cuda")
    ops.latent_q_rope(q.reshape(M, -1).cuda(), H, dn, dr, R, rd, mag, torch.tensor(pos, **I32), qlat)
    fullq = torch.zeros(5001, H, dr, dtype=torch.float64)
    fullq[pos] = q[..., dn:].double()
    want_q = O.rotate_pairs(fullq, want_rates, want_mag)[pos]
    gq = qlat.cpu().double().view(M, H, row)
    assert (gq[..., R:R + dr] - want_q).abs().max() < 5e-4
    assert float((gq[..., :R] - 3.0).abs().max()) == 0.0 and float(gq[..., R + dr:].abs().max()) == 0.0


# ---- the windowed attention kernels: far keys, window edges, tile borders ------------------------------------------------------
def window_case(T, H, G, d, win, hot=None, dtype=torch.float32, seed=0, boost=30.0, decode=False, cap=200.0, gate=True, penalty=True):
    """window_attn over T cached positions of one row; every token is a query at its own position (``decode``: one launch per
    token).  A hot pair (query position, key position) gets a score far above the rest so that a key that is wrongly masked,
    skipped or misplaced shows.  Returns (got, want, the weight every head gives the hot key)."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(seed + T)
    q = torch.randn(T, H, d, generator=g) * 0.3
    k = torch.randn(T, G, d, generator=g) * 0.3
    if hot is not None:
        u = torch.randn(d, generator=g)
        u = u / u.norm()
        q[hot[0]] += boost * u
        k[hot[1]] += 3.0 * u
    if dtype != torch.float32:
        q = q.to(dtype).float()            # the 16-bit kernels round the query to the cache's type: give both sides that query
    r1, r2 = torch.rand(H, generator=g) * 0.8 + 0.1, torch.rand(H, generator=g) * 0.8 + 0.1
    gz = torch.randn(T, H * d + 5, generator=g)
    kc = torch.zeros(2, G, T + 3, d)
    kc[1, :, :T] = k.transpose(0, 1)
    kc = kc.to(dtype)
    out = torch.zeros(T, H * d + 8, dtype=dtype, device="cuda")
    qd, kcd, gd = q.reshape(T, -1).contiguous().cuda(), kc.cuda(), gz.cuda()
    ws = torch.empty(max(ops.sink_attn_workspace_floats(1, H, d), 4), device="cuda")
    opt = dict(softcap=cap, r1=r1.cuda() if penalty else None, r2=r2.cuda() if penalty else None, window=win, workspace=ws)
    if decode:
        for t in range(T):
            ops.window_attn(qd[t:t + 1], kcd, kcd, torch.ones(1, **I32), torch.tensor([t], **I32), out[t:t + 1, :H * d], H, G, d, d,
                            gate=gd[t:t + 1, :H * d] if gate else None, cu=torch.tensor([0, 1], **I32), rows=torch.tensor([1], **I32), nb=1,
                            max_n=1, **opt)
    else:
        ops.window_attn(qd, kcd, kcd, torch.ones(T, **I32), torch.arange(T, **I32), out[:, :H * d], H, G, d, d,
                        gate=gd[:, :H * d] if gate else None, cu=torch.tensor([0, T], **I32), rows=torch.tensor([1], **I32), nb=1, max_n=T, **opt)
    kd = kc[1, :, :T].double()
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    hidden = (j > i) | ((i - j >= win) if win > 0 else torch.zeros(T, T, dtype=torch.bool))
    dist = (i - j).clamp(min=0).double()
    want = torch.zeros(T, H, d, dtype=torch.float64)
    seen = torch.zeros(T, H, dtype=torch.float64)
    for h in range(H):
        kv = h // (H // G)
        s = q[:, h].double() @ kd[kv].T
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        if penalty:
            s = s - r1[h].double() * torch.log1p(r2[h].double() * dist)
        p = torch.softmax(s.masked_fill(hidden, -math.inf), -1)
        if hot is not None:
            seen[:, h] = p[:, hot[1]]
        want[:, h] = p @ kd[kv]
    if gate:
        want = want * torch.sigmoid(gz[:, :H * d].double()).view(T, H, d)
    assert float(out[:, H * d:].float().abs().max()) == 0.0          # columns beside the heads are not touched
    return out[:, :H * d].double().cpu().view(T, H, d), want, seen


# (tokens, window, hot query, hot key, whether the query sees the key)
EDGES = [(600, 0, 599, 3, True), (600, 590, 599, 10, True), (600, 590, 599, 9, False), (70, 32, 63, 32, True), (70, 32, 64, 32, False),
         (70, 32, 64, 33, True), (130, 64, 127, 64, True), (130, 64, 128, 64, False), (130, 65, 128, 64, True), (97, 96, 95, 0, True),
         (97, 96, 96, 0, False), (40, 1, 7, 6, False), (40, 1, 7, 7, True), (1, 4, None, None, None), (2, 2, 1, 0, True), (3, 2, 2, 0, False),
         (200, 40, 199, 160, True), (200, 40, 199, 159, False)]


@pytest.mark.parametrize("T,win,hq,hk,visible", EDGES)
@pytest.mark.parametrize("decode", [False, True])
def test_window_attention_far_keys_and_window_edges(T, win, hq, hk, visible, decode):
    if decode and T > 200:
        T, win, hq, hk = T - 400, max(win - 400, 0), hq - 400, hq - 400 - (hq - hk - 400)      # the same edge 400 nearer: fewer launches
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        got, want, seen = window_case(T, 4, 2, 24, win, None if hq is None else (hq, hk), dtype=dtype, decode=decode)
        assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max()))
        if hq is not None:
            assert (float(seen[hq].min()) > 0.9) if visible else (float(seen[hq].max()) == 0.0)


@pytest.mark.parametrize("T,win,hq,hk", [(600, 0, 599, 3), (300, 256, 299, 44), (300, 256, 299, 43), (70, 64, 63, 0), (70, 64, 64, 1), (70, 64, 64, 0),
                                         (130, 0, 128, 63), (130, 0, 129, 64), (129, 128, 128, 1), (65, 0, 64, 0), (64, 0, 63, 0), (5, 0, 4, 1),
                                         (200, 33, 198, 166), (300, 40, 290, 251), (300, 100, 299, 200), (260, 10, 259, 250)])
def test_window_attention_tile_sizes_far_keys_and_tile_borders(T, win, hq, hk):
    """Sizes the tensor-core kernel takes (16-bit, vector sizes 64 and 128): hot pairs across its key tiles and its query tiles,
    windows that begin inside a tile and tiles that lie before a row's window, prompts and single tokens, with and without cap,
    penalty and gate."""
    for d in (64, 128):
        for decode in (False, True):
            if decode and T > 200:
                continue
            for plain in (False, True):
                got, want, seen = window_case(T, 4, 2, d, win, (hq, hk), dtype=torch.bfloat16, seed=d, decode=decode, cap=0.0 if plain else 40.0,
                                              gate=not plain, penalty=not plain, boost=20.0)
                assert (got - want).abs().max() < 3e-2 * max(1.0, float(want.abs().max())), (d, decode, plain)
                visible = hk <= hq and (win == 0 or hq - hk < win)
                assert (float(seen[hq].min()) > 0.5) if visible else (float(seen[hq].max()) == 0.0)


@pytest.mark.parametrize("H,G,d,nb", [(8, 2, 64, 5), (16, 1, 64, 3), (4, 4, 128, 40), (6, 3, 128, 150), (3, 1, 10, 9)])
def test_window_attention_decode_batches(H, G, d, nb):
    """Decode steps of many rows of unequal length in one launch (rows out of order, windows that cover all or part of a row)."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(H + nb)
    win = 70
    lens = [int(x) for x in torch.randint(1, 200, (nb,), generator=g)]
    rows = torch.randperm(nb + 2, generator=g)[:nb].tolist()
    Tcap = 256
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        kc = torch.zeros(nb + 2, G, Tcap, d)
        q = (torch.randn(nb, H, d, generator=g) * 0.3).to(dtype).float()
        for r, n in zip(rows, lens):
            kc[r, :, :n] = torch.randn(G, n, d, generator=g) * 0.6
        kc = kc.to(dtype)
        r1, r2 = torch.rand(H, generator=g), torch.rand(H, generator=g)
        out = torch.zeros(nb, H * d, dtype=dtype, device="cuda")
        ws = torch.empty(max(ops.sink_attn_workspace_floats(nb, H, d), 4), device="cuda")
        kcd = kc.cuda()
        ops.window_attn(q.reshape(nb, -1).cuda(), kcd, kcd, torch.tensor(rows, **I32), torch.tensor([n - 1 for n in lens], **I32), out, H, G, d, d,
                        softcap=8.0, r1=r1.cuda(), r2=r2.cuda(), window=win, cu=torch.arange(nb + 1, **I32), rows=torch.tensor(rows, **I32), nb=nb,
                        max_n=1, workspace=ws)
        for e, (r, n) in enumerate(zip(rows, lens)):
            lo = max(0, n - win)
            for h in range(H):
                kk = kc[r, h // (H // G), lo:n].double()
                s = 8.0 * torch.tanh(q[e, h].double() @ kk.T / 8.0)
                s = s - r1[h].double() * torch.log1p(r2[h].double() * torch.arange(n - 1 - lo, -1, -1).double())
                ref = torch.softmax(s, -1) @ kk
                assert (out[e, h * d:(h + 1) * d].double().cpu() - ref).abs().max() < tol * max(1.0, float(ref.abs().max())), (e, h)


# ---- whole models -----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prompt_logits_and_residuals_match_the_oracle(models, name):
    cfg, m, w = models[name]
    t = toks(cfg, 45, 1)
    want, res = residuals(cfg, w, t)
    got_res = []
    m.residual_tap = lambda layer, kind, h: got_res.append((layer, h.clone()))
    try:
        got = m.forward_ragged([t], m.make_cache(1), want=[list(range(len(t)))])
    finally:
        m.residual_tap = None
    assert [i for i, _ in got_res] == list(range(len(cfg["layers"])))
    for k, r in enumerate(res):
        assert (got_res[k][1].double().cpu() - r).abs().max() < 2e-4 * max(1.0, float(r.abs().max())), f"residual after layer {k}"
    assert O.logits_error(got, want) < F32_TOL


@pytest.mark.parametrize("name", list(CONFIGS))
def test_bfloat16_model(name):
    cfg = CONFIGS[name]()
    m, w = build(cfg, seed=3, dtype=torch.bfloat16, gain=0.5)       # rounding flips an expert now and then: keep its cost small
    t = toks(cfg, 60, 2)
    got = m.forward_ragged([t], m.make_cache(1), want=[list(range(len(t)))])
    want = O.forward(cfg, w, t)
    per_pos = sorted(O.logits_error(got[i:i + 1], want[i:i + 1]) for i in range(len(t)))
    assert per_pos[len(t) // 2] < BF16_TOL and per_pos[-1] < 1.0, per_pos[-3:]


def test_bfloat16_model_on_the_tensor_core_paths():
    """Vector sizes the tile attention kernels take, groups of experts large enough for the tcgen05 grouped product: a prompt,
    a ragged batch and decode steps through the captured step in bfloat16 against the oracle; positions compared by their
    typical error, as above."""
    from mlx_parallm_b200 import utils
    cfg = O.make_config([
        O.window_layer(4, 2, 64, 0.125, 100, 30.0, 3, mlp=O.moe_mlp(4, 2, 64)),
        O.latent_layer(8, 32, 32, 32, 64, 96, 0.125, scaling=(8.0, 128, 16.0, 1.0), mlp=O.moe_mlp(2, 1, 128)),
        O.delta_layer(4, 2, 64, 32, 4),
        O.window_layer(8, 8, 128, 0.09, 4096, 50.0, 2),
    ], vocab=200, width=128, streams=2, taps=3)
    m, w = build(cfg, seed=7, dtype=torch.bfloat16)
    t = toks(cfg, 330, 3)
    want = O.forward(cfg, w, t)
    got = m.forward_ragged([t[:300]], m.make_cache(1), want=[list(range(300))])
    per_pos = sorted(O.logits_error(got[i:i + 1], want[i:i + 1]) for i in range(300))
    assert per_pos[150] < BF16_TOL and per_pos[-1] < 1.0, per_pos[-3:]
    lens = [300, 70, 5]
    cache = utils._kv_pool.get_for(m, 3)
    first = m.forward_ragged([t[:n] for n in lens], cache, rows=[2, 0, 1])
    errs = [O.logits_error(first[i:i + 1], want[n - 1:n]) for i, n in enumerate(lens)]
    st = utils._decode_step_for(m, cache, 3, False)
    st.set_rows([2, 0, 1])
    for k in range(30):
        st.tok.copy_(torch.tensor([t[n + k] for n in lens], dtype=torch.int32))
        st.run()
        errs += [O.logits_error(st.logits[i:i + 1], want[n + k:n + k + 1]) for i, n in enumerate(lens)]
    errs.sort()
    assert errs[len(errs) // 2] < BF16_TOL and errs[-1] < 1.0, errs[-3:]


def test_experts_chosen_like_the_oracle(models):
    """The last routed layer's choices and weights, read back from the step's scratch, are the oracle's for every token."""
    cfg, m, w = models["mixed"]
    t = toks(cfg, 20, 9)
    P = {k: v.double() for k, v in w.items()}
    seen = {}
    real_route = O.route

    def spy(h, P_, pre, r):
        seen[pre] = real_route(h, P_, pre, r)
        return seen[pre]

    O.route = spy
    try:
        O.forward(cfg, w, t)
    finally:
        O.route = real_route
    m.forward_ragged([t], m.make_cache(1))
    ids, wts = seen["l2.mlp."]
    a = next(iter(m._arenas.values()))
    assert a["s"].get("moe_ids", torch.int32, len(t), 1).cpu().tolist() == ids.tolist()
    assert (a["s"].get("moe_wts", torch.float32, len(t), 1).cpu().double() - wts).abs().max() < 1e-5
    assert P["l2.mlp.router"].shape[0] == 5


def test_weight_on_the_input_is_not_weight_on_the_output():
    """The clamp makes the two differ: a model whose experts saturate must follow the oracle, which scales what the expert reads."""
    cfg = O.make_config([O.delta_layer(2, 2, 8, 8, 2, mlp=O.moe_mlp(4, 2, 16, limit=0.3))], width=16)
    w = O.random_weights(cfg, 4)
    for e in range(4):
        w[f"l0.mlp.e{e}.gate"] *= 6.0
    m, _ = build(cfg, weights=w)
    t = toks(cfg, 12, 1)
    assert O.logits_error(m.forward_ragged([t], m.make_cache(1), want=[list(range(12))]), O.forward(cfg, w, t)) < F32_TOL


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_single_tokens_equal_one_pass(models, name):
    """A prompt cut into portions of 1, 2, 3, ... tokens, and fed token by token, gives the logits of one pass; the portions
    cross the convolutions' reach and the attention's windows."""
    cfg, m, w = models[name]
    t = toks(cfg, 50, 4)
    want = O.forward(cfg, w, t)
    for cuts in ([50], [1, 2, 3, 5, 8, 13, 18], [2] * 25, [1] * 50, [47, 1, 2], [49, 1], [33, 17], [3, 1, 1, 45]):
        cache = m.make_cache(3)
        got, lo = [], 0
        for n in cuts:
            got.append(m.forward_ragged([t[lo:lo + n]], cache, rows=[2], want=[list(range(n))]))
            lo += n
        assert O.logits_error(torch.cat(got), want) < F32_TOL, cuts


@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_decode_step_graph_against_prompt(models, name):
    """Most of a prompt in one pass, the rest through the engine's captured decode step (the generation path)."""
    from mlx_parallm_b200 import utils
    cfg, m, w = models[name]
    t = toks(cfg, 100, 5)
    want = O.forward(cfg, w, t)
    cache = utils._kv_pool.get_for(m, 1)
    got = [m.forward_ragged([t[:30]], cache, want=[[29]])]
    st = utils._decode_step_for(m, cache, 1, False)
    for tok in t[30:]:
        st.tok.copy_(torch.tensor([tok], dtype=torch.int32))
        st.run()
        got.append(st.logits.clone())
    assert O.logits_error(torch.cat(got), want[29:]) < F32_TOL
    assert cache[-1].offsets == [100]
    # a second group of the same batch size, stepped in turns with the first one whose row list differs
    big = utils._kv_pool.get_for(m, 3)
    m.forward_ragged([t[:30]], big, rows=[2])
    st2 = utils._decode_step_for(m, big, 1, False)
    st2.set_rows([2])
    cache1 = m.make_cache(1)
    m.forward_ragged([t[:30]], cache1)
    st1 = utils._decode_step_for(m, cache1, 1, False)
    for k, tok in enumerate(t[30:36]):
        for s_ in (st2, st1):
            s_.tok.copy_(torch.tensor([tok], dtype=torch.int32))
            s_.run()
            assert torch.equal(s_.logits, got[1 + k]), (k, s_ is st1)


def test_ragged_batch_equals_each_alone_and_rows_end_early(models):
    """Four prompts of 1, 2, 17 and 40 tokens in one pass, then decoded together while the short ones end: equal to each
    request alone in a cache of its own, and right against the oracle."""
    from mlx_parallm_b200 import utils
    cfg, m, w = models["mixed"]
    lens, extra = [1, 2, 17, 40], [0, 3, 12, 12]
    seqs = [toks(cfg, n + e, 10 + n) for n, e in zip(lens, extra)]
    cache = utils._kv_pool.get_for(m, 4)
    rows = [2, 0, 3, 1]
    first = m.forward_ragged([s[:n] for s, n in zip(seqs, lens)], cache, rows=rows, want=[list(range(n)) for n in lens])
    together = {i: [] for i in range(4)}
    o = 0
    for i, n in enumerate(lens):
        together[i].append(first[o:o + n])
        o += n
    m.release_rows(cache, [rows[0]])
    for k in range(12):
        live = [i for i in range(1, 4) if k < extra[i]]
        st = utils._decode_step_for(m, cache, len(live), False)
        st.set_rows([rows[i] for i in live])
        st.tok.copy_(torch.tensor([seqs[i][lens[i] + k] for i in live], dtype=torch.int32))
        st.run()
        for j, i in enumerate(live):
            together[i].append(st.logits[j:j + 1].clone())
        if k + 1 == extra[1]:
            m.release_rows(cache, [rows[1]])
    for i in range(4):
        got = torch.cat(together[i])
        assert O.logits_error(got, O.forward(cfg, w, seqs[i])) < F32_TOL
        alone_cache = m.make_cache(1)
        alone = [m.forward_ragged([seqs[i][:lens[i]]], alone_cache, want=[list(range(lens[i]))])]
        for tok in seqs[i][lens[i]:]:
            alone.append(m.forward_ragged([[tok]], alone_cache))
        assert torch.equal(torch.cat(alone), got), f"request {i} depends on its batch"


def test_rows_given_back_start_from_nothing(models):
    """A row that held a long sequence is released and takes a new one, alone and beside a row that goes on: the new sequence
    sees no state, no convolution inputs (of the mixers or of the sublayers' inputs) and no keys of the old one."""
    for name in ("mixed", "wide"):
        cfg, m, w = models[name]
        cache = m.make_cache(2)
        old, keep, new = toks(cfg, 60, 20), toks(cfg, 30, 21), toks(cfg, 25, 22)
        m.forward_ragged([old, keep[:20]], cache)
        m.release_rows(cache, [0])
        assert cache[0].offsets == [0, 20]
        got = m.forward_ragged([new[:3], keep[20:]], cache, want=[[0, 1, 2], list(range(10))])
        assert O.logits_error(got[:3], O.forward(cfg, w, new)[:3]) < F32_TOL
        assert O.logits_error(got[3:], O.forward(cfg, w, keep)[20:]) < F32_TOL
        rest = m.forward_ragged([new[3:]], cache, rows=[0], want=[list(range(22))])
        assert O.logits_error(rest, O.forward(cfg, w, new)[3:]) < F32_TOL
        # and through the decode step: a released row starts a sequence with single tokens
        m.release_rows(cache, [0])
        one = torch.cat([m.forward_ragged([[tok]], cache, rows=[0]) for tok in new[:6]])
        assert O.logits_error(one, O.forward(cfg, w, new[:6])) < F32_TOL


def test_first_tokens_and_short_sequences(models):
    for name in ("mixed", "odd", "plain"):
        cfg, m, w = models[name]
        seqs = [toks(cfg, n, 30 + n) for n in (1, 1, 2, 3, 4)]
        got = m.forward_ragged(seqs, m.make_cache(5), want=[list(range(len(s))) for s in seqs])
        want = torch.cat([O.forward(cfg, w, s) for s in seqs])
        assert O.logits_error(got, want) < F32_TOL


def test_far_keys_in_the_latent_attention_and_a_window_edge_in_the_model():
    """Inside whole models: a latent attention with a sharp softmax over 520 positions, whose last answers change clearly when
    the first half of the sequence is withheld, fed in three portions and then token by token; and a windowed layer whose answer
    changes when a token just inside the window changes and does not when one just outside does, in a prompt cut at the edge
    and in decoding."""
    cfg = O.make_config([O.latent_layer(2, 16, 8, 16, 16, 32, 1.5, base=1e4, scaling=(4.0, 64, 8.0, 1.0))], vocab=40, width=32, streams=2, taps=2)
    w = O.random_weights(cfg, 12)
    m, _ = build(cfg, weights=w)
    t = toks(cfg, 520, 3)
    a = O.forward(cfg, w, t)
    assert O.logits_error(O.forward(cfg, w, t[260:])[-10:], a[-10:]) > 1e-2
    cache = m.make_cache(1)
    m.forward_ragged([t[:300]], cache)
    m.forward_ragged([t[300:510]], cache)
    got = torch.cat([m.forward_ragged([[tok]], cache) for tok in t[510:]])
    assert O.logits_error(got, a[-10:]) < F32_TOL
    win = 24
    cfg = O.make_config([O.window_layer(2, 1, 16, 0.3, win, 20.0, 1)], vocab=40, width=32, streams=2, taps=1)
    w = O.random_weights(cfg, 13)
    m, _ = build(cfg, weights=w)
    t = toks(cfg, 90, 4)
    base = O.forward(cfg, w, t)[-1]
    for pos, seen in ((89 - win + 1, True), (89 - win, False)):
        t2 = list(t)
        t2[pos] = (t[pos] + 1) % 40
        moved = O.logits_error(O.forward(cfg, w, t2)[-1][None], base[None])
        assert (moved > 1e-4) if seen else (moved < 1e-12)
        for cut in (89, 89 - win, 60):
            cache = m.make_cache(1)
            m.forward_ragged([t2[:cut]], cache)
            got = torch.cat([m.forward_ragged([[tok]], cache) for tok in t2[cut:]])[-1:]
            assert O.logits_error(got, O.forward(cfg, w, t2)[-1][None]) < F32_TOL


def test_far_memory_of_the_delta_state():
    """A slow decay keeps a token readable 150 positions later, across a portion boundary; without the first portion's state the
    answer is clearly different."""
    cfg = O.make_config([O.delta_layer(1, 1, 32, 8, 2)], vocab=40, width=16, streams=2, taps=2)
    w = O.random_weights(cfg, 9)
    w["l0.mix.A_log"] = torch.full((1,), -7.0)
    m, _ = build(cfg, weights=w)
    t = toks(cfg, 160, 6)
    t2 = list(t)
    t2[3] = (t[3] + 1) % 40
    a, b = O.forward(cfg, w, t)[-1], O.forward(cfg, w, t2)[-1]
    assert O.logits_error(a[None], b[None]) > 1e-3
    cache = m.make_cache(1)
    m.forward_ragged([t[:80]], cache)
    got = m.forward_ragged([t[80:]], cache)
    assert O.logits_error(got, a[None]) < F32_TOL
    lost = m.forward_ragged([t[80:]], m.make_cache(1))
    assert O.logits_error(lost, a[None]) > 1e-2


def test_long_decoding(models):
    from mlx_parallm_b200 import utils
    cfg, m, w = models["odd"]
    t = toks(cfg, 330, 8)
    want = O.forward(cfg, w, t)
    cache = utils._kv_pool.get_for(m, 1)
    m.forward_ragged([t[:5]], cache)
    st = utils._decode_step_for(m, cache, 1, False)
    got = []
    for tok in t[5:]:
        st.tok.copy_(torch.tensor([tok], dtype=torch.int32))
        st.run()
        got.append(st.logits.clone())
    assert O.logits_error(torch.cat(got), want[5:]) < F32_TOL


def test_greedy_generation_through_generate_step(models):
    """The engine's own entry point: left-padded prompts with their lengths, prefill, then the captured decode step feeding
    its own argmax back.  Compared with greedy decoding of the oracle, request by request."""
    from mlx_parallm_b200 import utils
    cfg, m, w = models["mixed"]
    prompts = [toks(cfg, n, 40 + n) for n in (3, 9, 6)]
    L = max(len(p) for p in prompts)
    padded = torch.tensor([[0] * (L - len(p)) + p for p in prompts])
    n_new = 8
    gen = utils.generate_step(padded, m, prompt_lengths=[len(p) for p in prompts])
    got = torch.cat([y for _, (y, _) in zip(range(n_new), gen)], 1).cpu().tolist()
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            lg = O.forward(cfg, w, seq)[-1]
            best = int(lg.argmax())
            assert tok == best or float(lg[best] - lg[tok]) < 1e-3 * float(lg.abs().max())
            seq.append(tok)


def test_batch_generate_front_end(models):
    from fake_tokenizer import FakeTokenizer
    from mlx_parallm_b200 import utils
    from mlx_parallm_b200.tokenizer_utils import TokenizerWrapper
    cfg, m, w = models["mixed"]
    tok = TokenizerWrapper(FakeTokenizer(vocab_size=cfg["vocab"]))
    out = utils.batch_generate(m, tok, ["w5 w6", "w5 w6 w7 w8 w9 w10 w11"], max_tokens=5, format_prompts=False)
    alone = utils.batch_generate(m, tok, ["w5 w6"], max_tokens=5, format_prompts=False)
    assert len(out) == 2 and out[0] == alone[0]


def test_checkpoint_on_disk_and_trace_runner(tmp_path, models):
    """config.json + model.safetensors through load_model (the registry picks the class by the architecture's name), then the
    command-line trace runner on the same folder: prompt, decode steps and a request that ends early, against the oracle."""
    import json
    import os
    import subprocess
    import sys
    from safetensors.torch import save_file
    cfg, _, w = models["odd"]
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
    wb = {k: v.to(torch.bfloat16) for k, v in w.items()}
    a, b = toks(cfg, 12, 1), toks(cfg, 5, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:9], "want": [0, 8]}, {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[9:10], "want": [0]}, {"id": "b", "tokens": b[4:5], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[10:11], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[11:12], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    wa, wbb = O.forward(cfg, wb, a), O.forward(cfg, wb, b)
    V = cfg["vocab"]
    s0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, V))
    assert O.logits_error(s0, torch.stack([wa[0], wa[8], wbb[3]])) < F32_TOL
    s1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V))
    assert O.logits_error(s1, wa[9:10]) < F32_TOL
    assert not (out / "2.f32").exists()
    s3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4").reshape(1, V))
    assert O.logits_error(s3, wa[11:12]) < F32_TOL

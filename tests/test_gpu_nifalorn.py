"""Nifalorn on the GPU against the slow float64 oracle (tests/nifalorn_oracle.py): each mechanism alone, prompts against
token-by-token decoding, portions, ragged batches, rows given back and used again, far keys and chunk borders in prompts and in
decoding, the rotation, the expert groups, the looped span, other sizes, greedy generation through generate_step."""
import math

import numpy as np
import pytest
import torch

import nifalorn_oracle as O

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4        # float32 model against the float64 oracle (centred rms over the vocabulary, relative)
BF16_TOL = 6e-2       # bfloat16 matrix products


def build(cfg, seed=0, dtype=torch.float32, weights=None):
    from mlx_parallm_b200.utils import _get_classes
    Model, Args = _get_classes(cfg)
    w = O.random_weights(cfg, seed) if weights is None else weights
    return Model(Args.from_dict(cfg)).load_weights(w, device="cuda", dtype=dtype), w


def toks(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def residuals(cfg, w, t):
    res = []
    logits = O.forward(cfg, w, t, tap=lambda run, x: res.append(x.clone()))
    return logits, res


CONFIGS = {
    # every branch: the three mixers, dense / routed / no feed-forward, experts in groups with and without a shared one, a span
    # of two layers in the middle that runs three times
    "mixed": lambda: O.make_config([
        O.ssm_layer(4, 8, 12, 2, 4, conv=4, mlp=O.dense_mlp(40)),
        O.attention_layer(6, 2, 8, 12, 0.3, 0.35, 11, 4, base=100.0, scaling=(3.0, 1.0, 4.0, 40),
                          mlp=O.moe_mlp(8, 3, 24, groups=(4, 2), scale=1.7, shared_ff=16)),
        O.lightning_layer(3, 8, 16, [0.6, 0.9, 0.995], mlp=O.moe_mlp(6, 2, 16, groups=(2, 1), scale=0.8)),
        O.lightning_layer(2, 16, 8, [0.97, 0.5]),
    ], loop=(1, 3, 3), embed_scale=3.0, logit_scale=0.6),
    # sizes off the fast paths (odd width, heads, vector sizes), one key head for three heads, one state group, three norm parts,
    # the whole vector rotated, every expert chosen, a span that starts at the first layer
    "odd": lambda: O.make_config([
        O.attention_layer(6, 2, 6, 9, 0.4, 0.2, 7, 6, base=50.0, mlp=O.moe_mlp(6, 3, 13, groups=(3, 2), scale=2.5, shared_ff=9)),
        O.ssm_layer(3, 7, 5, 1, 3, conv=3, mlp=O.moe_mlp(5, 5, 11, shared_ff=6)),
        O.lightning_layer(3, 6, 11, [0.8, 0.9, 0.95], mlp=O.dense_mlp(13)),
    ], vocab=31, width=27, eps=1e-3, loop=(0, 2, 2), embed_scale=0.7, logit_scale=1.3),
    # wider heads: vector sizes of the tile kernels, a state of 128 rows, a value size that spans two thread blocks, as many
    # key heads as heads and as many state groups as heads, no convolution, one norm part, a span that runs once, one chunk
    # longer than any test prompt
    "wide": lambda: O.make_config([
        O.ssm_layer(2, 160, 128, 2, 1, conv=1, mlp=O.moe_mlp(3, 1, 24, groups=(3, 3), shared_ff=8)),
        O.attention_layer(2, 2, 64, 128, 0.12, 0.5, 4096, 32, base=1e6, scaling=(8.0, 1.0, 4.0, 512), mlp=O.dense_mlp(40)),
        O.lightning_layer(1, 128, 64, [0.93]),
    ], vocab=130, width=64, loop=(0, 3, 1)),
    # no span at all, one head
    "plain": lambda: O.make_config([
        O.lightning_layer(2, 8, 8, [0.6, 0.99], mlp=O.dense_mlp(24)),
        O.attention_layer(1, 1, 8, 8, 0.35, 0.8, 16, 2, mlp=O.dense_mlp(24)),
        O.ssm_layer(1, 16, 8, 1, 2, conv=2),
    ], vocab=50, width=32),
}


@pytest.fixture(scope="module")
def models():
    out = {}
    for name, mk in CONFIGS.items():
        cfg = mk()
        m, w = build(cfg, seed=len(name))
        out[name] = (cfg, m, w)
    return out


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M", [2, 40, 300])
def test_gemm_squared_relu_epilogue(dtype, M):
    from mlx_parallm_b200 import _lib, ops
    g = torch.Generator().manual_seed(M)
    ff, K = 72, 64
    x = torch.randn(M, K, generator=g).to(dtype)
    up = torch.randn(ff, K, generator=g).to(dtype)
    want = O.relu_squared(x.double() @ up.double().T)
    got = ops.gemm(x.cuda(), up.cuda(), _lib.GEMM_RELU_SQ)
    assert got.shape == (M, ff) and got.dtype == dtype
    tol = 1e-4 if dtype == torch.float32 else 0.03
    assert ((got.double().cpu() - want).abs() / (1.0 + want.abs())).max() < tol * math.sqrt(K)
    assert float(got.min()) >= 0.0 and float((got == 0).float().mean()) > 0.3          # negative pre-activations give zero


@pytest.mark.parametrize("E,top,count,keep,M", [(8, 3, 4, 2, 7), (16, 4, 4, 3, 40), (6, 3, 3, 2, 33), (12, 2, 12, 5, 9), (5, 5, 1, 1, 3),
                                                 (64, 8, 8, 4, 50), (6, 2, 2, 1, 300), (9, 3, 3, 3, 11)])
def test_group_routing(E, top, count, keep, M):
    """The picked experts and their weights against the oracle's routing, with picking scores that are mostly negative (a
    dropped group must lose against them) and extra columns beside the router's; the combination with a gated shared expert."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(E * 100 + M)
    W = 16
    h = torch.randn(M, W, generator=g, dtype=torch.float64)
    P = {"r.router": torch.randn(E, W, generator=g, dtype=torch.float64), "r.correction": torch.randn(E, generator=g, dtype=torch.float64) - 1.2}
    r = {"experts": E, "top": top, "scale": 1.7, "groups": {"count": count, "keep": keep}}
    want_ids, want_w = O.route(h, P, "r.", r)
    logits = torch.zeros(M, E + 3)
    logits[:, :E] = (h @ P["r.router"].T).float()
    logits[:, E:] = 50.0                                               # columns that do not belong to the router
    i32 = dict(dtype=torch.int32, device="cuda")
    ids, slot_of, token_of = torch.zeros(M, top, **i32), torch.zeros(M, top, **i32), torch.zeros(M * top, **i32)
    wts, seg = torch.zeros(M, top, device="cuda"), torch.zeros(E + 1, **i32)
    ops.moe_route_sigmoid(logits.cuda(), P["r.correction"].float().cuda(), ids, wts, seg, slot_of, token_of, top, count, keep, 1.7, experts=E)
    assert torch.equal(ids.cpu().long(), want_ids)
    assert (wts.cpu().double() - want_w).abs().max() < 1e-5
    seg_h, slot_h, tok_h = seg.cpu().tolist(), slot_of.cpu().view(-1).tolist(), token_of.cpu().tolist()
    assert seg_h[0] == 0 and seg_h[-1] == M * top and sorted(slot_h) == list(range(M * top))
    for i, s in enumerate(slot_h):
        e = int(ids.view(-1)[i])
        assert seg_h[e] <= s < seg_h[e + 1] and tok_h[s] == i // top
    ye, sh = torch.randn(M * top, 16, generator=g).cuda(), torch.randn(M, 16, generator=g).cuda()
    out = torch.empty(M, 16, device="cuda")
    gate = logits[:, E - 1:E].cuda()                                   # any column: one pre-activation per token
    ops.moe_combine(ye, slot_of, wts, sh, out, top, shared_gate=gate)
    want = torch.sigmoid(gate.cpu().double()) * sh.cpu().double() + (wts.cpu().double().unsqueeze(-1) * ye.cpu().double()[slot_of.cpu().long()]).sum(1)
    assert (out.cpu().double() - want).abs().max() < 1e-5
    ops.moe_combine(ye, slot_of, wts, sh, out, top)                    # no gate: the shared output is added as it is
    want = sh.cpu().double() + (wts.cpu().double().unsqueeze(-1) * ye.cpu().double()[slot_of.cpu().long()]).sum(1)
    assert (out.cpu().double() - want).abs().max() < 1e-5


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


@pytest.mark.parametrize("H,dv,N,G,parts,conv", [(4, 16, 16, 2, 2, 4), (3, 7, 5, 1, 3, 3), (2, 160, 40, 2, 1, 1), (6, 8, 130, 3, 4, 2),
                                                  (1, 70, 300, 1, 5, 6), (8, 4, 8, 8, 1, 4)])
def test_state_space_alone(H, dv, N, G, parts, conv):
    cfg = one_layer(O.ssm_layer(H, dv, N, G, parts, conv), vocab=40, width=24)
    w = O.random_weights(cfg, H * dv)
    got, want = mixer_alone(cfg, w, 37, 2)
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    got, want = mixer_alone(cfg, w, 37, 2, cuts=[1, 2, 5, 1, 1, 20, 7])         # the convolution's inputs cross every cut
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_state_space_parts():
    """What a wrong reading would change: the skip term, the gate before (not after) the norm, the norm's parts, the groups of
    B and C, the bias of the convolution.  Each variant of the weights moves the oracle, and the framework follows it."""
    cfg = one_layer(O.ssm_layer(4, 8, 6, 2, 2, 3), vocab=40, width=16)
    w = O.random_weights(cfg, 5)
    base = mixer_alone(cfg, w, 20, 3)
    assert (base[0] - base[1]).abs().max() < 2e-4 * max(1.0, float(base[1].abs().max()))
    for name, change in (("l0.mix.D", lambda t: t + 2.0), ("l0.mix.conv.b", lambda t: t + 1.0), ("l0.mix.dt_bias", lambda t: t + 3.0),
                         ("l0.mix.A_log", lambda t: t + 2.0), ("l0.mix.norm", lambda t: torch.cat([t[:16] * 3.0, t[16:]]))):
        w2 = dict(w)
        w2[name] = change(w[name])
        got, want = mixer_alone(cfg, w2, 20, 3)
        assert (want - base[1]).abs().max() > 1e-3, name
        assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max())), name
    # one half of the channels made huge: with the norm taken over all channels at once the other half would vanish
    w3 = dict(w)
    big = w["l0.mix.in"].clone()
    big[32:48] *= 40.0                                                           # the x channels of heads 0 and 1 (first norm part)
    w3["l0.mix.in"] = big
    got, want = mixer_alone(cfg, w3, 20, 3)
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("H,dk,dv", [(4, 16, 16), (3, 6, 11), (1, 128, 64), (2, 40, 160)])
def test_lightning_alone(H, dk, dv):
    decay = [0.5 + 0.499 * (i + 1) / H for i in range(H)]
    cfg = one_layer(O.lightning_layer(H, dk, dv, decay), vocab=40, width=32)
    w = O.random_weights(cfg, H + dk)
    got, want = mixer_alone(cfg, w, 41, 4)
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    got, want = mixer_alone(cfg, w, 41, 4, cuts=[3, 1, 30, 2, 5])
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("H,G,d,dv,chunk,rot,scaling", [(4, 2, 16, 16, 8, 8, None), (6, 2, 6, 9, 7, 6, None), (2, 2, 64, 128, 50, 32, (8.0, 1.0, 4.0, 64)),
                                                         (3, 1, 10, 5, 1, 4, None), (8, 1, 32, 32, 1000, 2, (4.0, 1.0, 4.0, 16)), (1, 1, 7, 3, 5, 6, None)])
def test_differential_attention_alone(H, G, d, dv, chunk, rot, scaling):
    cfg = one_layer(O.attention_layer(H, G, d, dv, d ** -0.5, 0.3, chunk, rot, base=200.0, scaling=scaling), vocab=40, width=32)
    w = O.random_weights(cfg, H + d)
    got, want = mixer_alone(cfg, w, 41, 4)
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    got, want = mixer_alone(cfg, w, 41, 4, cuts=[5, 1, 1, 9, 2, 23])
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_rotation_kernel():
    """Queries and keys of rows that stand at different positions: only the first rot_dims dimensions of every vector turn,
    in neighbouring pairs, by the position times the pair's rate; the values pass unchanged; the query takes the scale."""
    from mlx_parallm_b200 import ops
    from mlx_parallm_b200.models._sequence import rotary_rates
    H, G, maps, d, dv, rot = 3, 1, 2, 10, 5, 6
    rot_cfg = {"dims": rot, "base": 30.0, "scaling": {"factor": 5.0, "low": 1.0, "high": 4.0, "original": 20}}
    rates = rotary_rates(rot, 30.0, rot_cfg["scaling"])
    g = torch.Generator().manual_seed(1)
    pos = [0, 1, 2, 700, 31, 5]
    rows = [0, 0, 0, 1, 2, 2]
    M, Tcap = len(pos), 704
    nq, nk = H * maps * d, G * maps * d
    proj = torch.randn(M, nq + nk + G * dv + 3, generator=g)
    kc, vc = torch.zeros(3, G, Tcap, maps * d, device="cuda"), torch.zeros(3, G, Tcap, dv, device="cuda")
    q = torch.zeros(M, nq, device="cuda")
    i32 = dict(dtype=torch.int32, device="cuda")
    ops.rope_attn_prep(proj.cuda(), 0, nq, nq + nk, torch.tensor(rates, dtype=torch.float32, device="cuda"), rot, 0.25, q, kc, vc,
                       torch.tensor(rows, **i32), torch.tensor(pos, **i32), H, G, maps, d, dv)
    R = O.rotation_rates(rot_cfg)
    for t in range(M):
        wq = O.rotate_pairs(proj[t:t + 1, :nq].double().view(1, H * maps, d), R, start=pos[t]) * 0.25
        wk = O.rotate_pairs(proj[t:t + 1, nq:nq + nk].double().view(1, G * maps, d), R, start=pos[t])
        tol = 1e-6 * max(1.0, pos[t])                                      # the angle itself is a float32 product
        assert (q[t].double().cpu() - wq.reshape(-1)).abs().max() < tol
        assert (kc[rows[t], :, pos[t]].double().cpu().reshape(-1) - wk.reshape(-1)).abs().max() < 4 * tol
        assert torch.equal(vc[rows[t], :, pos[t]].cpu().reshape(-1), proj[t, nq + nk:nq + nk + G * dv])
        assert torch.equal(q[t].cpu().view(H * maps, d)[:, rot:], proj[t, :nq].view(H * maps, d)[:, rot:] * 0.25)
    assert int((kc != 0).any(-1).sum()) == M * G                            # nothing else was written


def attn_kernel_case(T, H, G, d, dv, chunk, hot=None, lam=0.7, dtype=torch.float32, seed=0, boost=30.0, decode=False, hot_map=0):
    """diff_attn over T cached positions of one row; every token is a query at its own position (``decode``: one launch per
    token, one token each).  A hot pair (query position, key position, in map ``hot_map``) gets a score far above the rest so
    that a key that is wrongly masked, skipped or misplaced shows."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(seed + T)
    q = torch.randn(T, H, 2, d, generator=g) * 0.3
    k = torch.randn(T, G, 2, d, generator=g) * 0.3
    v = torch.randn(T, G, dv, generator=g)
    if hot is not None:
        u = torch.randn(d, generator=g)
        u = u / u.norm()
        q[hot[0], :, hot_map] += boost * u
        k[hot[1], :, hot_map] += 3.0 * u
    if dtype != torch.float32:
        q = q.to(dtype).float()            # the 16-bit kernels round the query to the cache's type: give both sides that query
    kc = torch.zeros(2, G, T + 3, 2 * d)
    vc = torch.zeros(2, G, T + 3, dv)
    kc[1, :, :T] = k.reshape(T, G, 2 * d).transpose(0, 1)
    vc[1, :, :T] = v.transpose(0, 1)
    kc, vc = kc.to(dtype), vc.to(dtype)
    out = torch.zeros(T, H * dv + 8, dtype=dtype, device="cuda")
    i32 = dict(dtype=torch.int32, device="cuda")
    qd, kcd, vcd = q.reshape(T, -1).contiguous().cuda(), kc.cuda(), vc.cuda()
    eps, post = 1e-4, 0.6
    ws = torch.empty(max(ops.diff_attn_workspace_floats(1, H, 2, dv), 4), device="cuda")
    if decode:
        for t in range(T):
            ops.diff_attn(qd[t:t + 1], kcd, vcd, torch.ones(1, **i32), torch.tensor([t], **i32), out[t:t + 1, :H * dv], H, G, 2, d, dv,
                          chunk=chunk, lam=lam, eps=eps, post=post, cu=torch.tensor([0, 1], **i32), rows=torch.tensor([1], **i32), nb=1,
                          max_n=1, workspace=ws)
    else:
        ops.diff_attn(qd, kcd, vcd, torch.ones(T, **i32), torch.arange(T, **i32), out[:, :H * dv], H, G, 2, d, dv, chunk=chunk, lam=lam,
                      eps=eps, post=post, cu=torch.tensor([0, T], **i32), rows=torch.tensor([1], **i32), nb=1, max_n=T, workspace=ws)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    kd, vd = kc[1, :, :T].double().view(G, T, 2, d), vc[1, :, :T].double()
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    hidden = (j > i) | ((i // chunk != j // chunk) if chunk > 0 else torch.zeros(T, T, dtype=torch.bool))
    seen = torch.zeros(T, H, 2, dtype=torch.float64)                       # the weight of the hot key in each map
    for h in range(H):
        kv = h // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, h, mp].double() @ kd[kv, :, mp].T).masked_fill(hidden, -math.inf)
            p = torch.softmax(s, -1)
            if hot is not None:
                seen[:, h, mp] = p[:, hot[1]]
            a.append(p @ vd[kv])
        want[:, h] = post * O.rms_unit(a[0] - lam * a[1], eps)
    assert float(out[:, H * dv:].float().abs().max()) == 0.0          # columns beside the heads are not touched
    return out[:, :H * dv].double().cpu().view(T, H, dv), want, seen


# (tokens, chunk, hot query, hot key, whether the query sees the key)
BORDERS = [(600, 0, 599, 3, True), (600, 512, 599, 512, True), (600, 512, 599, 511, False), (70, 32, 63, 32, True), (70, 32, 64, 63, False),
           (70, 32, 64, 64, True), (130, 64, 127, 64, True), (130, 64, 128, 127, False), (97, 96, 95, 0, True), (97, 96, 96, 95, False),
           (33, 33, 32, 0, True), (40, 1, 7, 6, False), (1, 4, None, None, None), (2, 2, 1, 0, True), (3, 2, 2, 1, False)]


@pytest.mark.parametrize("T,chunk,hq,hk,visible", BORDERS)
@pytest.mark.parametrize("decode", [False, True])
def test_attention_far_keys_and_chunk_borders(T, chunk, hq, hk, visible, decode):
    if decode and T > 200:
        T, chunk, hq, hk = T - 400, max(chunk - 400, 0), hq - 400, max(hk - 400, 0)    # the same border, fewer launches
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        for hot_map in (0, 1):
            got, want, seen = attn_kernel_case(T, 4, 2, 16, 24, chunk, None if hq is None else (hq, hk), dtype=dtype, decode=decode,
                                               hot_map=hot_map)
            assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max()))
            if hq is not None:
                w_hot = float(seen[hq, :, hot_map].min())
                assert (w_hot > 0.9) if visible else (float(seen[hq].max()) == 0.0)


@pytest.mark.parametrize("T,chunk,hq,hk", [(600, 0, 599, 3), (300, 256, 299, 256), (300, 256, 299, 255), (70, 64, 63, 31), (70, 64, 64, 63),
                                           (130, 0, 128, 63), (130, 0, 129, 64), (129, 128, 128, 128), (65, 0, 64, 0), (64, 0, 63, 0),
                                           (5, 0, 4, 1), (100, 33, 98, 66)])
def test_attention_tile_sizes_far_keys_and_tile_borders(T, chunk, hq, hk):
    """Sizes the tensor-core kernel takes (16-bit, vector and value sizes 32, 64, 128): hot pairs across its key tiles and its
    query tiles, chunks that start inside a tile, prompts and single tokens."""
    for d, dv in ((64, 64), (128, 64), (64, 128), (32, 32), (32, 128), (128, 128), (32, 64), (64, 32), (128, 32)):
        for decode in (False, True):
            if decode and T > 200:
                continue
            got, want, _ = attn_kernel_case(T, 4, 2, d, dv, chunk, (hq, hk), dtype=torch.bfloat16, seed=d + dv, decode=decode, lam=0.45)
            assert (got - want).abs().max() < 3e-2 * max(1.0, float(want.abs().max())), (d, dv, decode)


def test_attention_over_ragged_portions():
    """Three entries in one launch: a fresh prompt, a short and a long continuation of rows that already hold keys (their
    first positions are neither multiples of the tile sizes nor of the chunk), in rows out of order; float32 and bfloat16."""
    from mlx_parallm_b200 import ops
    H, G, d, dv, chunk, lam, eps, post = 6, 3, 64, 128, 48, 0.8, 1e-5, 0.4
    g = torch.Generator().manual_seed(5)
    entries = [(2, 0, 70), (0, 37, 5), (1, 100, 130)]                    # (cache row, first position, tokens)
    Tcap = 256
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        kc = (torch.randn(3, G, Tcap, 2 * d, generator=g) * 0.3).to(dtype)
        vc = torch.randn(3, G, Tcap, dv, generator=g).to(dtype)
        M = sum(n for _, _, n in entries)
        q = (torch.randn(M, H, 2, d, generator=g) * 0.3).to(dtype).float()
        i32 = dict(dtype=torch.int32, device="cuda")
        cu, t_row, t_pos = [0], [], []
        for r, p0, n in entries:
            cu.append(cu[-1] + n)
            t_row += [r] * n
            t_pos += list(range(p0, p0 + n))
        out = torch.zeros(M, H * dv, dtype=dtype, device="cuda")
        ops.diff_attn(q.reshape(M, -1).contiguous().cuda(), kc.cuda(), vc.cuda(), torch.tensor(t_row, **i32), torch.tensor(t_pos, **i32), out,
                      H, G, 2, d, dv, chunk=chunk, lam=lam, eps=eps, post=post, cu=torch.tensor(cu, **i32),
                      rows=torch.tensor([e[0] for e in entries], **i32), nb=3, max_n=130)
        got = out.double().cpu().view(M, H, dv)
        for t in range(M):
            r, p = t_row[t], t_pos[t]
            lo = p // chunk * chunk
            for h in range(H):
                kv = h // (H // G)
                a = []
                for mp in range(2):
                    s = kc[r, kv, lo:p + 1, mp * d:(mp + 1) * d].double() @ q[t, h, mp].double()
                    a.append(torch.softmax(s, 0) @ vc[r, kv, lo:p + 1].double())
                want = post * O.rms_unit(a[0] - lam * a[1], eps)
                assert (got[t, h] - want).abs().max() < tol * max(1.0, float(want.abs().max())), (t, h)


@pytest.mark.parametrize("H,G,d,dv,nb", [(8, 2, 64, 64, 5), (16, 1, 32, 128, 3), (4, 4, 64, 128, 40), (6, 3, 128, 64, 150), (3, 1, 10, 7, 9)])
def test_attention_decode_batches(H, G, d, dv, nb):
    """One token per entry at positions from 0 to several hundred (first token, tile and chunk borders, many tiles), rows out of
    order."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(H + nb)
    Tcap, chunk, lam, eps, post = 700, 200, 0.6, 1e-5, 0.7
    special = [0, 1, 63, 64, 65, 127, 128, 199, 200, 201, 699, 640, 400, 399]
    pos = [special[i] if i < len(special) else int(torch.randint(0, Tcap, (1,), generator=g)) for i in range(nb)]
    rows = torch.randperm(nb, generator=g).tolist()
    R = min(nb, 14)                                                        # check these entries against the slow sum
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 2e-2)):
        kc = (torch.randn(nb, G, Tcap, 2 * d, generator=g) * 0.3).to(dtype)
        vc = torch.randn(nb, G, Tcap, dv, generator=g).to(dtype)
        q = (torch.randn(nb, H, 2, d, generator=g) * 0.4).to(dtype).float()
        i32 = dict(dtype=torch.int32, device="cuda")
        out = torch.zeros(nb, H * dv, dtype=dtype, device="cuda")
        ws = torch.empty(max(ops.diff_attn_workspace_floats(min(nb, 64), H, 2, dv), 4), device="cuda")
        ops.diff_attn(q.reshape(nb, -1).contiguous().cuda(), kc.cuda(), vc.cuda(), torch.tensor(rows, **i32), torch.tensor(pos, **i32), out,
                      H, G, 2, d, dv, chunk=chunk, lam=lam, eps=eps, post=post, cu=torch.arange(nb + 1, **i32),
                      rows=torch.tensor(rows, **i32), nb=nb, max_n=1, workspace=ws)
        got = out.double().cpu().view(nb, H, dv)
        for e in range(R):
            r, p = rows[e], pos[e]
            lo = p // chunk * chunk
            for h in range(H):
                kv = h // (H // G)
                a = []
                for mp in range(2):
                    s = kc[r, kv, lo:p + 1, mp * d:(mp + 1) * d].double() @ q[e, h, mp].double()
                    a.append(torch.softmax(s, 0) @ vc[r, kv, lo:p + 1].double())
                want = post * O.rms_unit(a[0] - lam * a[1], eps)
                assert (got[e, h] - want).abs().max() < tol * max(1.0, float(want.abs().max())), (e, h, p)


def test_one_map_is_plain_attention():
    """maps = 1, no division by the root mean square: the kernel is an ordinary chunked softmax attention."""
    from mlx_parallm_b200 import ops
    T, H, G, d, dv, chunk = 50, 4, 2, 16, 8, 20
    g = torch.Generator().manual_seed(2)
    q, k, v = torch.randn(T, H, d, generator=g) * 0.5, torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
    i32 = dict(dtype=torch.int32, device="cuda")
    out = torch.zeros(T, H * dv, device="cuda")
    ops.diff_attn(q.reshape(T, -1).contiguous().cuda(), k.transpose(0, 1).contiguous()[None].cuda(), v.transpose(0, 1).contiguous()[None].cuda(),
                  torch.zeros(T, **i32), torch.arange(T, **i32), out, H, G, 1, d, dv, chunk=chunk, post=2.0)
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // 2].double().T).masked_fill((j > i) | (i // chunk != j // chunk), -math.inf)
        want = 2.0 * torch.softmax(s, -1) @ v[:, h // 2].double()
        assert (out.view(T, H, dv)[:, h].double().cpu() - want).abs().max() < 1e-4


# ---- whole models -------------------------------------------------------------------------------------------------------------
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
    assert [i for i, _ in got_res] == O.layer_runs(cfg)
    for k, r in enumerate(res):
        assert (got_res[k][1].double().cpu() - r).abs().max() < 2e-4 * max(1.0, float(r.abs().max())), f"residual after run {k}"
    assert O.logits_error(got, want) < F32_TOL


@pytest.mark.parametrize("name", list(CONFIGS))
def test_bfloat16_model(name):
    cfg = CONFIGS[name]()
    m, w = build(cfg, seed=3, dtype=torch.bfloat16)
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
        O.attention_layer(4, 2, 64, 128, 0.125, 0.4, 128, 32, base=1e4, mlp=O.moe_mlp(4, 2, 64, groups=(2, 1), scale=1.5, shared_ff=64)),
        O.ssm_layer(4, 32, 64, 2, 2, conv=4, mlp=O.dense_mlp(128)),
        O.lightning_layer(2, 64, 64, [0.9, 0.99]),
        O.attention_layer(8, 8, 32, 64, 0.17, 0.6, 100, 16),
    ], vocab=200, width=128, loop=(0, 2, 2))
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
    """The last routed layer's choices, read back from the step's scratch, are the oracle's for every token."""
    cfg, m, w = models["mixed"]
    t = toks(cfg, 20, 9)
    _, res = residuals(cfg, w, t)
    m.forward_ragged([t], m.make_cache(1))
    # runs: 0 | 1 2 | 1 2 | 1 2 | 3; the last routed run is layer 2 in run 6.  Its feed-forward reads the stream after its mixer.
    P = {k: v.double() for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = res[5]
    x = x + O.lightning(O.norm_one_plus(x, P["l2.norm1"], eps), P, "l2.mix.", cfg["layers"][2]["mixer"], eps)
    ids, _ = O.route(O.norm_one_plus(x, P["l2.norm2"], eps), P, "l2.mlp.", cfg["layers"][2]["mlp"]["router"])
    a = next(iter(m._arenas.values()))
    got = a["s"].get("moe_ids", torch.int32, len(t), 2).cpu().tolist()
    assert got == ids.tolist()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_single_tokens_equal_one_pass(models, name):
    """A prompt cut into portions of 1, 2, 3, ... tokens, and fed token by token, gives the logits of one pass; the portions
    cross the convolution's reach and the attention's chunks."""
    cfg, m, w = models[name]
    t = toks(cfg, 50, 4)
    want = O.forward(cfg, w, t)
    for cuts in ([50], [1, 2, 3, 5, 8, 13, 18], [2] * 25, [1] * 50, [47, 1, 2], [49, 1], [33, 17]):
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
    sees no state, no convolution inputs and no keys of the old one, in any pass of the span."""
    cfg, m, w = models["mixed"]
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


def test_first_tokens_and_short_sequences(models):
    for name in ("mixed", "odd"):
        cfg, m, w = models[name]
        seqs = [toks(cfg, n, 30 + n) for n in (1, 1, 2, 3, 4)]
        got = m.forward_ragged(seqs, m.make_cache(5), want=[list(range(len(s))) for s in seqs])
        want = torch.cat([O.forward(cfg, w, s) for s in seqs])
        assert O.logits_error(got, want) < F32_TOL


def test_each_pass_of_the_span_keeps_its_own_state():
    """Layers that run twice hold two states and two key caches: decoding after a prompt must continue each pass from its own.
    With one shared state (or the second pass starting from the first one's) the continuation differs from the oracle."""
    cfg = O.make_config([O.ssm_layer(2, 8, 8, 1, 1, conv=3), O.attention_layer(2, 1, 8, 8, 0.4, 0.3, 64, 4), O.lightning_layer(2, 8, 8, [0.9, 0.99])],
                        vocab=40, width=16, loop=(0, 3, 2))
    m, w = build(cfg, seed=11)
    t = toks(cfg, 40, 3)
    want = O.forward(cfg, w, t)
    cache = m.make_cache(1)
    assert len(cache) == 6 + 1
    got = [m.forward_ragged([t[:25]], cache, want=[[24]])]
    for tok in t[25:]:
        got.append(m.forward_ragged([[tok]], cache))
    assert O.logits_error(torch.cat(got), want[24:]) < F32_TOL


def test_far_memory_of_the_recurrent_states():
    """A decay close to one keeps a token readable 150 positions later, across a portion boundary, in the linear attention and
    in the state-space layer; without the first portion's state the answer is clearly different."""
    layers = {"lightning": O.lightning_layer(1, 32, 8, [0.9995]), "mamba2": O.ssm_layer(1, 8, 32, 1, 1, conv=2)}
    for kind, layer in layers.items():
        cfg = O.make_config([layer], vocab=40, width=16)
        w = O.random_weights(cfg, 9)
        if kind == "mamba2":
            w["l0.mix.A_log"] = torch.full((1,), -7.0)                         # exp(-exp(-7) dt): almost nothing is forgotten
        m, _ = build(cfg, weights=w)
        t = toks(cfg, 160, 6)
        t2 = list(t)
        t2[3] = (t[3] + 1) % 40
        a, b = O.forward(cfg, w, t)[-1], O.forward(cfg, w, t2)[-1]
        assert O.logits_error(a[None], b[None]) > 1e-3, kind
        cache = m.make_cache(1)
        m.forward_ragged([t[:80]], cache)
        got = m.forward_ragged([t[80:]], cache)
        assert O.logits_error(got, a[None]) < F32_TOL, kind
        lost = m.forward_ragged([t[80:]], m.make_cache(1))
        assert O.logits_error(lost, a[None]) > 1e-2, kind


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

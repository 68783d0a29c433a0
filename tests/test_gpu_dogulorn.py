"""Dogulorn on the GPU against the slow float64 oracle (tests/dogulorn_oracle.py): each mechanism alone, prompts against
token-by-token decoding, portions, ragged batches, rows given back and used again, window edges and far keys, other sizes,
greedy generation through generate_step."""
import math

import numpy as np
import pytest
import torch

import dogulorn_oracle as O

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4        # float32 model against the float64 oracle (centred rms over the vocabulary, relative)
BF16_TOL = 6e-2       # bfloat16 matrix products


def build(cfg, seed=0, dtype=torch.float32):
    from mlx_parallm_b200.utils import _get_classes
    Model, Args = _get_classes(cfg)
    w = O.random_weights(cfg, seed)
    return Model(Args.from_dict(cfg)).load_weights(w, device="cuda", dtype=dtype), w


def toks(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


MLP = {"kind": "dense", "ff": 40, "limit": 1.5}
CONFIGS = {
    # every branch: own latents, shared latents, delta with and without feed-forward, attention without feed-forward, no window
    "mixed": lambda: O.make_config([
        O.attn_layer(3, 8, 16, 24, 32, window=7, scale=0.3, mlp=MLP),
        O.delta_layer(4, 2, 16, 8, conv=4),
        O.attn_layer(2, 16, 8, 16, 32, window=5, kv_from=0),
        O.delta_layer(3, 3, 8, 24, conv=2, mlp={"kind": "dense", "ff": 56, "limit": 0.75}),
        O.attn_layer(5, 8, 8, 8, 16, window=0, mlp=MLP),
    ]),
    # sizes off the fast paths (odd width and ranks), one kv head for three heads, no bigram, no token input, window 1
    "odd": lambda: O.make_config([
        O.delta_layer(3, 1, 5, 7, conv=3),
        O.attn_layer(1, 6, 10, 9, 11, window=1, mlp={"kind": "dense", "ff": 13, "limit": 3.0}),
        O.attn_layer(2, 6, 10, 9, 11, window=3, kv_from=1),
    ], vocab=31, width=27, eps=1e-3, emb_scale=1.0, bigram=None, side_dim=0),
    # wider heads: key size 40 pads to 64 state rows, value size 160 spans two thread blocks, rank 72
    "wide": lambda: O.make_config([
        O.delta_layer(2, 1, 40, 160, conv=1, mlp=MLP),
        O.attn_layer(4, 16, 24, 40, 72, window=33),
    ], vocab=130, width=64, bigram=(7, 3, 1), side_dim=4),
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
@pytest.mark.parametrize("M,N,K", [(1, 10, 16), (3, 7, 5), (8, 64, 48), (9, 130, 72), (70, 33, 40), (200, 96, 128), (300, 64, 24)])
def test_gemm_shapes(dtype, M, N, K):
    from mlx_parallm_b200 import _lib, ops
    g = torch.Generator().manual_seed(M * N + K)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = torch.randn(N, K, generator=g).to(dtype)
    want = x.double() @ w.double().T
    got = ops.gemm(x.cuda(), w.cuda(), _lib.GEMM_STORE_F32)
    tol = 1e-5 if dtype == torch.float32 else 1e-5          # same products and fp32 accumulation: only summation order differs
    assert (got.double().cpu() - want).abs().max() <= tol * math.sqrt(K) * 8
    got16 = ops.gemm(x.cuda(), w.cuda(), _lib.GEMM_STORE)
    assert got16.dtype == dtype and (got16.double().cpu() - want).abs().max() <= (1e-4 if dtype == torch.float32 else 0.05) * math.sqrt(K)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M", [2, 40])
def test_gemm_gated_epilogue_and_heads(dtype, M):
    from mlx_parallm_b200 import _lib, ops
    g = torch.Generator().manual_seed(5)
    K, F, lim = 32, 24, 0.8
    x = torch.randn(M, K, generator=g).to(dtype)
    gate, up = torch.randn(F, K, generator=g).to(dtype), torch.randn(F, K, generator=g).to(dtype)
    gu = torch.stack([gate, up], 1).reshape(2 * F, K)
    a = torch.clamp(x.double() @ gate.double().T, max=lim)
    u = torch.clamp(x.double() @ up.double().T, -lim, lim)
    want = a * torch.sigmoid(1.702 * a) * (u + 1)
    got = ops.gemm(x.cuda(), gu.cuda().contiguous(), _lib.GEMM_GLU_CLAMP, limit=lim)
    assert got.shape == (M, F) and (got.double().cpu() - want).abs().max() < (1e-4 if dtype == torch.float32 else 0.04)
    # one weight block per head, operands strided inside wider rows
    H, dk, R = 3, 8, 16
    q = torch.randn(M, H * dk, generator=g).to(dtype)
    wk = torch.randn(H, R, dk, generator=g).to(dtype)
    out = torch.empty(M, H * R, dtype=torch.float32, device="cuda")
    ops.gemm(q.cuda(), wk.cuda(), _lib.GEMM_STORE_F32, out=out, batch=H, strides=(dk, R * dk, R), M=M, N=R, K=dk, ldx=H * dk, ldw=dk,
             ldy=H * R)
    want = torch.einsum("mhd,hrd->mhr", q.double().view(M, H, dk), wk.double()).reshape(M, H * R)
    assert (out.double().cpu() - want).abs().max() < 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(9, 130, 72), (17, 72, 64), (40, 264, 200), (64, 520, 128), (65, 8, 64), (128, 72, 72), (300, 264, 200), (1000, 520, 512), (129, 1100, 64), (4100, 640, 136),
                                   (33, 9700, 64), (20, 9500, 200), (32, 2048, 2080), (50, 1000, 1700)])
def test_gemm_tcgen05_tiles(dtype, M, N, K):
    """Nine rows and more with K >= 64 run on tcgen05: ragged tile edges in all three dimensions, every tile width, all epilogues,
    against float64 and against the mma.sync kernel.  Up to 64 rows take the decode variant (weights on the M side, a 32- or
    64-token N side, transposed store, K split over several CTAs where the output is narrow and K long)."""
    from mlx_parallm_b200 import _lib, ops
    L = _lib.lib()
    g = torch.Generator().manual_seed(M + N + K)
    x = (torch.randn(M, K, generator=g) / 4).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) / 4).to(dtype).cuda()
    want = x.double() @ w.double().T
    got = ops.gemm(x, w, _lib.GEMM_STORE_F32)
    got16 = ops.gemm(x, w, _lib.GEMM_STORE)
    L.b200p_gemm_set_path(1)
    try:
        other = ops.gemm(x, w, _lib.GEMM_STORE_F32)
    finally:
        L.b200p_gemm_set_path(0)
    assert L.b200p_gemm_tc_fault() == 0
    assert (got.double() - want).abs().max() <= 2e-5 * math.sqrt(K)
    assert (got - other).abs().max() <= 2e-5 * math.sqrt(K)
    assert got16.dtype == dtype and (got16.double() - want).abs().max() <= 0.02 * math.sqrt(K) / 4
    if N % 2 == 0:
        lim = 0.7
        a = torch.clamp(want[:, 0::2], max=lim)
        u = torch.clamp(want[:, 1::2], -lim, lim)
        glu = ops.gemm(x, w, _lib.GEMM_GLU_CLAMP, limit=lim)
        assert glu.shape == (M, N // 2) and (glu.double() - a * torch.sigmoid(1.702 * a) * (u + 1)).abs().max() < 0.02


@pytest.mark.parametrize("M", [330, 24, 57])
def test_gemm_tcgen05_heads_and_strides(M):
    """One weight block per head, operands and outputs strided inside wider rows (3-d tensor maps)."""
    from mlx_parallm_b200 import _lib, ops
    g = torch.Generator().manual_seed(11)
    H, dk, R = 3, 64, 40
    q = (torch.randn(M, H * dk, generator=g) / 4).to(torch.bfloat16).cuda()
    wk = (torch.randn(H, R, dk, generator=g) / 4).to(torch.bfloat16).cuda()
    want = torch.einsum("mhd,hrd->mhr", q.double().view(M, H, dk), wk.double()).reshape(M, H * R)
    for epi, dt, tol in ((_lib.GEMM_STORE_F32, torch.float32, 2e-4), (_lib.GEMM_STORE, torch.bfloat16, 0.03)):
        out = torch.full((M, H * R), 7.0, dtype=dt, device="cuda")
        ops.gemm(q, wk, epi, out=out, batch=H, strides=(dk, R * dk, R), M=M, N=R, K=dk, ldx=H * dk, ldw=dk, ldy=H * R)
        assert (out.double() - want).abs().max() < tol
    assert _lib.lib().b200p_gemm_tc_fault() == 0


def test_norm_add_norm_parts():
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(1)
    M, W, eps = 5, 37, 1e-3
    h, y = torch.randn(M, W, generator=g), torch.randn(M, W, generator=g) * 3
    wp, wn = torch.randn(W, generator=g), torch.randn(W, generator=g)
    hd = h.cuda()
    x = torch.empty(M, W, device="cuda")
    raw = torch.empty(M, W, device="cuda")
    ops.norm_add_norm(hd, eps, torch.float32, y=y.cuda(), w_post=wp.cuda(), w_next=wn.cuda(), x_out=x, raw_out=raw)
    h2 = h.double() + O.rms_norm(y.double(), wp.double(), eps)
    assert (hd.double().cpu() - h2).abs().max() < 1e-5 and (raw.double().cpu() - h2).abs().max() < 1e-5
    assert (x.double().cpu() - O.rms_norm(h2, wn.double(), eps)).abs().max() < 1e-5


def test_hashed_embedding_across_portions():
    """The pair (previous, current) must also be right at the start of a portion (previous token from the row's state) and at
    the very first token (the extra row); large multipliers must not overflow."""
    cfg = O.make_config([O.delta_layer(1, 1, 4, 4, conv=1)], vocab=50, width=8, bigram=(47, 2 ** 30 + 3, 2 ** 29 + 1), side_dim=0)
    m, w = build(cfg)
    t = toks(cfg, 9, 3)
    P = {k: v.double() for k, v in w.items()}
    big = cfg["embedding"]["bigram"]
    want = O.hashed_embedding(t, P["embed"], P["bigram"], cfg["embedding"]["scale"], big["buckets"], big["mul_prev"], big["mul_cur"])
    got = []
    from mlx_parallm_b200 import ops
    for lo, hi in ((0, 1), (1, 4), (4, 5), (5, 9)):          # the kernel alone, one portion at a time, in row 1 of 2
        n = hi - lo
        ids = torch.tensor(t[lo:hi], dtype=torch.int32, device="cuda")
        i32 = dict(dtype=torch.int32, device="cuda")
        cu, rows = torch.tensor([0, n], **i32), torch.tensor([1], **i32)
        lengths = torch.tensor([0, lo], **i32)
        last = torch.tensor([0, t[lo - 1] if lo else 0], **i32)
        tr, tp, to = (torch.empty(n, **i32) for _ in range(3))
        ops.ragged_plan(cu, rows, lengths, tr, tp, to, 1, n)
        h = torch.empty(n, 8, device="cuda")
        ops.embed_hashed(ids, tr, tp, to, last, m.embed.weight, m.embed.bigram, h, m.embed.scale, m.embed.buckets, m.embed.mul_prev,
                         m.embed.mul_cur)
        got.append(h.cpu())
    assert (torch.cat(got).double() - want).abs().max() < 1e-6


def _attn_kernel_case(T, H, R, window, hot_query, hot_key, dtype=torch.float32):
    """Random latents and queries; query ``hot_query`` and latent ``hot_key`` are made parallel and long, so that head 0 of
    that query puts nearly all its weight on that key exactly when it may see it."""
    g = torch.Generator().manual_seed(T + R)
    c = torch.randn(T, R, generator=g) * 0.3
    q = torch.randn(T, H, R, generator=g) * 0.3
    d = torch.randn(R, generator=g)
    d = d / d.norm()
    c[hot_key] = 6.0 * d
    q[hot_query, 0] = 6.0 * d
    c = c.to(dtype)
    want = torch.zeros(T, H, R, dtype=torch.float64)
    for i in range(T):
        lo = 0 if window <= 0 else max(0, i - window + 1)
        p = torch.softmax(torch.einsum("hr,jr->hj", q[i].double(), c[lo:i + 1].double()) * 0.5, -1)
        want[i] = p @ c[lo:i + 1].double()
    return q, c, want


@pytest.mark.parametrize("T,window,dist", [(80, 16, 15), (80, 16, 16), (70, 33, 32), (70, 33, 33), (600, 0, 577), (90, 64, 63), (90, 64, 64),
                                           (40, 1, 0), (40, 1, 1)])
def test_latent_attention_window_edges_prompt_and_decode(T, window, dist):
    """A dominant key ``dist`` positions back: just inside the window it decides the output, one further it must be unseen.
    The same positions through one prompt pass and through single-token steps over the cache."""
    from mlx_parallm_b200 import ops
    H, R = 3, 40
    iq = T - 2
    q, c, want = _attn_kernel_case(T, H, R, window, iq, iq - dist)
    i32 = dict(dtype=torch.int32, device="cuda")
    cache = torch.zeros(2, T + 5, R, device="cuda")
    cache[1, :T] = c.cuda()
    rows, pos = torch.full((T,), 1, **i32), torch.arange(T, **i32)
    out = torch.empty(T, H * R, device="cuda")
    ops.latent_attn(q.reshape(T, H * R).cuda().contiguous(), cache, rows, pos, out, H, R, window, 0.5)
    assert (out.double().cpu().view(T, H, R) - want).abs().max() < 1e-4
    inside = window <= 0 or dist < window
    assert (want[iq, 0] - c[iq - dist].double()).abs().max() < 0.2 if inside else (want[iq, 0] - c[iq - dist].double()).abs().max() > 1.0
    for i in (iq - 1, iq, iq + 1):          # decoded alone
        o1 = torch.empty(1, H * R, device="cuda")
        ops.latent_attn(q[i].reshape(1, H * R).cuda().contiguous(), cache, rows[:1], pos[i:i + 1], o1, H, R, window, 0.5)
        assert torch.equal(o1[0], out[i])


# ---- whole models -------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prompt_logits_and_residuals_match_the_oracle(models, name):
    cfg, m, w = models[name]
    t = toks(cfg, 45, 1)
    res = []
    want = O.forward(cfg, w, t, res)
    got_res = {}
    m.residual_tap = lambda layer, kind, h: got_res.__setitem__(layer, h.clone())
    try:
        got = m.forward_ragged([t], m.make_cache(1), want=[list(range(len(t)))])
    finally:
        m.residual_tap = None
    for i, r in enumerate(res):
        assert (got_res[i].double().cpu() - r).abs().max() < 2e-4 * max(1.0, float(r.abs().max())), f"residual after layer {i}"
    assert O.logits_error(got, want) < F32_TOL


@pytest.mark.parametrize("name", list(CONFIGS))
def test_bfloat16_model(name):
    cfg = CONFIGS[name]()
    m, w = build(cfg, seed=3, dtype=torch.bfloat16)
    t = toks(cfg, 60, 2)
    got = m.forward_ragged([t], m.make_cache(1), want=[list(range(len(t)))])
    want = O.forward(cfg, w, t)
    per_pos = sorted(O.logits_error(got[i:i + 1], want[i:i + 1]) for i in range(len(t)))
    # 8 mantissa bits through several narrow layers: a few percent at the typical position, never a different answer
    assert per_pos[len(t) // 2] < BF16_TOL and per_pos[-1] < 1.0, per_pos[-3:]


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_single_tokens_equal_one_pass(models, name):
    """A prompt cut into portions of 1, 2, 3, ... tokens, and fed token by token, gives the logits of one pass; the portions
    cross every window edge and the convolution's reach."""
    cfg, m, w = models[name]
    t = toks(cfg, 50, 4)
    want = O.forward(cfg, w, t)
    for cuts in ([50], [1, 2, 3, 5, 8, 13, 18], [2] * 25, [1] * 50, [47, 1, 2], [49, 1]):
        cache = m.make_cache(3)
        got, lo = [], 0
        for n in cuts:
            got.append(m.forward_ragged([t[lo:lo + n]], cache, rows=[2], want=[list(range(n))]))
            lo += n
        assert O.logits_error(torch.cat(got), want) < F32_TOL, cuts


@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_decode_step_graph_against_prompt(models, name):
    """Most of a prompt in one pass, the rest through the engine's captured decode step (the generation path), 70 tokens long:
    past every window of the config."""
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
    # a second group of the same batch size, stepped in turns with the first one whose row list differs: the scratch (and the
    # row list the captured graph reads) is shared by both steps and must be rewritten when the other one ran in between
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
    """Four prompts of 1, 2, 17 and 40 tokens in one pass, then decoded together while the short ones end: bit-equal to each
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
    sees no state, no latents and no previous token of the old one."""
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
    """Sequences shorter than the convolution, one-token sequences in a batch, and the first-token bucket."""
    cfg, m, w = models["mixed"]
    seqs = [toks(cfg, n, 30 + n) for n in (1, 1, 2, 3, 4)]
    got = m.forward_ragged(seqs, m.make_cache(5), want=[list(range(len(s))) for s in seqs])
    want = torch.cat([O.forward(cfg, w, s) for s in seqs])
    assert O.logits_error(got, want) < F32_TOL


def test_far_memory_of_the_recurrence():
    """With decay close to one and wide keys a write is still readable 150 tokens later (every later write erases only the part
    along its own key): the state must survive a long prompt and a portion boundary in between."""
    cfg = O.make_config([O.delta_layer(1, 1, 64, 8, conv=2)], vocab=40, width=16, bigram=None, side_dim=0)
    w = O.random_weights(cfg, 9)
    w["l0.mix.A_log"] = torch.full((1,), -9.0).to(torch.bfloat16)          # decay = exp(-exp(-9) * softplus) ~ 1
    from mlx_parallm_b200.utils import _get_classes
    Model, Args = _get_classes(cfg)
    m = Model(Args.from_dict(cfg)).load_weights(w, device="cuda", dtype=torch.float32)
    t = toks(cfg, 160, 6)
    t2 = list(t)
    t2[3] = (t[3] + 1) % 40
    a, b = O.forward(cfg, w, t)[-1], O.forward(cfg, w, t2)[-1]
    assert O.logits_error(a[None], b[None]) > 1e-3                        # the oracle itself remembers token 3
    cache = m.make_cache(1)
    m.forward_ragged([t[:80]], cache)
    got = m.forward_ragged([t[80:]], cache)
    assert O.logits_error(got, a[None]) < F32_TOL
    lost = m.forward_ragged([t[80:]], m.make_cache(1))                    # without the first portion's state: clearly different
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
    its own argmax back.  Compared with greedy decoding of the oracle, request by request (float32: no near-ties expected at
    these sizes; a differing token must be a near-tie of the oracle)."""
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
    # the rectangular call without lengths feeds the padding like any token (the other models' behaviour)
    gen = utils.generate_step(padded[1:2, L - 9:], m)
    again = torch.cat([y for _, (y, _) in zip(range(n_new), gen)], 1).cpu().tolist()[0]
    assert again == got[1]


def test_batch_generate_front_end(models):
    from fake_tokenizer import FakeTokenizer
    from mlx_parallm_b200 import utils
    from mlx_parallm_b200.tokenizer_utils import TokenizerWrapper
    cfg, m, w = models["mixed"]
    tok = TokenizerWrapper(FakeTokenizer(vocab_size=cfg["vocab"]))
    out = utils.batch_generate(m, tok, ["w5 w6", "w5 w6 w7 w8 w9 w10 w11"], max_tokens=5, format_prompts=False)
    alone = utils.batch_generate(m, tok, ["w5 w6"], max_tokens=5, format_prompts=False)
    assert len(out) == 2 and out[0] == alone[0]


@pytest.mark.parametrize("R,window", [(32, 0), (64, 9), (96, 64), (256, 65), (512, 40), (576, 0), (640, 70), (544, 64)])
def test_latent_attention_tile_kernel(R, window):
    """The tensor-core prompt kernel against float64, on a ragged batch whose entries start at different positions of
    different cache rows (1 to 70 tokens, so tiles are full, partial and single), with a dominant key placed exactly at the
    window's edge of one query: inside for one entry, one position too far for another."""
    from mlx_parallm_b200 import ops
    H, scale = 3, 0.4
    starts, counts, rows = [0, 3, 100, 0, 20], [1, 5, 16, 17, 70], [4, 0, 2, 1, 3]
    g = torch.Generator().manual_seed(R + window)
    Tcap = 192
    cache = (torch.randn(5, Tcap, R, generator=g) * 0.3).to(torch.bfloat16)
    M = sum(counts)
    q = torch.randn(M, H, R, generator=g) * 0.3
    cu = [0]
    for n in counts:
        cu.append(cu[-1] + n)
    d = torch.randn(R, generator=g)
    d = d / d.norm()
    if window > 1:
        # entry 2 (row 2): query at position 110, key window - 1 back (seen); entry 4 (row 3): query at position 80, key window back
        cache[2, 110 - (window - 1)] = (5.0 * d).to(torch.bfloat16)
        q[cu[2] + 10, 0] = 5.0 * d
        cache[3, 80 - window] = (5.0 * d).to(torch.bfloat16)
        q[cu[4] + 60, 0] = 5.0 * d
    i32 = dict(dtype=torch.int32, device="cuda")
    t_row = torch.tensor([r for r, n in zip(rows, counts) for _ in range(n)], **i32)
    t_pos = torch.tensor([s + i for s, n in zip(starts, counts) for i in range(n)], **i32)
    cd, qd = cache.cuda(), q.reshape(M, H * R).cuda().contiguous()
    tiles = torch.empty(M, H * R, dtype=torch.bfloat16, device="cuda")
    ops.latent_attn(qd, cd, t_row, t_pos, tiles, H, R, window, scale, cu=torch.tensor(cu, **i32), rows=torch.tensor(rows, **i32),
                    nb=5, max_n=70)
    from mlx_parallm_b200 import _lib
    for buffers in (1, 2):                 # one chunk buffer, or the next chunk in flight during the products: the same numbers
        other = torch.empty_like(tiles)
        _lib.lib().b200p_latent_attn_set_buffers(buffers)
        try:
            ops.latent_attn(qd, cd, t_row, t_pos, other, H, R, window, scale, cu=torch.tensor(cu, **i32), rows=torch.tensor(rows, **i32),
                            nb=5, max_n=70)
        finally:
            _lib.lib().b200p_latent_attn_set_buffers(0)
        assert torch.equal(other, tiles), buffers
    single = torch.empty_like(tiles)
    ops.latent_attn(qd, cd, t_row, t_pos, single, H, R, window, scale)
    want = torch.zeros(M, H, R, dtype=torch.float64)
    c64 = cache.double()
    for t in range(M):
        r, p = int(t_row[t]), int(t_pos[t])
        lo = 0 if window <= 0 else max(0, p - window + 1)
        pr = torch.softmax(torch.einsum("hr,jr->hj", q[t].double(), c64[r, lo:p + 1]) * scale, -1)
        want[t] = pr @ c64[r, lo:p + 1]
    want = want.reshape(M, H * R)
    assert (single.double().cpu() - want).abs().max() < 0.02
    assert (tiles.double().cpu() - want).abs().max() < 0.04
    if window > 1:
        seen, unseen, hot = want[cu[2] + 10, :R], want[cu[4] + 60, :R], 5.0 * d.double()
        assert (seen - hot).norm() < 0.2 * hot.norm() and (unseen - hot).norm() > 0.6 * hot.norm()


@pytest.mark.parametrize("splits", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("H,R,window", [(20, 64, 33), (8, 128, 0), (16, 32, 64), (3, 512, 130), (9, 576, 0), (32, 640, 100)])
def test_latent_attention_decode_tiles_over_heads(H, R, window, splits):
    """A decode step (one token per entry) tiles over the heads of each token: against float64 and against the per-token
    kernel, entries at different positions (also position 0), a head count that leaves the last tile partial.  With the keys
    of a tile shared between the CTAs of a cluster (2, 4, 8; 0 = the launch's own choice), some of which get no key at all
    at the early positions."""
    from mlx_parallm_b200 import _lib, ops
    L = _lib.lib()
    g = torch.Generator().manual_seed(H + R)
    pos, rows = [0, 1, 63, 64, 150], [1, 4, 0, 3, 2]
    cache = (torch.randn(5, 160, R, generator=g) * 0.3).to(torch.bfloat16)
    q = torch.randn(5, H, R, generator=g) * 0.3
    i32 = dict(dtype=torch.int32, device="cuda")
    t_row, t_pos = torch.tensor(rows, **i32), torch.tensor(pos, **i32)
    cd, qd = cache.cuda(), q.reshape(5, H * R).cuda().contiguous()
    tiles, single = torch.empty(5, H * R, dtype=torch.bfloat16, device="cuda"), torch.empty(5, H * R, dtype=torch.bfloat16, device="cuda")
    L.b200p_latent_attn_set_splits(splits)
    try:
        ops.latent_attn(qd, cd, t_row, t_pos, tiles, H, R, window, 0.3, cu=torch.arange(6, **i32), rows=t_row, nb=5, max_n=1)
    finally:
        L.b200p_latent_attn_set_splits(0)
    ops.latent_attn(qd, cd, t_row, t_pos, single, H, R, window, 0.3)
    c64 = cache.double()
    for t in range(5):
        lo = 0 if window <= 0 else max(0, pos[t] - window + 1)
        keys = c64[rows[t], lo:pos[t] + 1]
        want = (torch.softmax(q[t].double() @ keys.T * 0.3, -1) @ keys).reshape(-1)
        assert (single[t].double().cpu() - want).abs().max() < 0.02 and (tiles[t].double().cpu() - want).abs().max() < 0.04


def test_latent_attention_tiles_sharing_keys_between_heads():
    """One, two or four 16-row tiles per CTA read the same staged keys: identical numbers, also when the head count leaves
    groups of the last CTA without a head."""
    from mlx_parallm_b200 import _lib, ops
    L = _lib.lib()
    g = torch.Generator().manual_seed(3)
    H, R, window, nb, T = 5, 128, 21, 2, 37
    cache = (torch.randn(nb, 64, R, generator=g) * 0.3).to(torch.bfloat16).cuda()
    q = (torch.randn(nb * T, H * R, generator=g) * 0.3).cuda()
    i32 = dict(dtype=torch.int32, device="cuda")
    t_row = torch.arange(nb, **i32).repeat_interleave(T)
    t_pos = torch.arange(T, **i32).repeat(nb) + 9
    outs = []
    try:
        for groups in (1, 2, 4, 0):
            L.b200p_latent_attn_set_groups(groups)
            out = torch.empty(nb * T, H * R, dtype=torch.bfloat16, device="cuda")
            ops.latent_attn(q, cache, t_row, t_pos, out, H, R, window, 0.2, cu=torch.tensor([0, T, 2 * T], **i32), rows=torch.arange(nb, **i32),
                            nb=nb, max_n=T)
            outs.append(out)
    finally:
        L.b200p_latent_attn_set_groups(0)
    single = torch.empty_like(outs[0])
    ops.latent_attn(q, cache, t_row, t_pos, single, H, R, window, 0.2)
    assert all(torch.equal(o, outs[0]) for o in outs[1:])
    assert (outs[0].float() - single.float()).abs().max() < 0.03


def test_latent_attention_rank_above_the_tile_kernel():
    """Rank 672 runs on the per-token kernel (the tile kernel stops at 640)."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(8)
    H, R, window, T = 2, 672, 6, 19
    cache = (torch.randn(1, 32, R, generator=g) * 0.2).to(torch.bfloat16)
    q = torch.randn(T, H, R, generator=g) * 0.2
    i32 = dict(dtype=torch.int32, device="cuda")
    t_row, t_pos = torch.zeros(T, **i32), torch.arange(T, **i32) + 4
    out = torch.empty(T, H * R, dtype=torch.bfloat16, device="cuda")
    ops.latent_attn(q.reshape(T, H * R).cuda().contiguous(), cache.cuda(), t_row, t_pos, out, H, R, window, 0.25,
                    cu=torch.tensor([0, T], **i32), rows=torch.zeros(1, **i32), nb=1, max_n=T)
    c64 = cache[0].double()
    for t in range(T):
        p = t + 4
        keys = c64[max(0, p - window + 1):p + 1]
        want = (torch.softmax(q[t].double() @ keys.T * 0.25, -1) @ keys).reshape(-1)
        assert (out[t].double().cpu() - want).abs().max() < 0.02


@pytest.mark.parametrize("dk,dv,H,KH", [(16, 100, 2, 1), (128, 64, 4, 2), (200, 24, 2, 2), (300, 70, 3, 1)])
def test_delta_scan_key_and_value_sizes(dk, dv, H, KH):
    """The recurrence kernel alone against a float64 loop: key sizes that put 4, 8 and 16 lanes on a column, value sizes that
    leave column slots empty or need several thread blocks; one entry continues a stored state, one starts from nothing."""
    import ctypes as C
    from mlx_parallm_b200 import _lib
    L = _lib.lib()
    g = torch.Generator().manual_seed(dk + dv)
    counts, rows, lengths = [11, 3], [2, 0], [5, 0]
    M = sum(counts)
    qn = torch.randn(M, KH, dk, generator=g) / dk
    kn = torch.nn.functional.normalize(torch.randn(M, KH, dk, generator=g), dim=-1)
    v = torch.randn(M, H, dv, generator=g)
    beta, decay = torch.rand(M, H, generator=g), 0.5 + 0.5 * torch.rand(M, H, generator=g)
    state0 = torch.randn(3, H, dk, dv, generator=g) * 0.3
    want_o, want_s = torch.zeros(M, H, dv, dtype=torch.float64), state0.double().clone()
    t = 0
    for n, r, ln in zip(counts, rows, lengths):
        for h in range(H):
            S = want_s[r, h].clone() if ln > 0 else torch.zeros(dk, dv, dtype=torch.float64)
            for i in range(t, t + n):
                k, q_ = kn[i, h // (H // KH)].double(), qn[i, h // (H // KH)].double()
                S = S * decay[i, h].double()
                u = beta[i, h].double() * (v[i, h].double() - S.T @ k)
                S = S + torch.outer(k, u)
                want_o[i, h] = S.T @ q_
            want_s[r, h] = S
        t += n
    i32 = dict(dtype=torch.int32, device="cuda")
    dev = [x.contiguous().cuda() for x in (qn.reshape(M, -1), kn.reshape(M, -1), v.reshape(M, -1), beta, decay, state0)]
    cu, rw, ln = torch.tensor([0, counts[0], M], **i32), torch.tensor(rows, **i32), torch.tensor([0, 0, 5], **i32)
    o = torch.empty(M, H * dv, device="cuda")
    p = lambda x: C.c_void_p(x.data_ptr())
    assert L.b200p_delta_scan(p(dev[0]), p(dev[1]), p(dev[2]), p(dev[3]), p(dev[4]), p(dev[5]), p(cu), p(rw), p(ln), p(o), 2, H, KH, dk, dv,
                              0, None) == 0
    assert (o.double().cpu().view(M, H, dv) - want_o).abs().max() < 1e-4
    assert (dev[5].double().cpu()[[0, 2]] - want_s[[0, 2]]).abs().max() < 1e-4
    assert torch.equal(dev[5].cpu()[1], state0[1])               # a row that no entry names is not touched

"""Thin torch-tensor wrappers over the C-ABI (include/b200p.h).

torch is plumbing here: device memory, the current stream, CUDA-graph capture.  Every function
launches hand-written sm_100a kernels from libb200parallm.so on ``torch.cuda.current_stream()``;
none of them has a CPU or eager-PyTorch fallback -- a CPU tensor raises.
"""
from __future__ import annotations

from typing import Optional

import os

import torch

from . import _lib
from ._lib import (DQ_F32_MULADD, EPI_ADD_RESIDUAL, EPI_SILU_MUL, EPI_STORE, EPI_STORE_F32, check, lib)

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise TypeError(f"unsupported storage dtype {dt}") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.B200PError("b200p ops need CUDA tensors: there is no CPU fallback")


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


# ---- launch accounting / optional per-kernel CUDA-event timing (bench.py, profiles/) ----------------
LAUNCHES = 0            # b200p kernel-launching calls issued from Python (captured ones count once)
PROFILER = None         # set to a dict name -> list[(start_event, end_event)] to time each call


def _call(name: str, rc_fn):
    """Run one C-ABI launch; count it; bracket it with events when a profiler is attached."""
    global LAUNCHES
    LAUNCHES += 1
    if PROFILER is None:
        check(rc_fn(), name if isinstance(name, str) else name[0])
        return
    key = name if isinstance(name, str) else f"{name[0]}[N={name[1]},K={name[2]}" + (f",heads={name[3]}]" if len(name) > 3 and name[3] > 1 else "]")
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    check(rc_fn(), key)
    e.record()
    PROFILER.setdefault(key, []).append((s, e))


# ------------------------------------------------------------------------------------------------
def dequantize(w, scales, biases, group_size=64, bits=4, mode=DQ_F32_MULADD, out=None):
    """mx.dequantize: w int32/uint32 [N, K*bits/32] -> [N, K] in scales.dtype."""
    _dev(w, scales, biases)
    N = w.shape[0]
    K = w.shape[1] * 32 // bits
    if out is None:
        out = torch.empty((N, K), dtype=scales.dtype, device=w.device)
    _call("b200p_dequantize", lambda: lib().b200p_dequantize(_p(w), _p(scales), _p(biases), _p(out), N, K, group_size, bits,
                                 dtype_code(scales.dtype), mode, _stream()))
    return out


def quantize(w, group_size=64, bits=4):
    """mx.quantize: w [N, K] (float32 / float16 / bfloat16) -> (wq int32 [N, K*bits/32], scales, biases [N, K/gs])."""
    _dev(w)
    assert w.dim() == 2 and w.is_contiguous()
    N, K = w.shape
    wq = torch.empty((N, K * bits // 32), dtype=torch.int32, device=w.device)
    s = torch.empty((N, K // group_size), dtype=w.dtype, device=w.device)
    b = torch.empty_like(s)
    _call("b200p_quantize", lambda: lib().b200p_quantize(_p(w), _p(wq), _p(s), _p(b), N, K, group_size, bits, dtype_code(w.dtype),
                                                         _stream()))
    return wq, s, b


def embed(ids, w, scales, biases, group_size=64, bits=4, mode=DQ_F32_MULADD, out=None, out_f32=True):
    """QuantizedEmbedding.__call__: ids int32 [M] -> [M, K] (float32 carrier of dtype-rounded values)."""
    _dev(ids, w, scales, biases)
    assert ids.dtype == torch.int32 and ids.is_contiguous()
    M = ids.numel()
    V = w.shape[0]
    K = w.shape[1] * 32 // bits
    if out is None:
        out = torch.empty((M, K), dtype=torch.float32 if out_f32 else scales.dtype, device=w.device)
    _call("b200p_embed", lambda: lib().b200p_embed(_p(ids), _p(w), _p(scales), _p(biases), _p(out), M, V, K, group_size, bits,
                            dtype_code(scales.dtype), mode, 1 if out_f32 else 0, _stream()))
    return out


def qmm_workspace_bytes(M, N, K) -> int:
    return int(lib().b200p_qmm_workspace_bytes(M, N, K))


_SMALLSCALE_OK = os.environ.get("B200P_NO_SMALLSCALE", "0") != "1"      # A/B switch for the subnormal-operand dequant


def qmm(x, w, scales, biases, group_size=64, bits=4, epilogue=EPI_STORE, out=None, workspace=None,
        x_perm=False, y_perm=False, small_scale=False):
    """quantized_matmul(x, w, scales, biases, transpose=True) with a fused epilogue.

    ``x_perm`` / ``y_perm``: x arrives / the 16-bit y leaves in the PERM8 column order (include/b200p.h).
    ``small_scale``: the caller has checked max|scales| < 0.0625 (B200P_W_SMALLSCALE).

    x [M, K] (row stride = x.stride(0)); out per epilogue:
      EPI_STORE -> [M, N] x.dtype; EPI_STORE_F32 -> [M, N] float32; EPI_ADD_RESIDUAL -> out (float32
      [M, N], required) += result; EPI_SILU_MUL -> [M, N/2] x.dtype."""
    _dev(x, w, scales, biases, out)
    assert x.dim() == 2 and x.stride(1) == 1
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] * 32 // bits == K, (w.shape, K, bits)
    if out is None:
        if epilogue == EPI_STORE:
            out = torch.empty((M, N), dtype=x.dtype, device=x.device)
        elif epilogue == EPI_STORE_F32:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        elif epilogue == EPI_SILU_MUL:
            out = torch.empty((M, N // 2), dtype=x.dtype, device=x.device)
        else:
            raise ValueError("EPI_ADD_RESIDUAL needs the residual tensor as `out`")
    epi_flags = (epilogue | (_lib.X_PERM8 if x_perm else 0) | (_lib.Y_PERM8 if y_perm else 0)
                 | (_lib.W_SMALLSCALE if (small_scale and _SMALLSCALE_OK) else 0))
    ws_ptr, ws_bytes = (0, 0) if workspace is None else (workspace.data_ptr(), workspace.numel() * workspace.element_size())
    _call(("b200p_qmm", N, K), lambda: lib().b200p_qmm(_p(x), _p(w), _p(scales), _p(biases), _p(out), M, N, K, x.stride(0), out.stride(0),
                          group_size, bits, dtype_code(x.dtype), epi_flags, ws_ptr, ws_bytes, _stream()))
    return out


def rmsnorm(x, w, eps, out=None, out_perm=False):
    """mx.fast.rms_norm on the float32 residual stream -> w.dtype (``out_perm``: PERM8 column order for a 4-bit qmm)."""
    _dev(x, w, out)
    assert x.dtype == torch.float32 and x.is_contiguous()
    M, H = x.shape
    if out is None:
        out = torch.empty((M, H), dtype=w.dtype, device=x.device)
    _call("b200p_rmsnorm", lambda: lib().b200p_rmsnorm(_p(x), _p(w), _p(out), M, H, float(eps), dtype_code(w.dtype),
                                                      _lib.OUT_PERM8 if out_perm else 0, _stream()))
    return out


def rope_kv_append(qkv, q_out, kcache, vcache, lengths, B, L, Hq, Hkv, D, rope_base, rope_scale=1.0,
                   q_norm_w=None, k_norm_w=None, norm_eps=1e-6):
    _dev(qkv, q_out, kcache, vcache, lengths)
    assert lengths.dtype == torch.int32
    Tcap = kcache.shape[2]
    _call("b200p_rope_kv_append", lambda: lib().b200p_rope_kv_append(_p(qkv), _p(q_out), _p(kcache), _p(vcache), _p(lengths), _p(q_norm_w),
                                     _p(k_norm_w), B, L, Hq, Hkv, D, Tcap, float(rope_base), float(rope_scale),
                                     float(norm_eps), dtype_code(kcache.dtype), 1 if qkv.dtype == torch.float32 and kcache.dtype != torch.float32 else 0,
                                     _stream()))


def silu_mul(gu, out, out_perm=False):
    """silu(gate) * up from the fp32 accumulation buffer gu [M, 2*I] of the fused gate|up projection; re-zeroes gu."""
    _dev(gu, out)
    assert gu.dtype == torch.float32 and gu.stride(1) == 1 and out.stride(1) == 1
    M, I = out.shape
    _call("b200p_silu_mul", lambda: lib().b200p_silu_mul(_p(gu), _p(out), M, I, gu.stride(0), out.stride(0), dtype_code(out.dtype),
                                                         _lib.OUT_PERM8 if out_perm else 0, _stream()))
    return out


def lora_add(x, At, Bt, y, col0: int, scale: float):
    """y[:, col0:col0+N] += scale * (x @ lora_a) @ lora_b with At = lora_a^T [16, K], Bt = lora_b^T [N, 16] (rank padded)."""
    _dev(x, At, Bt, y)
    M, K = x.shape
    N = Bt.shape[0]
    assert At.shape == (16, K) and Bt.shape[1] == 16 and At.is_contiguous() and Bt.is_contiguous() and x.stride(1) == 1
    _call("b200p_lora_add", lambda: lib().b200p_lora_add(_p(x), _p(At), _p(Bt), _p(y), M, N, K, x.stride(0), y.stride(0), int(col0),
                                                         float(scale), dtype_code(x.dtype), 1 if y.dtype == torch.float32 else 0,
                                                         _stream()))
    return y


def advance_lengths(lengths, delta: int):
    _dev(lengths)
    _call("b200p_advance_lengths", lambda: lib().b200p_advance_lengths(_p(lengths), lengths.numel(), int(delta), _stream()))


def kv_overflow_count(reset: bool = False) -> int:
    """Rows b200p_rope_kv_append had to drop since the last reset because their position reached the cache capacity
    (include/b200p.h).  Synchronises the current stream: call it at generation boundaries, never under graph capture."""
    import ctypes as C
    n = C.c_uint(0)
    _lib.check(lib().b200p_kv_overflow_count(C.byref(n), 1 if reset else 0, _stream()), "b200p_kv_overflow_count")
    return int(n.value)


def attn_workspace_bytes(B, L, Hq, D) -> int:
    return int(lib().b200p_attn_workspace_bytes(B, L, Hq, D))


def attn(q, kcache, vcache, lengths, out, B, L, Hq, Hkv, D, scale, workspace=None, out_perm=False):
    _dev(q, kcache, vcache, lengths, out)
    Tcap = kcache.shape[2]
    ws_ptr, ws_bytes = (0, 0) if workspace is None else (workspace.data_ptr(), workspace.numel() * workspace.element_size())
    _call("b200p_attn", lambda: lib().b200p_attn(_p(q), _p(kcache), _p(vcache), _p(lengths), _p(out), B, L, Hq, Hkv, D, Tcap, float(scale),
                           dtype_code(q.dtype), _lib.OUT_PERM8 if out_perm else 0, ws_ptr, ws_bytes, _stream()))
    return out


def argmax(logits, out=None, probs_out=None):
    """mx.argmax(logits, -1): float32 [B, V] -> int32 [B]."""
    _dev(logits, out, probs_out)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    B, V = logits.shape
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    _call("b200p_argmax", lambda: lib().b200p_argmax(_p(logits), _p(out), _p(probs_out), B, V, logits.stride(0), _stream()))
    return out


def argmax_partial(logits, vocab_offset: int, rec_out):
    """Vocab-shard reduction for the tensor-parallel greedy head: float32 [B, V_local] -> records [B, 4]."""
    _dev(logits, rec_out)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    B, V = logits.shape
    _call("b200p_argmax_partial", lambda: lib().b200p_argmax_partial(_p(logits), _p(rec_out), B, V, logits.stride(0),
                                                                     int(vocab_offset), _stream()))
    return rec_out


def argmax_merge(recs, out, probs_out=None):
    """records [W, B, 4] (all-gathered) -> tokens int32 [B] (+ softmax prob of the token)."""
    _dev(recs, out, probs_out)
    W, B = recs.shape[0], recs.shape[1]
    _call("b200p_argmax_merge", lambda: lib().b200p_argmax_merge(_p(recs), _p(out), _p(probs_out), W, B, _stream()))
    return out


def sample_top_p(logits, temperature, top_p, seed, offset, out=None, probs_out=None):
    _dev(logits, out, probs_out)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    B, V = logits.shape
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    _call("b200p_sample_top_p", lambda: lib().b200p_sample_top_p(_p(logits), _p(out), _p(probs_out), B, V, logits.stride(0), float(temperature),
                                   float(top_p), int(seed) & (2**64 - 1), int(offset) & (2**64 - 1), _stream()))
    return out


# ---- dense linear layers, ragged batches, gated delta rule, latent attention ------------------------------------------
def gemm(x, w, epilogue=_lib.GEMM_STORE, out=None, limit=0.0, batch=1, strides=(0, 0, 0), M=None, N=None, K=None,
         ldx=None, ldw=None, ldy=None):
    """y = x . w^T with fp32 accumulation (b200p_gemm).  Plain call: x [M, K], w [N, K] of one dtype.  Batched call (one
    weight block per head): pass M, N, K, the row strides and ``strides`` = element strides of x, w, y between products."""
    _dev(x, w, out)
    assert x.dtype == w.dtype and x.stride(-1) == 1 and w.stride(-1) == 1
    if M is None:
        M, K = x.shape
        N = w.shape[0]
        assert w.shape[1] == K, (tuple(x.shape), tuple(w.shape))
        ldx, ldw = x.stride(0), w.stride(0)
    if out is None:
        n_out = N // 2 if _lib.gemm_is_gated(epilogue) else N
        out = torch.empty((M, n_out * batch), dtype=torch.float32 if epilogue == _lib.GEMM_STORE_F32 else x.dtype, device=x.device)
    if ldy is None:
        ldy = out.stride(0)
    want = torch.float32 if epilogue == _lib.GEMM_STORE_F32 else x.dtype
    assert out.dtype == want and out.stride(-1) == 1, (out.dtype, want)
    _call(("b200p_gemm", N, K, batch), lambda: lib().b200p_gemm(_p(x), _p(w), _p(out), M, N, K, ldx, ldw, ldy, batch, strides[0], strides[1],
                                                        strides[2], dtype_code(x.dtype), epilogue, float(limit), _stream()))
    return out


def ragged_plan(cu, rows, lengths, t_row, t_pos, t_off, nb: int, M: int):
    _dev(cu, rows, lengths, t_row, t_pos, t_off)
    _call("b200p_ragged_plan", lambda: lib().b200p_ragged_plan(_p(cu), _p(rows), _p(lengths), _p(t_row), _p(t_pos), _p(t_off), nb, M,
                                                              _stream()))


def ragged_advance(lengths, last_token, ids, cu, rows, nb: int):
    _dev(lengths, last_token, ids, cu, rows)
    _call("b200p_ragged_advance", lambda: lib().b200p_ragged_advance(_p(lengths), _p(last_token), _p(ids), _p(cu), _p(rows), nb, _stream()))


def embed_hashed(ids, t_row, t_pos, t_off, last_token, embed, bigram, h, scale, buckets=0, mul_prev=0, mul_cur=0):
    _dev(ids, t_row, t_pos, t_off, last_token, embed, bigram, h)
    M = ids.numel()
    V, W = embed.shape
    assert h.dtype == torch.float32 and h.shape[1] == W and (bigram is None or bigram.shape == (buckets + 1, W))
    _call("b200p_embed_hashed", lambda: lib().b200p_embed_hashed(_p(ids), _p(t_row), _p(t_pos), _p(t_off), _p(last_token), _p(embed),
                                                                _p(bigram), _p(h), M, W, V, float(scale), int(buckets), int(mul_prev),
                                                                int(mul_cur), dtype_code(embed.dtype), _stream()))
    return h


def norm_add_norm(h, eps, dtype, y=None, w_post=None, w_next=None, x_out=None, raw_out=None):
    """h += rms_norm(y) * w_post; raw_out = h; x_out = rms_norm(h) * w_next (each part optional; b200p_norm_add_norm)."""
    _dev(h, y, w_post, w_next, x_out, raw_out)
    M, W = h.shape
    assert h.dtype == torch.float32 and h.is_contiguous()
    for t in (y, w_post, w_next):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    for t in (x_out, raw_out):
        assert t is None or (t.dtype == dtype and t.is_contiguous())
    _call("b200p_norm_add_norm", lambda: lib().b200p_norm_add_norm(_p(y), _p(w_post), _p(h), _p(w_next), _p(x_out), _p(raw_out), M, W,
                                                                  float(eps), dtype_code(dtype), _stream()))


def token_gate(gate, table, ids, out, col0: int):
    _dev(gate, table, ids, out)
    M, d = gate.shape
    assert gate.dtype == torch.float32 and gate.is_contiguous() and out.is_contiguous() and out.dtype == table.dtype
    _call("b200p_token_gate", lambda: lib().b200p_token_gate(_p(gate), _p(table), _p(ids), _p(out), M, d, table.stride(0), int(col0),
                                                            dtype_code(table.dtype), _stream()))
    return out


def delta_prep(proj, col_b, a, conv_w, conv_state, A_log, dt_bias, t_row, t_pos, t_off, qn, kn, v, beta, decay, H, KH, dk, dv, taps):
    """``a``: the decay's step input, fp32 [M, H] (one decay per head; may be a column slice of ``proj``) or [M, H * dk] (one
    per key channel); ``decay`` takes the same shape."""
    _dev(proj, a, conv_w, conv_state, A_log, dt_bias, t_row, t_pos, t_off, qn, kn, v, beta, decay)
    M = proj.shape[0]
    per = a.shape[1] // H
    assert a.dtype == torch.float32 and a.stride(1) == 1 and a.shape[1] == H * per and decay.shape[1] == H * per and decay.is_contiguous()
    _call("b200p_delta_prep", lambda: lib().b200p_delta_prep(_p(proj), proj.stride(0), int(col_b), _p(a), a.stride(0), per, _p(conv_w),
                                                            _p(conv_state), _p(A_log), _p(dt_bias), _p(t_row), _p(t_pos), _p(t_off), _p(qn),
                                                            _p(kn), _p(v), _p(beta), _p(decay), M, H, KH, dk, dv, taps, _stream()))


def delta_conv_commit(proj, conv_state, cu, rows, nb: int, C: int, taps: int):
    _dev(proj, conv_state, cu, rows)
    _call("b200p_delta_conv_commit", lambda: lib().b200p_delta_conv_commit(_p(proj), proj.stride(0), _p(conv_state), _p(cu), _p(rows), nb,
                                                                          C, taps, _stream()))


def delta_scan(qn, kn, v, beta, decay, state, cu, rows, lengths, o, nb, H, KH, dk, dv, mode=_lib.SCAN_DELTA):
    """The recurrence over every entry's tokens; ``mode`` one of _lib.SCAN_* (decay per head, per head and key channel, or
    the plain decayed accumulation without the delta correction)."""
    _dev(qn, kn, v, beta, decay, state, cu, rows, lengths, o)
    assert state.dtype == torch.float32 and state.is_contiguous()
    _call("b200p_delta_scan", lambda: lib().b200p_delta_scan(_p(qn), _p(kn), _p(v), _p(beta), _p(decay), _p(state), _p(cu), _p(rows),
                                                            _p(lengths), _p(o), nb, H, KH, dk, dv, int(mode), _stream()))


def delta_out(o, gate, norm_w, out, H, dv, eps, gate_act=_lib.GATE_SILU, out_scale=1.0):
    """out = out_scale * rms_norm(o per group of dv) * norm_w * act(gate); ``gate`` fp32 [M, H * dv] (may be a column slice),
    ``out`` [M, >= H * dv] (may be a column slice of a wider buffer)."""
    _dev(o, gate, norm_w, out)
    M = o.shape[0]
    assert gate.dtype == torch.float32 and gate.stride(1) == 1 and out.stride(1) == 1 and o.is_contiguous()
    _call("b200p_delta_out", lambda: lib().b200p_delta_out(_p(o), _p(gate), gate.stride(0), _p(norm_w), _p(out), out.stride(0), M, H, dv,
                                                          float(eps), int(gate_act), float(out_scale), dtype_code(out.dtype), _stream()))


def linear_attn_prep(proj, head_decay, q, k, v, decay, H, dk, dv):
    """q, k, v = silu of the columns [q | k | v] of ``proj``; decay[t, h] = head_decay[h] (inputs of SCAN_ACCUMULATE)."""
    _dev(proj, head_decay, q, k, v, decay)
    M = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and head_decay.dtype == torch.float32
    _call("b200p_linear_attn_prep", lambda: lib().b200p_linear_attn_prep(_p(proj), proj.stride(0), _p(head_decay), _p(q), _p(k), _p(v),
                                                                        _p(decay), M, H, dk, dv, _stream()))


def gemm_grouped(x, w, seg, max_rows: int, epilogue=_lib.GEMM_STORE, out=None, limit=0.0):
    """Rows [seg[z], seg[z+1]) of x times the z-th block of w [groups, N, K] (b200p_gemm_grouped); ``seg`` int32 on the device."""
    _dev(x, w, seg, out)
    groups, N, K = w.shape
    assert x.dtype == w.dtype and x.stride(-1) == 1 and w.is_contiguous() and x.shape[1] == K and seg.dtype == torch.int32
    glu = _lib.gemm_is_gated(epilogue)
    want = torch.float32 if epilogue == _lib.GEMM_STORE_F32 else x.dtype
    if out is None:
        out = torch.empty((x.shape[0], N // 2 if glu else N), dtype=want, device=x.device)
    assert out.dtype == want and out.stride(-1) == 1
    _call(("b200p_gemm_grouped", N, K, groups), lambda: lib().b200p_gemm_grouped(
        _p(x), _p(w), _p(out), _p(seg), x.shape[0], int(max_rows), N, K, x.stride(0), K, out.stride(0), groups, N * K, dtype_code(x.dtype),
        epilogue,
        float(limit), _stream()))
    return out


def residual_add_norm(h, eps, dtype, y1=None, c1=1.0, y2=None, c2=1.0, w_next=None, x_out=None, raw_out=None):
    """h += c1 y1 + c2 y2; raw_out = h (may be a column slice); x_out = rms_norm(h) * w_next (b200p_residual_add_norm)."""
    _dev(h, y1, y2, w_next, x_out, raw_out)
    M, W = h.shape
    assert h.dtype == torch.float32 and h.is_contiguous()
    for t in (y1, y2, w_next):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    assert x_out is None or (x_out.dtype == dtype and x_out.is_contiguous())
    assert raw_out is None or (raw_out.dtype == dtype and raw_out.stride(1) == 1)
    _call("b200p_residual_add_norm", lambda: lib().b200p_residual_add_norm(
        _p(h), _p(y1), float(c1), _p(y2), float(c2), _p(w_next), _p(x_out), _p(raw_out), 0 if raw_out is None else raw_out.stride(0), M, W,
        float(eps), dtype_code(dtype), _stream()))


def cast_columns(src, dst):
    """dst (16-bit or fp32, may be a column slice) = src (fp32, may be a column slice)."""
    _dev(src, dst)
    M, n = src.shape
    assert src.dtype == torch.float32 and src.stride(1) == 1 and dst.stride(1) == 1 and dst.shape == src.shape
    _call("b200p_cast_columns", lambda: lib().b200p_cast_columns(_p(src), src.stride(0), _p(dst), dst.stride(0), M, n,
                                                                dtype_code(dst.dtype), _stream()))


def sink_attn_prep(proj, col_q, col_k, col_v, wq, wk, eps, scale, temp_coef, temp_every, q_out, kcache, vcache, t_row, t_pos, H, G, dk, dv):
    """Queries (normed, scaled, temperature applied) to ``q_out`` fp32; normed keys and the values into the caches
    [rows, G, Tcap, dk] / [rows, G, Tcap, dv] at every token's (row, position)."""
    _dev(proj, wq, wk, q_out, kcache, vcache, t_row, t_pos)
    M = proj.shape[0]
    assert proj.dtype == torch.float32 and kcache.is_contiguous() and vcache.is_contiguous() and kcache.dtype == vcache.dtype
    assert kcache.shape[1:] == (G, kcache.shape[2], dk) and vcache.shape[1:] == (G, kcache.shape[2], dv)
    _call("b200p_sink_attn_prep", lambda: lib().b200p_sink_attn_prep(
        _p(proj), proj.stride(0), int(col_q), int(col_k), int(col_v), _p(wq), _p(wk), float(eps), float(scale), float(temp_coef),
        float(temp_every), _p(q_out), _p(kcache), _p(vcache), kcache.shape[2], _p(t_row), _p(t_pos), M, H, G, dk, dv,
        dtype_code(kcache.dtype), _stream()))


def sink_attn_workspace_floats(nb: int, H: int, dv: int) -> int:
    return lib().b200p_sink_attn_workspace_bytes(nb, H, dv) // 4


def sink_attn(q, kcache, vcache, t_row, t_pos, sink, slope_log2, out, H, G, dk, dv, out_scale=1.0, cu=None, rows=None, nb=0, max_n=1,
              workspace=None):
    """Causal attention with a distance bias and a sink over the caches; ``out`` [M, >= H * dv] in the caches' dtype.
    ``workspace`` (fp32): room for the partial sums of a decode step on the tile kernel."""
    _dev(q, kcache, vcache, t_row, t_pos, sink, out, cu, rows)
    M = q.shape[0]
    assert q.dtype == torch.float32 and q.is_contiguous() and out.stride(1) == 1 and out.dtype == kcache.dtype
    _call("b200p_sink_attn", lambda: lib().b200p_sink_attn(
        _p(q), _p(kcache), _p(vcache), kcache.shape[2], _p(t_row), _p(t_pos), _p(cu), _p(rows), int(nb), int(max_n), _p(sink),
        float(slope_log2), _p(out), out.stride(0), float(out_scale), M, H, G, dk, dv, dtype_code(kcache.dtype), _p(workspace),
        0 if workspace is None else workspace.numel() * 4, _stream()))
    return out


def moe_route(logits, bias, ids, wts, seg, slot_of, token_of, top: int):
    _dev(logits, bias, ids, wts, seg, slot_of, token_of)
    M, E = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _call("b200p_moe_route", lambda: lib().b200p_moe_route(_p(logits), logits.stride(0), _p(bias), _p(ids), _p(wts), _p(seg), _p(slot_of),
                                                          _p(token_of), M, E, int(top), _stream()))


def moe_gather(x, token_of, xs):
    _dev(x, token_of, xs)
    assert x.is_contiguous() and xs.is_contiguous() and x.dtype == xs.dtype and x.shape[1] == xs.shape[1]
    _call("b200p_moe_gather", lambda: lib().b200p_moe_gather(_p(x), _p(token_of), _p(xs), xs.shape[0], x.shape[1], dtype_code(x.dtype),
                                                            _stream()))


def moe_route_sigmoid(logits, correction, ids, wts, seg, slot_of, token_of, top: int, groups: int = 1, keep: int = 1, scale: float = 1.0,
                      experts: Optional[int] = None):
    """Routing by sigmoid scores inside the ``keep`` best of ``groups`` expert groups; ``logits`` may hold more columns than
    ``experts`` (say a shared expert's gate beside the router's)."""
    _dev(logits, correction, ids, wts, seg, slot_of, token_of)
    M = logits.shape[0]
    E = logits.shape[1] if experts is None else int(experts)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _call("b200p_moe_route_sigmoid", lambda: lib().b200p_moe_route_sigmoid(_p(logits), logits.stride(0), _p(correction), _p(ids), _p(wts),
                                                                          _p(seg), _p(slot_of), _p(token_of), M, E, int(top), int(groups),
                                                                          int(keep), float(scale), _stream()))


def moe_combine(ye, slot_of, wts, shared_y, y, top: int, shared_gate=None):
    """``shared_gate``: fp32 column (one pre-activation per token, any row stride) whose sigmoid multiplies ``shared_y``."""
    _dev(ye, slot_of, wts, shared_y, y, shared_gate)
    M, W = y.shape
    assert ye.dtype == torch.float32 and ye.is_contiguous() and y.is_contiguous() and (shared_y is None or shared_y.is_contiguous())
    assert shared_gate is None or (shared_gate.dtype == torch.float32 and shared_gate.shape[0] == M)
    _call("b200p_moe_combine", lambda: lib().b200p_moe_combine(_p(ye), _p(slot_of), _p(wts), _p(shared_y), _p(shared_gate),
                                                              0 if shared_gate is None else shared_gate.stride(0), _p(y), M, W, int(top),
                                                              _stream()))


def ssm_prep(proj, col_x, col_dt, conv_w, conv_b, conv_state, A_log, dt_bias, t_row, t_pos, t_off, xs, v, kn, qn, decay, H, dv, groups,
             state, taps):
    """Convolution + silu of the x | B | C columns of ``proj`` (from ``col_x``), dt and the decay: the inputs of the
    plain-accumulation scan (k = B, q = C, v = dt x) and the convolved x for the skip term."""
    _dev(proj, conv_w, conv_b, conv_state, A_log, dt_bias, t_row, t_pos, t_off, xs, v, kn, qn, decay)
    M = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1
    for t in (xs, v, kn, qn, decay):
        assert t.dtype == torch.float32 and t.is_contiguous()
    _call("b200p_ssm_prep", lambda: lib().b200p_ssm_prep(_p(proj), proj.stride(0), int(col_x), int(col_dt), _p(conv_w), _p(conv_b),
                                                        _p(conv_state), _p(A_log), _p(dt_bias), _p(t_row), _p(t_pos), _p(t_off), _p(xs),
                                                        _p(v), _p(kn), _p(qn), _p(decay), M, H, dv, groups, state, taps, _stream()))


def ssm_out(o, xs, z, D, norm_w, out, H, dv, parts, eps):
    """out = group_rms_norm((o + D xs) * silu(z)) * norm_w over ``parts`` equal runs of the channels; ``z`` may be a column slice."""
    _dev(o, xs, z, D, norm_w, out)
    M = o.shape[0]
    assert z.dtype == torch.float32 and z.stride(1) == 1 and out.stride(1) == 1 and o.is_contiguous() and xs.is_contiguous()
    _call("b200p_ssm_out", lambda: lib().b200p_ssm_out(_p(o), _p(xs), _p(z), z.stride(0), _p(D), _p(norm_w), _p(out), out.stride(0), M, H,
                                                      dv, int(parts), float(eps), dtype_code(out.dtype), _stream()))


def rope_attn_prep(proj, col_q, col_k, col_v, rates, rot_dims, scale, q_out, kcache, vcache, t_row, t_pos, H, G, maps, d, dv):
    """Rotated, scaled queries to ``q_out`` fp32 [M, H maps d]; rotated keys and the values into the caches
    [rows, G, Tcap, maps d] / [rows, G, Tcap, dv] at every token's (row, position)."""
    _dev(proj, rates, q_out, kcache, vcache, t_row, t_pos)
    M = proj.shape[0]
    assert proj.dtype == torch.float32 and kcache.is_contiguous() and vcache.is_contiguous() and kcache.dtype == vcache.dtype
    assert kcache.shape[1:] == (G, kcache.shape[2], maps * d) and vcache.shape[1:] == (G, kcache.shape[2], dv)
    _call("b200p_rope_attn_prep", lambda: lib().b200p_rope_attn_prep(
        _p(proj), proj.stride(0), int(col_q), int(col_k), int(col_v), _p(rates), int(rot_dims), float(scale), _p(q_out), _p(kcache),
        _p(vcache), kcache.shape[2], _p(t_row), _p(t_pos), M, H, G, maps, d, dv, dtype_code(kcache.dtype), _stream()))


def diff_attn_workspace_floats(nb: int, H: int, maps: int, dv: int) -> int:
    return lib().b200p_diff_attn_workspace_bytes(nb, H, maps, dv) // 4


def diff_attn(q, kcache, vcache, t_row, t_pos, out, H, G, maps, d, dv, chunk=0, lam=0.0, eps=-1.0, post=1.0, cu=None, rows=None, nb=0,
              max_n=1, workspace=None):
    """Chunk-masked attention with ``maps`` score maps per head over the caches: out = post * unit_rms(a_1 - lam a_2) (``eps``
    < 0: no division by the root mean square); ``out`` [M, >= H dv] in the caches' dtype."""
    _dev(q, kcache, vcache, t_row, t_pos, out, cu, rows, workspace)
    M = q.shape[0]
    assert q.dtype == torch.float32 and q.is_contiguous() and out.stride(1) == 1 and out.dtype == kcache.dtype
    _call("b200p_diff_attn", lambda: lib().b200p_diff_attn(
        _p(q), _p(kcache), _p(vcache), kcache.shape[2], _p(t_row), _p(t_pos), _p(cu), _p(rows), int(nb), int(max_n), int(chunk), int(maps),
        float(lam), float(eps), float(post), _p(out), out.stride(0), M, H, G, d, dv, dtype_code(kcache.dtype), _p(workspace),
        0 if workspace is None else workspace.numel() * 4, _stream()))
    return out


def scale_(y, s: float):
    """y *= s in place (fp32, contiguous)."""
    _dev(y)
    assert y.dtype == torch.float32 and y.is_contiguous()
    _call("b200p_scale", lambda: lib().b200p_scale(_p(y), y.numel(), float(s), _stream()))
    return y


def latent_prep(proj, q_rank, kv_rank, wq, wkv, eps, cq_out, cache, t_row, t_pos):
    """``cache`` [rows, Tcap, kv_rank] or None for a layer that reads another layer's latents (kv_rank 0)."""
    _dev(proj, wq, wkv, cq_out, cache, t_row, t_pos)
    M = proj.shape[0]
    Tcap = 0 if cache is None else cache.shape[1]
    _call("b200p_latent_prep", lambda: lib().b200p_latent_prep(_p(proj), proj.stride(0), q_rank, kv_rank if cache is not None else 0,
                                                              _p(wq), _p(wkv), float(eps), _p(cq_out), _p(cache), Tcap, _p(t_row),
                                                              _p(t_pos), M, dtype_code(cq_out.dtype), _stream()))


# The tensor-core tile kernel takes prompts (entries of at least LATENT_TILES_MIN_TOKENS tokens: tiles over tokens) and decode
# steps of models with at least LATENT_TILES_MIN_HEADS heads (one token per entry: tiles over its heads); the per-token kernel
# takes what is left (very short portions, few heads, float32, odd ranks).
LATENT_TILES_MIN_TOKENS = 4
LATENT_TILES_MIN_HEADS = 8


def latent_attn(q, cache, t_row, t_pos, out, H, R, window, scale, cu=None, rows=None, nb=0, max_n=1):
    """Windowed attention of H heads over the latent cache.  With the ragged description (cu, rows, nb, longest entry max_n)
    prompts of 16-bit models run on the tensor-core tile kernel; everything else on the per-token kernel."""
    _dev(q, cache, t_row, t_pos, out, cu, rows)
    M = q.shape[0]
    assert q.dtype == torch.float32 and q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and out.dtype == cache.dtype
    if (cu is not None and (max_n >= LATENT_TILES_MIN_TOKENS or (max_n == 1 and H >= LATENT_TILES_MIN_HEADS))
            and lib().b200p_latent_attn_tiles_supported(R, dtype_code(cache.dtype))):
        _call("b200p_latent_attn_tiles", lambda: lib().b200p_latent_attn_tiles(_p(q), _p(cache), cache.shape[1], _p(cu), _p(rows),
                                                                              _p(t_pos), _p(out), nb, int(max_n), H, R, int(window),
                                                                              float(scale), dtype_code(cache.dtype), _stream()))
        return out
    _call("b200p_latent_attn", lambda: lib().b200p_latent_attn(_p(q), _p(cache), cache.shape[1], _p(t_row), _p(t_pos), _p(out), M, H, R,
                                                              int(window), float(scale), dtype_code(cache.dtype), _stream()))
    return out


def latent_rope_prep(proj, q_rank, kv_rank, rot_dim, wq, wkv, eps, rates, mag, cq_out, cache, t_row, t_pos):
    """Latent attention with a rotated key part: ``proj`` = [query | key/value | rotated part]; ``cache`` [rows, Tcap, row] gets
    [normed latent | rotated part | zeros]."""
    _dev(proj, wq, wkv, rates, cq_out, cache, t_row, t_pos)
    M = proj.shape[0]
    assert proj.dtype == torch.float32 and cache.is_contiguous() and cq_out.is_contiguous() and cq_out.dtype == cache.dtype
    _call("b200p_latent_rope_prep", lambda: lib().b200p_latent_rope_prep(
        _p(proj), proj.stride(0), int(q_rank), int(kv_rank), int(rot_dim), cache.shape[2], _p(wq), _p(wkv), float(eps), _p(rates), float(mag),
        _p(cq_out), _p(cache), cache.shape[1], _p(t_row), _p(t_pos), M, dtype_code(cache.dtype), _stream()))


def latent_q_rope(q, H, dim, rot_dim, kv_rank, rates, mag, t_pos, q_lat):
    """The rotated part of the queries ``q`` [M, H * (dim + rot_dim)] into columns [kv_rank, kv_rank + rot_dim) of every head's
    row of ``q_lat`` fp32 [M, H * row]; the columns behind become zero."""
    _dev(q, rates, t_pos, q_lat)
    M = q.shape[0]
    row = q_lat.shape[1] // H
    assert q.is_contiguous() and q_lat.is_contiguous() and q_lat.dtype == torch.float32 and q.shape[1] == H * (dim + rot_dim)
    _call("b200p_latent_q_rope", lambda: lib().b200p_latent_q_rope(_p(q), H, int(dim), int(rot_dim), int(kv_rank), row, _p(rates), float(mag),
                                                                  _p(t_pos), _p(q_lat), M, dtype_code(q.dtype), _stream()))


def window_attn_prep(proj, col_q, conv_w, conv_state, taps, scale, q_out, kcache, t_row, t_pos, t_off, H, G, dk):
    """Convolved q (scaled, fp32) to ``q_out``; convolved k into ``kcache`` [rows, G, Tcap, dk] at every token's (row, position)."""
    _dev(proj, conv_w, conv_state, q_out, kcache, t_row, t_pos, t_off)
    M = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and kcache.is_contiguous() and q_out.is_contiguous()
    assert kcache.shape[1:] == (G, kcache.shape[2], dk) and conv_w.shape == (taps, (H + G) * dk)
    _call("b200p_window_attn_prep", lambda: lib().b200p_window_attn_prep(
        _p(proj), proj.stride(0), int(col_q), _p(conv_w), _p(conv_state), int(taps), float(scale), _p(q_out), _p(kcache), kcache.shape[2],
        _p(t_row), _p(t_pos), _p(t_off), M, H, G, dk, dtype_code(kcache.dtype), _stream()))


def window_attn(q, kcache, vcache, t_row, t_pos, out, H, G, dk, dv, softcap=0.0, r1=None, r2=None, window=0, gate=None, cu=None,
                rows=None, nb=0, max_n=1, workspace=None):
    """Sliding-window attention with capped scores, a logarithmic distance penalty and an output gate (every option off at its
    default); ``vcache`` may be ``kcache``.  ``gate``: fp32 [M, >= H * dv] pre-activations (a column slice is fine)."""
    _dev(q, kcache, vcache, t_row, t_pos, out, r1, r2, gate, cu, rows)
    M = q.shape[0]
    assert q.dtype == torch.float32 and q.is_contiguous() and out.stride(1) == 1 and out.dtype == kcache.dtype
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    _call("b200p_window_attn", lambda: lib().b200p_window_attn(
        _p(q), _p(kcache), _p(vcache), kcache.shape[2], _p(t_row), _p(t_pos), _p(cu), _p(rows), int(nb), int(max_n), float(softcap), _p(r1),
        _p(r2), int(window), _p(gate), 0 if gate is None else gate.stride(0), _p(out), out.stride(0), M, H, G, dk, dv,
        dtype_code(kcache.dtype), _p(workspace), 0 if workspace is None else workspace.numel() * 4, _stream()))
    return out


def moe_route_scores(logits, ids, wts, seg, slot_of, token_of, top: int, experts: Optional[int] = None):
    """Routing by the largest sigmoid scores; the weights are the scores themselves."""
    _dev(logits, ids, wts, seg, slot_of, token_of)
    M = logits.shape[0]
    E = logits.shape[1] if experts is None else int(experts)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _call("b200p_moe_route_scores", lambda: lib().b200p_moe_route_scores(_p(logits), logits.stride(0), _p(ids), _p(wts), _p(seg), _p(slot_of),
                                                                        _p(token_of), M, E, int(top), _stream()))


def moe_scatter_scaled(x, slot_of, wts, xs, top: int):
    """xs[slot of (t, k)] = wts[t, k] * x[t]: the routing weight on the expert's input."""
    _dev(x, slot_of, wts, xs)
    assert x.is_contiguous() and xs.is_contiguous() and x.dtype == xs.dtype and x.shape[1] == xs.shape[1] and wts.dtype == torch.float32
    _call("b200p_moe_scatter_scaled", lambda: lib().b200p_moe_scatter_scaled(_p(x), _p(slot_of), _p(wts), _p(xs), x.shape[0], x.shape[1],
                                                                            int(top), dtype_code(x.dtype), _stream()))


def hyper_step(xs, streams: int, y=None, src=None, mix=None, out=None, read=None, alpha=None, w=None, b=None, n_out=None, sum_out=None,
               conv_w=None, conv_state=None, t_row=None, t_pos=None, taps=1, x_out=None):
    """One pass over the copies of the residual stream ``xs`` fp32 [M, streams * W]: write a sublayer's output ``y`` back
    (``mix`` [from, to], ``out``), read for the next one (``read``) and norm it with tanh(alpha u) w + b into ``n_out``; with
    ``x_out`` (a decode step) the short convolution over the carried inputs is added and the carried inputs are shifted too."""
    _dev(xs, y, src, mix, out, read, alpha, w, b, n_out, sum_out, conv_w, conv_state, t_row, t_pos, x_out)
    M = xs.shape[0]
    W = xs.shape[1] // streams
    assert xs.dtype == torch.float32 and xs.is_contiguous()
    for t in (y, src, n_out, sum_out):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.shape == (M, W))
    for t in (mix, out, read, alpha, w, b, conv_w):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    assert (mix is None) == (out is None) and (mix is None or mix.numel() == streams * streams)
    assert x_out is None or (x_out.is_contiguous() and conv_w.shape == (taps, W) and conv_state.is_contiguous())
    _call("b200p_hyper_step", lambda: lib().b200p_hyper_step(
        _p(xs), _p(y), _p(src), _p(mix), _p(out), _p(read), _p(alpha), _p(w), _p(b), _p(n_out), _p(sum_out), M, int(streams), W, _p(conv_w),
        _p(conv_state), _p(t_row), _p(t_pos), int(taps), _p(x_out), dtype_code(x_out.dtype if x_out is not None else torch.float32),
        _stream()))


def canon_conv(n, conv_w, conv_state, t_row, t_pos, t_off, x_out, taps: int):
    """x_out = n + causal convolution of n over time (``conv_w`` [taps, W], tap by tap; ``conv_state`` [rows, taps-1, W] = earlier
    steps)."""
    _dev(n, conv_w, conv_state, t_row, t_pos, t_off, x_out)
    M, W = n.shape
    assert n.dtype == torch.float32 and n.is_contiguous() and x_out.is_contiguous() and conv_w.shape == (taps, W) and conv_state.is_contiguous()
    _call("b200p_canon_conv", lambda: lib().b200p_canon_conv(_p(n), _p(conv_w), _p(conv_state), _p(t_row), _p(t_pos), _p(t_off), _p(x_out), M,
                                                            W, int(taps), dtype_code(x_out.dtype), _stream()))


def tanh_norm(h, alpha, w, b, x_out):
    """x_out = tanh(alpha h) w + b, rows of fp32 ``h`` into the storage type."""
    _dev(h, alpha, w, b, x_out)
    M, W = h.shape
    assert h.dtype == torch.float32 and h.is_contiguous() and x_out.is_contiguous()
    _call("b200p_tanh_norm", lambda: lib().b200p_tanh_norm(_p(h), _p(alpha), _p(w), _p(b), _p(x_out), M, W, dtype_code(x_out.dtype),
                                                          _stream()))

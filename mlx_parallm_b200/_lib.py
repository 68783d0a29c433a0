"""ctypes binding of libb200parallm.so (the C-ABI declared in include/b200p.h).

There is no fallback: if the shared library is missing or the device is not sm_100 every call
raises.  Build it with ``python -c "import __graft_entry__ as g; g.build()"`` or
``make -C mlx_parallm_b200/csrc``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200parallm.so")
# profiling builds only (scripts/tc_bisect.py): a library compiled with -DB200P_TC_DEBUG=<mask> under build/
LIB_PATH = os.environ.get("B200P_LIB", LIB_PATH)

F32, F16, BF16 = 0, 1, 2
DQ_F32_MULADD, DQ_FMA, DQ_T_MULADD = 0, 1, 2
EPI_STORE, EPI_STORE_F32, EPI_ADD_RESIDUAL, EPI_SILU_MUL = 0, 1, 2, 3
X_PERM8, Y_PERM8, OUT_PERM8 = 0x100, 0x200, 0x1      # activation-layout flags (include/b200p.h)
W_SMALLSCALE = 0x400                                 # every |scale| < 0.0625: subnormal-operand dequant (f16 only)

_vp, _i64, _i32, _f32, _u64, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_uint64, C.c_size_t

# name -> (restype, argtypes); mirrors include/b200p.h one to one
SIGNATURES = {
    "b200p_version": (C.c_char_p, []),
    "b200p_last_error": (C.c_char_p, []),
    "b200p_arch_check": (_i32, []),
    "b200p_sm_count": (_i32, []),
    "b200p_set_pdl": (_i32, [_i32]),
    "b200p_dequantize": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _vp]),
    "b200p_quantize": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _vp]),
    "b200p_embed": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200p_qmm": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "b200p_qmm_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "b200p_qmm_tensor_supported": (_i32, [_i64, _i64, _i64, _i32, _i32, _i32, _i32]),
    "b200p_qmm_set_path": (_i32, [_i32]),
    "b200p_qmm_set_min_tensor_m": (_i32, [_i32]),
    "b200p_rmsnorm": (_i32, [_vp, _vp, _vp, _i64, _i64, _f32, _i32, _i32, _vp]),
    "b200p_rope_kv_append": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i64,
                                    _f32, _f32, _f32, _i32, _i32, _vp]),
    "b200p_silu_mul": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "b200p_lora_add": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _i32, _i32, _vp]),
    "b200p_advance_lengths": (_i32, [_vp, _i64, _i32, _vp]),
    "b200p_kv_overflow_count": (_i32, [C.POINTER(C.c_uint), _i32, _vp]),
    "b200p_attn": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i64, _f32, _i32, _i32, _vp, _sz, _vp]),
    "b200p_attn_workspace_bytes": (_sz, [_i64, _i64, _i32, _i32]),
    "b200p_attn_decode_static": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i64, _f32, _i32, _i32, _vp]),
    "b200p_attn_set_path": (_i32, [_i32]),
    "b200p_argmax": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200p_argmax_partial": (_i32, [_vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "b200p_argmax_merge": (_i32, [_vp, _vp, _vp, _i32, _i64, _vp]),
    "b200p_sample_top_p": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _f32, _f32, _u64, _u64, _vp]),
    "b200p_symm_alloc": (_i32, [C.POINTER(_vp), _sz]),
    "b200p_symm_free": (_i32, [_vp]),
    "b200p_ipc_export": (_i32, [_vp, _vp]),
    "b200p_ipc_import": (_i32, [_vp, C.POINTER(_vp)]),
    "b200p_ipc_close": (_i32, [_vp]),
    "b200p_allreduce_flag_bytes": (_sz, []),
    "b200p_allreduce_set_max_ctas": (_i32, [_i32]),
    "b200p_allreduce_residual_rmsnorm": (_i32, [_vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _i32, _vp]),
    "b200p_allreduce_rows_rmsnorm": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _i32, _vp]),
    "b200p_peer_allgather": (_i32, [_vp, _vp, _i32, _i32, _vp, _i64, _vp]),
    "b200p_peer_status": (_i32, [_vp, _vp, _vp]),
    # dense linear layers, ragged batches, gated delta rule, latent attention
    "b200p_gemm": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _f32, _vp]),
    "b200p_gemm_set_path": (_i32, [_i32]),
    "b200p_gemm_tc_fault": (_i32, []),
    "b200p_ragged_plan": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _vp]),
    "b200p_ragged_advance": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _vp]),
    "b200p_embed_hashed": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _i64, _i64, _i64, _i32, _vp]),
    "b200p_norm_add_norm": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32, _i32, _vp]),
    "b200p_token_gate": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i64, _i64, _i32, _vp]),
    "b200p_delta_prep": (_i32, [_vp, _i64, _i64, _vp, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200p_delta_conv_commit": (_i32, [_vp, _i64, _vp, _vp, _vp, _i32, _i64, _i32, _vp]),
    "b200p_delta_scan": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200p_delta_out": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _i32, _i32, _f32, _i32, _f32, _i32, _vp]),
    "b200p_linear_attn_prep": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp]),
    "b200p_gemm_grouped": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _f32, _vp]),
    "b200p_residual_add_norm": (_i32, [_vp, _vp, _f32, _vp, _f32, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _vp]),
    "b200p_cast_columns": (_i32, [_vp, _i64, _vp, _i64, _i64, _i64, _i32, _vp]),
    "b200p_sink_attn_prep": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, _vp, _f32, _f32, _f32, _f32, _vp, _vp, _vp, _i64, _vp, _vp,
                                    _i64, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200p_sink_attn": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _f32, _vp, _i64, _f32, _i64, _i32, _i32, _i32,
                               _i32, _i32, _vp, _sz, _vp]),
    "b200p_sink_attn_workspace_bytes": (_sz, [_i64, _i32, _i32]),
    "b200p_sink_attn_tiles_supported": (_i32, [_i32, _i32, _i32]),
    "b200p_moe_route": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "b200p_moe_gather": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp]),
    "b200p_moe_route_sigmoid": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _f32, _vp]),
    "b200p_moe_combine": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i32, _vp]),
    "b200p_moe_route_scores": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "b200p_moe_scatter_scaled": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b200p_ssm_prep": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32,
                              _i32, _i32, _i32, _vp]),
    "b200p_ssm_out": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _f32, _i32, _vp]),
    "b200p_rope_attn_prep": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, _i32, _f32, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32,
                                    _i32, _i32, _i32, _vp]),
    "b200p_diff_attn": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _i32, _f32, _f32, _f32, _vp, _i64, _i64, _i32,
                               _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "b200p_diff_attn_workspace_bytes": (_sz, [_i64, _i32, _i32, _i32]),
    "b200p_scale": (_i32, [_vp, _i64, _f32, _vp]),
    "b200p_latent_prep": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp, _f32, _vp, _vp, _i64, _vp, _vp, _i64, _i32, _vp]),
    "b200p_latent_attn": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _i64, _i32, _i32, _i64, _f32, _i32, _vp]),
    "b200p_latent_attn_set_groups": (_i32, [_i32]),
    "b200p_latent_attn_set_splits": (_i32, [_i32]),
    "b200p_latent_attn_set_buffers": (_i32, [_i32]),
    "b200p_latent_attn_tiles_supported": (_i32, [_i32, _i32]),
    "b200p_latent_attn_tiles": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i64, _f32, _i32, _vp]),
    "b200p_latent_rope_prep": (_i32, [_vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _f32, _vp, _f32, _vp, _vp, _i64, _vp, _vp, _i64, _i32,
                                      _vp]),
    "b200p_latent_q_rope": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _vp, _f32, _vp, _vp, _i64, _i32, _vp]),
    "b200p_window_attn_prep": (_i32, [_vp, _i64, _i64, _vp, _vp, _i32, _f32, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32,
                                      _vp]),
    "b200p_window_attn": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _f32, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64,
                                 _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "b200p_hyper_step": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i64, _vp, _vp, _vp, _vp, _i32, _vp,
                                _i32, _vp]),
    "b200p_canon_conv": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b200p_tanh_norm": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _vp]),
}

# Translation units a model family needs (csrc/*.cu): the library can be linked from a subset, so that a fresh checkout
# that serves one design compiles that design's kernels only.  ``None`` = every unit (libb200parallm.so).
UNIT_SETS = {
    "sequence": ("runtime", "dense_gemm", "dense_gemm_tc", "ragged", "delta_rule", "latent_attn", "sampler"),
    "sequence_moe": ("runtime", "dense_gemm", "dense_gemm_tc", "ragged", "delta_rule", "sink_attn", "moe", "sampler"),
    "sequence_ssm": ("runtime", "dense_gemm", "dense_gemm_tc", "ragged", "delta_rule", "ssm", "diff_attn", "moe", "sampler"),
    "sequence_hyper": ("runtime", "dense_gemm", "dense_gemm_tc", "ragged", "hyper", "delta_rule", "latent_attn", "sink_attn", "moe",
                       "sampler"),
}
GEMM_STORE, GEMM_STORE_F32, GEMM_GLU_CLAMP, GEMM_GLU_GELU_TANH, GEMM_GLU_SILU, GEMM_RELU_SQ = 0, 1, 2, 3, 4, 5


def gemm_is_gated(epilogue: int) -> bool:
    """Epilogues that read (gate, up) row pairs and write half as many columns."""
    return GEMM_GLU_CLAMP <= epilogue <= GEMM_GLU_SILU

SCAN_DELTA, SCAN_DELTA_CHANNEL, SCAN_ACCUMULATE = 0, 1, 2
GATE_SILU, GATE_SIGMOID = 0, 1

_lib = None


class B200PError(RuntimeError):
    pass


def _bind(path: str, partial: bool) -> C.CDLL:
    L = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(L, name)          # AttributeError on the full library = header/library drift
        except AttributeError:
            if not partial:
                raise
            continue
        fn.restype, fn.argtypes = res, args
    return L


def lib() -> C.CDLL:
    """Load (once) and return the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200PError(
                f"{LIB_PATH} not found: the CUDA extension is not built and there is no CPU fallback "
                "(run `make -C mlx_parallm_b200/csrc`)")
        _lib = _bind(LIB_PATH, partial=False)
    return _lib


def ensure_built(unit_set: str, verbose: bool = False) -> C.CDLL:
    """Make sure a library that holds the kernels of ``unit_set`` (a key of UNIT_SETS) is loaded.  The complete library is
    used when it exists; otherwise the set's translation units are compiled with nvcc for sm_100a and linked into
    ``libb200parallm_<unit_set>.so`` next to it (first call only: make sees the objects afterwards).  A function of a unit
    that is not in the set is absent from that library and raises AttributeError when called."""
    global _lib
    if _lib is not None:
        return _lib
    if os.path.exists(LIB_PATH):
        return lib()
    import subprocess
    units = UNIT_SETS[unit_set]
    part = os.path.join(_HERE, f"libb200parallm_{unit_set}.so")
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), f"-j{min(8, os.cpu_count() or 1)}",
           "SRCS=" + " ".join(u + ".cu" for u in units), "LIB=" + part]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0 or not os.path.exists(part):
        raise B200PError(f"building {part} failed:\n{r.stdout[-4000:]}")
    if verbose:
        print(r.stdout)
    _lib = _bind(part, partial=True)
    return _lib


def last_error() -> str:
    return lib().b200p_last_error().decode()


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        raise B200PError(f"{what or 'b200p call'} failed ({rc}): {last_error()}")


def require_device() -> None:
    """Fail loudly unless an sm_100 device is current."""
    check(lib().b200p_arch_check(), "b200p_arch_check")

/*
 * b200p.h -- C-ABI of libb200parallm.so: the sm_100a kernels under the batched decode step.
 *
 * The reference (misanthropic-ai/mlx_parallm) has no FFI of its own: its arithmetic is reached
 * through mlx.core (nanobind).  Each entry point below therefore cites the *MLX call site in the
 * reference* that it replaces (paths relative to the reference root).  A maintainer binds these
 * with ctypes; mlx_parallm_b200/_lib.py is that binding.
 *
 * Conventions
 *   - every function returns 0 on success or a negative B200P_ERR_*; b200p_last_error() gives a
 *     thread-local message.
 *   - all pointers are CALLER-OWNED DEVICE pointers unless named host_*; nothing is allocated,
 *     freed or synchronised inside; every launch is ordered on `stream` (a cudaStream_t passed as
 *     void*) and is CUDA-graph capturable.
 *   - `dtype` is the storage type of activations, scales, biases and KV (MLX unifies them through
 *     result_type before quantized_matmul): B200P_F32 / F16 / BF16.
 *   - quantized weights are in MLX layout: w uint32 [N, K*bits/32] (element j of a word in bits
 *     [j*bits,(j+1)*bits)), scales/biases [N, K/group_size]; group_size 64 or 128... (any multiple
 *     of 32 dividing K for the generic path; the tensor path requires 64), bits in {4, 8}.
 *   - there is NO CPU fallback: without an sm_100 device b200p_arch_check() fails and every
 *     launch returns B200P_ERR_ARCH / B200P_ERR_CUDA.
 */
#ifndef B200P_H
#define B200P_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200P_OK          0
#define B200P_ERR_ARG    -1   /* bad shape / null pointer / unsupported combination */
#define B200P_ERR_ALIGN  -2   /* pointer or leading dimension not aligned as required */
#define B200P_ERR_ARCH   -3   /* device is not sm_100 */
#define B200P_ERR_CUDA   -4   /* CUDA runtime error (message in b200p_last_error) */

enum { B200P_F32 = 0, B200P_F16 = 1, B200P_BF16 = 2 };

/* dequantize rounding (oracle/mlx_ops.py MODE_*) */
enum { B200P_DQ_F32_MULADD = 0, B200P_DQ_FMA = 1, B200P_DQ_T_MULADD = 2 };

/* b200p_qmm epilogues */
enum {
  B200P_EPI_STORE = 0,        /* y[M,N] (dtype) = acc                                   */
  B200P_EPI_STORE_F32 = 1,    /* y[M,N] (float) = acc                (lm_head logits)    */
  B200P_EPI_ADD_RESIDUAL = 2, /* y[M,N] (float) += acc               (o_proj, down_proj) */
  B200P_EPI_SILU_MUL = 3      /* y[M,N/2] (dtype) = silu(acc[:, :N/2]) * acc[:, N/2:]
                                 rows [0,N/2) of w are gate_proj, rows [N/2,N) up_proj   */
};

/* Activation-layout flags OR-ed into the `epilogue` argument of b200p_qmm, and passed as `flags` to the producer
 * kernels (b200p_rmsnorm, b200p_attn).  PERM8: inside every aligned group of 8 consecutive elements of a row
 * the values sit in the order [0,4,1,5,2,6,3,7] -- the order in which the nibbles of a 4-bit weight word unpack as
 * packed 16-bit pairs -- so the tensor path skips the re-pairing PRMTs.  Purely internal to a chain of our kernels:
 * a tensor written with Y_PERM8 / OUT_PERM8 must be consumed with X_PERM8. */
#define B200P_X_PERM8   0x100   /* x of b200p_qmm is PERM8 (4-bit weights only)                          */
#define B200P_Y_PERM8   0x200   /* 16-bit y of b200p_qmm (STORE, SILU_MUL) is written PERM8              */
#define B200P_OUT_PERM8 0x1     /* flags of b200p_rmsnorm / b200p_attn: write the 16-bit output PERM8 */
/* Caller's promise about the weights of a b200p_qmm call, OR-ed into `epilogue` like the layout flags: every scale of the
 * matrix satisfies |s| < 0.0625 (checked once at load time by the host: mlx_parallm_b200/models/_transformer.py).  F16
 * calls then dequantise with ONE half2 FMA per code pair on subnormal operands (csrc/dequant.cuh) -- same rounding of
 * q*s+b, two thirds of the instructions.  Ignored for BF16 / F32. */
#define B200P_W_SMALLSCALE 0x400

const char* b200p_version(void);
const char* b200p_last_error(void);
/* 0 iff the current device is compute capability 10.x */
int b200p_arch_check(void);
int b200p_sm_count(void);
/* Programmatic dependent launch for every kernel of the library (default on): kernel N+1's prologue and weight
 * prefetch overlap kernel N's tail; each kernel executes griddepcontrol.wait before touching its inputs. */
int b200p_set_pdl(int enabled);

/* mx.dequantize(w, scales, biases, group_size, bits)            [nn.QuantizedEmbedding.__call__,
 * models/llama.py:212, models/qwen3.py:166; bit-exactness target of the north star]
 * out[N,K] in `dtype`. */
int b200p_dequantize(const uint32_t* w, const void* scales, const void* biases, void* out,
                     int64_t N, int64_t K, int group_size, int bits, int dtype, int mode,
                     void* stream);

/* mx.quantize(w, group_size, bits)                                  [nn.quantize, utils.py:886-905; convert, utils.py:934-981]
 * w `dtype` [N,K] -> wq uint32 [N, K*bits/32], scales / biases `dtype` [N, K/group_size]; every step rounded to `dtype`
 * where MLX's composed ops round it: bit-exact against oracle/mlx_ops.py quantize.
 * group_size 32, 64 or 128. */
int b200p_quantize(const void* w, uint32_t* wq, void* scales, void* biases, int64_t N, int64_t K, int group_size,
                   int bits, int dtype, void* stream);

/* embed_tokens(ids): gather rows + dequantize                    [models/llama.py:212]
 * ids int32 [M]; out float [M,K] if out_f32 else `dtype` [M,K] (values are the dtype-rounded
 * dequantised weights either way). */
int b200p_embed(const int32_t* ids, const uint32_t* w, const void* scales, const void* biases,
                void* out, int64_t M, int64_t V, int64_t K, int group_size, int bits, int dtype,
                int mode, int out_f32, void* stream);

/* mx.quantized_matmul(x, w, scales, biases, transpose=True)       [nn.QuantizedLinear.__call__:
 * models/llama.py:93,143,165,250-252; models/qwen3.py:63,115]
 * x `dtype` [M,K] row-major (ldx elements between rows), y per `epilogue` (ldy elements between
 * rows).  fp32 accumulation.  Internally: the mma.sync register GEMV (4-bit g64, 16-bit, M <= 16, fp32 outputs), the
 * tcgen05 tile path (F16/BF16, group 64) or the generic CUDA-core GEMV (any dtype / shape).  `workspace` (>= b200p_qmm_workspace_bytes) is
 * required by the split-K tensor path; may be NULL for the GEMV path. */
int b200p_qmm(const void* x, const uint32_t* w, const void* scales, const void* biases, void* y,
              int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldy, int group_size, int bits,
              int dtype, int epilogue, void* workspace, size_t workspace_bytes, void* stream);
size_t b200p_qmm_workspace_bytes(int64_t M, int64_t N, int64_t K);
/* 1 if the tcgen05 tile path can run this call, else 0 */
int b200p_qmm_tensor_supported(int64_t M, int64_t N, int64_t K, int group_size, int bits, int dtype,
                               int epilogue);
/* force a path for tests/benchmarks: 0 = auto, 1 = CUDA-core GEMV only, 2 = tcgen05 tile kernels only, 3 = mma.sync
 * GEMV only, 4 = mma.sync small-matrix GEMM only (csrc/qmm_mma.cu: ADD_RESIDUAL, M <= 64, N % 128 == 0, K % 256 == 0)
 * (2, 3 and 4: error if the call is unsupported on that path) */
int b200p_qmm_set_path(int path);
/* smallest M routed to the tensor path in auto mode (default 1: measured, scripts/qmm_sweep.py, profiles/r1_run11_qmm_sweep_gemv_vs_tensor.txt) */
int b200p_qmm_set_min_tensor_m(int m);

/* mx.fast.rms_norm(x, w, eps)                                      [nn.RMSNorm: models/llama.py:187,
 * 189,231]  x float [M,H] (the fp32 residual stream) -> y `dtype` [M,H]; w `dtype` [H]. */
int b200p_rmsnorm(const float* x, const void* w, void* y, int64_t M, int64_t H, float eps,
                  int dtype, int flags, void* stream);

/* per-head q/k RMSNorm (qwen3 only) + mx.fast.rope at per-row offsets + cache append
 *                      [models/qwen3.py:65-70; models/llama.py:107-117; models/base.py:119-140]
 * qkv `dtype` [B*L, (Hq+2*Hkv)*D] (q heads, then k heads, then v heads);
 * q_out `dtype` [B, L, Hq, D]; kcache/vcache `dtype` [B, Hkv, Tcap, D];
 * lengths int32 [B] = tokens already in the cache per row (position of token l is lengths[b]+l);
 * q_norm_w / k_norm_w `dtype` [D] or NULL.  Does NOT advance lengths.
 * qkv_f32 = 1: qkv is instead the float accumulation buffer of the fused projection (b200p_qmm with
 * B200P_EPI_ADD_RESIDUAL into a zeroed buffer); values are rounded to `dtype` on read and the buffer is re-zeroed. */
int b200p_rope_kv_append(void* qkv, void* q_out, void* kcache, void* vcache,
                         const int32_t* lengths, const void* q_norm_w, const void* k_norm_w,
                         int64_t B, int64_t L, int Hq, int Hkv, int D, int64_t Tcap,
                         float rope_base, float rope_scale, float norm_eps, int dtype,
                         int qkv_f32, void* stream);
/* nn.silu(gate) * up                                                  [models/llama.py:165]
 * gu float [M, 2*I] (ldg floats between rows): columns [0,I) = gate_proj, [I,2I) = up_proj sums, as accumulated by
 * b200p_qmm(..., B200P_EPI_ADD_RESIDUAL) of the fused gate|up matrix into a ZEROED buffer (stream-K partial tiles
 * then need no second pass); out `dtype` [M, I] (ldo), optionally PERM8 (flags = B200P_OUT_PERM8).
 * The kernel re-zeroes gu behind its read, so the buffer is ready for the next step. */
int b200p_silu_mul(float* gu, void* out, int64_t M, int64_t I, int64_t ldg, int64_t ldo, int dtype, int flags,
                   void* stream);
/* LoRA low-rank update (mlx_lm LoRALinear: y = linear(x) + (scale * (x @ lora_a) @ lora_b).astype(x.dtype))
 *                                       [adapters on q_proj / v_proj: lora_init.py:63-73; SURVEY A.9, row f4]
 * x `dtype` [M,K] (ldx); At `dtype` [16, K] = lora_a transposed, rank padded to 16 with zero rows (k axis permuted like x
 * when x is PERM8); Bt `dtype` [N, 16] = lora_b transposed, padded likewise; y[m, col0 + n] += update for n < N:
 * out_f32 = 1 -> y is the float accumulation buffer of the projection (ldy floats), else its `dtype` output (the update
 * is rounded to `dtype` first, as MLX's astype does).  16-bit types only. */
int b200p_lora_add(const void* x, const void* At, const void* Bt, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx,
                   int64_t ldy, int64_t col0, float scale, int dtype, int out_f32, void* stream);
/* Rows that b200p_rope_kv_append could NOT append because lengths[b] + l reached Tcap (their K / V are dropped and the
 * attention of that step reads a stale slot): *count = number of (token, V head) pairs since the last reset on the current
 * device; reset != 0 clears it.  Synchronises `stream`; not capturable.  The Python surface (models/base.py) grows the cache
 * before every step and checks this at generation boundaries; direct C-ABI callers should do the same.
 *                      [no MLX counterpart: the reference's caches grow inside update_and_fetch, models/base.py:104-117] */
int b200p_kv_overflow_count(unsigned int* count, int reset, void* stream);
/* lengths[b] += delta (device side, keeps the decode graph replayable) */
int b200p_advance_lengths(int32_t* lengths, int64_t B, int32_t delta, void* stream);

/* mx.fast.scaled_dot_product_attention for cached decode / chunked prefill
 *                      [models/llama.py:139-141, models/qwen3.py:111-113; causal rule of
 *                       models/base.py:17-40 applied by bound, not by an additive -1e9 mask]
 * q `dtype` [B, L, Hq, D]; caches as above; query (b,l) attends to keys [0, lengths[b]+l+1)
 * (lengths = tokens in cache BEFORE this call's L tokens were appended).
 * out `dtype` [B, L, Hq*D].  workspace: float, >= b200p_attn_workspace_bytes. */
int b200p_attn(const void* q, const void* kcache, const void* vcache, const int32_t* lengths,
               void* out, int64_t B, int64_t L, int Hq, int Hkv, int D, int64_t Tcap,
               float scale, int dtype, int flags, void* workspace, size_t workspace_bytes, void* stream);
size_t b200p_attn_workspace_bytes(int64_t B, int64_t L, int Hq, int D);
/* Decode attention (L == 1) that allocates NOTHING: b200p_attn's split-K decode kernel with its split partials in a
 * file-scope device array of the library instead of a caller-allocated workspace.
 *                      [no counterpart in the reference: added at the request of the run's operators, for callers that
 *                       cannot call cudaMalloc -- code under CUDA graph capture, tight serving loops, harnesses that forbid it]
 * Same arguments and result as b200p_attn with L = 1 (bit-identical: same kernels, same split count); 16-bit caches,
 * D == 128, Hq / Hkv <= 16 only.  The scratch is B200P_ATTN_STATIC_SCRATCH_BYTES (16 MiB, held by every GPU that loads the
 * library until the process exits), i.e. B * Hq <= 992; larger calls are rejected with B200P_ERR_ARG -- use b200p_attn.
 * The call makes no cudaMalloc / cudaFree and calls no allocating routine; its first use on a device resolves the array's
 * device address (cudaGetSymbolAddress), so make that first call outside a stream capture.
 * Every call shares the array, which keeps the last call's contents (nothing in it has to start at zero: each call writes
 * every record it later reads).  Calls that overlap on the GPU -- two streams, concurrent graph branches -- RACE on it:
 * serialise them. */
#define B200P_ATTN_STATIC_SCRATCH_BYTES (16u << 20)
int b200p_attn_decode_static(const void* q, const void* kcache, const void* vcache, const int32_t* lengths,
                             void* out, int64_t B, int Hq, int Hkv, int D, int64_t Tcap,
                             float scale, int dtype, int flags, void* stream);
/* 0 = auto, 1 = generic CUDA-core kernel only, 2 = tensor (mma) kernels only: split-K decode for L == 1, causal flash
 * prefill for L > 1 (16-bit, head_dim 128) */
int b200p_attn_set_path(int path);

/* mx.argmax(logits, axis=-1, keepdims=True)                         [utils.py:350-352,363]
 * logits float [B, V] (ldl floats between rows) -> tokens int32 [B]; lowest index among ties.
 * probs_out (optional, float [B]) receives softmax(logits)[b, token] computed in the same pass.
 * B <= 65535.  Each row is split over a thread-block cluster of 8 / 4 / 2 / 1 CTAs so that B x cluster fills the SMs once
 * (env B200P_SAMPLER_CLUSTER forces a size); the same holds for b200p_argmax_partial and b200p_sample_top_p. */
int b200p_argmax(const float* logits, int32_t* tokens, float* probs_out, int64_t B, int64_t V,
                 int64_t ldl, void* stream);

/* Vocab-parallel greedy head (tensor parallelism; new -- the reference is single-device): each rank
 * reduces ITS logits shard [B, V_local] to a 16-byte record per row {max, sum exp(l - max), global
 * argmax index (int bits), 0}; after an all-gather of the records b200p_argmax_merge picks the token
 * (highest max, lowest global index among ties = mx.argmax's rule) and softmax(logits)[token]. */
int b200p_argmax_partial(const float* logits, float* rec_out, int64_t B, int64_t V, int64_t ldl,
                         int32_t vocab_offset, void* stream);
int b200p_argmax_merge(const float* recs /* [W, B, 4] */, int32_t* tokens, float* probs_out, int W,
                       int64_t B, void* stream);

/* top_p_sampling(logits, top_p, temperature) / mx.random.categorical(logits/temp)
 *                                                        [sample_utils.py:3-39; utils.py:354-361]
 * Draws from the renormalised nucleus {tokens whose inclusive sorted cumulative mass <= top_p}
 * (top_p >= 1 -> plain categorical).  Philox counter RNG keyed by (seed, offset, row).
 * If the nucleus is empty (p_max > top_p; the reference divides 0/0) the argmax is returned.
 * Selection is by value: a nucleus that ends inside a run of exactly equal probabilities drops the run.
 * probs_out (optional, float [B]) receives softmax(logits)[b, token] (untempered, utils.py:363). */
int b200p_sample_top_p(const float* logits, int32_t* tokens, float* probs_out, int64_t B,
                       int64_t V, int64_t ldl, float temperature, float top_p, uint64_t seed,
                       uint64_t offset, void* stream);

/* ---- tensor-parallel exchange over NVLink peer memory (new; the reference is single-device) -----------------
 * Setup calls (host side, synchronous, NOT graph-capturable; the only entry points that allocate):
 *   b200p_symm_alloc   cudaMalloc + zero a buffer peers may map;   b200p_symm_free releases it
 *   b200p_ipc_export   64-byte cudaIpcMemHandle of such a buffer (ship it to the peers with any host transport)
 *   b200p_ipc_import   map a peer's buffer into this process (peer access enabled lazily); b200p_ipc_close unmaps it
 * Each rank owns one flag array of b200p_allreduce_flag_bytes() bytes (zeroed) mapped by every peer. */
#define B200P_AR_MAX_CTAS 1024
int b200p_symm_alloc(void** ptr, size_t bytes);
int b200p_symm_free(void* ptr);
int b200p_ipc_export(void* ptr, void* handle64);
int b200p_ipc_import(const void* handle64, void** ptr);
int b200p_ipc_close(void* ptr);
size_t b200p_allreduce_flag_bytes(void);
/* cap on the exchange grid (0 = auto: the number of CTAs the device can hold at once); tests / tuning */
int b200p_allreduce_set_max_ctas(int n);

/* One-shot all-reduce of the row-parallel partial sums + residual add + the next RMSNorm, one kernel per rank
 *                      [replaces, under TP, the residual adds of models/llama.py:188,190 and the nn.RMSNorm that follows
 *                       (models/llama.py:187,189,231) around a sum over ranks the single-device reference does not need]
 * peer_partial[p] / peer_flags[p]: HOST arrays of `world` device pointers -- rank p's fp32 partial buffer [M, ld_partial]
 * and flag array as mapped in this process (entry `rank` is the local buffer).  h float [M,H] += sum_p partial_p (rank
 * order: bit-identical on all ranks); y `dtype` [M,H] = rms_norm(h, norm_w, eps) (both NULL to skip), optionally PERM8
 * (flags = B200P_OUT_PERM8); zero_buf (local fp32 [M, ld_partial], may be NULL) is zeroed behind the handshake: pass the
 * OTHER partial buffer of a two-buffer rotation (see csrc/allreduce.cu for the protocol and why two buffers suffice).
 * Every rank must issue the same sequence of exchange calls with the same M. */
int b200p_allreduce_residual_rmsnorm(const void* const* peer_partial, void* const* peer_flags, int world, int rank,
                                     float* h, const void* norm_w, void* y, float* zero_buf, int64_t M, int64_t H,
                                     int64_t ld_partial, float eps, int dtype, int flags, void* stream);
/* Two-shot variant with a ROW-SHARDED residual stream (csrc/allreduce.cu): rank r owns rows [r*rpr, (r+1)*rpr), rpr =
 * ceil(M/world); it pulls only its rows of the partials, updates its rows of h (other rows of h go stale on this rank) and
 * pushes rms_norm(h rows) into EVERY rank's x buffer (peer_x[p]: `dtype` [M,H] as mapped here).  1/world of the one-shot
 * traffic; two handshakes.  norm_w is required (x is the product).  Same calling discipline as above. */
int b200p_allreduce_rows_rmsnorm(const void* const* peer_partial, void* const* peer_x, void* const* peer_flags,
                                 int world, int rank, float* h, const void* norm_w, float* zero_buf, int64_t M,
                                 int64_t H, int64_t ld_partial, float eps, int dtype, int flags, void* stream);
/* dst[p * bytes_per_rank ...] = peer p's src block, through peer memory (vocab-parallel greedy head: the W records of
 * b200p_argmax_partial, then b200p_argmax_merge).  bytes_per_rank % 16 == 0. */
int b200p_peer_allgather(const void* const* peer_src, void* const* peer_flags, int world, int rank, void* dst,
                         int64_t bytes_per_rank, void* stream);
/* host_out[0] = 1 if a handshake of this rank ever timed out (a peer stopped), else 0; synchronises `stream` */
int b200p_peer_status(const void* flags_local, uint32_t* host_out, void* stream);

/* ---- dense linear layers, ragged batches, gated delta rule, windowed latent attention ------------------------------------
 * Nothing in the reference corresponds to these (its graphs are Llama-like): they carry decoder designs whose layers mix a
 * recurrent state with a sliding-window attention over a shared low-rank latent.
 *
 * Ragged batch convention: a step brings nb "entries"; entry e owns the packed tokens [cu[e], cu[e+1]) and continues the
 * sequence held in cache row rows[e], whose next position is lengths[rows[e]].  b200p_ragged_plan expands that to
 * per-token arrays; every state-carrying kernel treats position 0 as "no history" (zero state, zero convolution inputs,
 * the first-token bucket), so giving a row back is lengths[row] = 0 and nothing else. */

/* b200p_gemm epilogues */
enum {
  B200P_GEMM_STORE = 0,      /* y[M,N] (dtype) = acc                                                             */
  B200P_GEMM_STORE_F32 = 1,  /* y[M,N] (float) = acc                                                             */
  B200P_GEMM_GLU_CLAMP = 2,  /* rows 2i / 2i+1 of w are gate_i / up_i: y[M,N/2] (dtype) = g * sigmoid(1.702 g) * (u + 1),
                                g = min(gate, limit), u = clamp(up, -limit, limit)                                  */
  B200P_GEMM_GLU_GELU_TANH = 3, /* same row pairs: y = gelu_tanh(gate) * up                                          */
  B200P_GEMM_GLU_SILU = 4,   /* same row pairs: y = gate * sigmoid(gate) * up                                       */
  B200P_GEMM_RELU_SQ = 5     /* y[M,N] (dtype) = max(acc, 0)^2: the hidden units of an ungated feed-forward           */
};
/* y = x . w^T, x [M,K] and w [N,K] in `dtype` (row strides ldx / ldw elements), fp32 accumulation; `batch` independent
 * products at element strides stride_x / stride_w / stride_y.  B200P_F32 runs true fp32 FMAs in ascending k.  16-bit calls
 * with K % 8 == 0 and 16-byte aligned rows take the tensor-core tile kernels (more than 8 rows) or the row-streaming kernel;
 * everything else takes a generic kernel. */
int b200p_gemm(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy,
               int64_t batch, int64_t stride_x, int64_t stride_w, int64_t stride_y, int dtype, int epilogue, float limit,
               void* stream);

/* Grouped product (the experts of a mixture): group z < groups multiplies the rows [seg[z], seg[z+1]) of x (and writes the same
 * rows of y) by its own weight block w + z * stride_w ([N, K]); seg is a DEVICE array of groups + 1 ascending offsets and
 * max_rows an upper bound of a group's row count, which sizes the launch (so the launch does not depend on the routing);
 * total_rows = rows of x and y (seg[groups] <= total_rows).  16-bit calls of more than 64 rows per group run on tcgen05. */
int b200p_gemm_grouped(const void* x, const void* w, void* y, const int32_t* seg, int64_t total_rows, int64_t max_rows, int64_t N, int64_t K,
                       int64_t ldx, int64_t ldw, int64_t ldy, int64_t groups, int64_t stride_w, int dtype, int epilogue,
                       float limit, void* stream);

/* 0 (default): calls of 9 rows and more run on tcgen05 (TMA-fed shared-memory operands, TMEM accumulators; up to 64 rows with the
 * weights on the MMA's M side and K split where the output is narrow, which adds fp32 partial sums in no fixed order) and fall
 * back to the mma.sync kernels for shapes it declines (K < 64); 1: mma.sync kernels only; 2: the same as 0. */
int b200p_gemm_set_path(int path);
/* 0, or 1 + the role (0 loader, 1 MMA issuer, 2 epilogue) whose bounded barrier wait ran out in a tcgen05 dense GEMM since the
 * last call (which clears it).  Synchronises the device. */
int b200p_gemm_tc_fault(void);

/* t_row[t] = rows[e], t_pos[t] = lengths[rows[e]] + (t - cu[e]), t_off[t] = t - cu[e] for the entry e that owns token t */
int b200p_ragged_plan(const int32_t* cu, const int32_t* rows, const int32_t* lengths, int32_t* t_row, int32_t* t_pos,
                      int32_t* t_off, int nb, int64_t M, void* stream);
/* end of a step: lengths[rows[e]] += cu[e+1] - cu[e]; last_token[rows[e]] = ids[cu[e+1] - 1] (entries with no token: nothing) */
int b200p_ragged_advance(int32_t* lengths, int32_t* last_token, const int32_t* ids, const int32_t* cu, const int32_t* rows,
                         int nb, void* stream);
/* h[t,:] (float) = embed[ids[t],:] * scale + bigram[bucket(t),:]; bucket = (prev * mul_prev + ids[t] * mul_cur) mod buckets with
 * prev the token before t in its sequence (ids[t-1] inside a portion, last_token[row] at its start), and row `buckets` of the
 * table at position 0.  bigram may be NULL.  Tables [*, W] in `dtype`. */
int b200p_embed_hashed(const int32_t* ids, const int32_t* t_row, const int32_t* t_pos, const int32_t* t_off,
                       const int32_t* last_token, const void* embed, const void* bigram, float* h, int64_t M, int64_t W,
                       int64_t V, float scale, int64_t buckets, int64_t mul_prev, int64_t mul_cur, int dtype, void* stream);
/* Residual stream with a norm on both sides of a sublayer, one pass per row:
 *   y given:      h += y / sqrt(mean(y^2) + eps) * w_post          (all fp32)
 *   raw_out given: raw_out = h in `dtype`
 *   x_out given:  x_out = h / sqrt(mean(h^2) + eps) * w_next in `dtype`
 * rows [M, W]; weights fp32. */
int b200p_norm_add_norm(const float* y, const float* w_post, float* h, const float* w_next, void* x_out, void* raw_out,
                        int64_t M, int64_t W, float eps, int dtype, void* stream);
/* Residual stream of designs that add their sublayers without a norm of their own, one pass per row:
 *   h += c1 * y1 + c2 * y2 (either may be NULL);  raw_out (rows of stride ld_raw) = h in `dtype`;
 *   x_out = h / sqrt(mean(h^2) + eps) * w_next in `dtype`.  rows [M, W]; h, y, weights fp32. */
int b200p_residual_add_norm(float* h, const float* y1, float c1, const float* y2, float c2, const float* w_next, void* x_out,
                            void* raw_out, int64_t ld_raw, int64_t M, int64_t W, float eps, int dtype, void* stream);
/* dst[t, c] (dtype, row stride ld_dst) = src[t, c] (fp32, row stride ld_src), c < n */
int b200p_cast_columns(const float* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t M, int64_t n, int dtype, void* stream);
/* out[t, c] (dtype) = gelu_tanh(gate[t, c]) * table[ids[t], col0 + c], c < d; gate fp32 [M, d], table [*, ld_table] `dtype` */
int b200p_token_gate(const float* gate, const void* table, const int32_t* ids, void* out, int64_t M, int d, int64_t ld_table,
                     int64_t col0, int dtype, void* stream);

/* Gated delta rule, step 1.  proj fp32 [M, ldp] holds the fused projection [q | k | v | ...]: q, k (KH heads x dk) and
 * v (H heads x dv) are columns [0, C), C = 2 KH dk + H dv; b (H columns) starts at col_b; the decay's step input is `a`
 * (fp32, row stride lda: a slice of proj or a tensor of its own) with decay_per_head values per head: 1 (one decay for the
 * head's whole state) or dk (one per key channel, i.e. per row of the state).  Per channel a causal convolution of `taps` taps (conv_w [C, taps],
 * last column = current token; inputs before position 0 are zero, inputs before the portion come from conv_state
 * [rows, taps-1, C]) then silu; q and k are made unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q times dk^-1/2;
 * beta = sigmoid(b); decay = exp(-exp(A_log[head]) * softplus(a + dt_bias)), dt_bias one per decay.  Outputs fp32: qn, kn
 * [M, KH dk], v [M, H dv], beta [M, H], decay [M, H * decay_per_head]. */
int b200p_delta_prep(const float* proj, int64_t ldp, int64_t col_b, const float* a, int64_t lda, int decay_per_head,
                     const float* conv_w, const float* conv_state,
                     const float* A_log, const float* dt_bias, const int32_t* t_row, const int32_t* t_pos, const int32_t* t_off,
                     float* qn, float* kn, float* v, float* beta, float* decay, int64_t M, int H, int KH, int dk, int dv,
                     int taps, void* stream);
/* step 2 (after b200p_delta_prep of the same step): conv_state of every entry's row takes the last taps-1 inputs */
int b200p_delta_conv_commit(const float* proj, int64_t ldp, float* conv_state, const int32_t* cu, const int32_t* rows, int nb,
                            int64_t C, int taps, void* stream);
/* b200p_delta_scan modes */
enum {
  B200P_SCAN_DELTA = 0,          /* decay [M, H]:      S *= g;          u = beta (v - S^T k); S += k u^T; o = S^T q */
  B200P_SCAN_DELTA_CHANNEL = 1,  /* decay [M, H, dk]:  S = diag(g) S;   then the same                                */
  B200P_SCAN_ACCUMULATE = 2      /* decay [M, H]:      S = g S + k v^T; o = S^T q   (beta may be NULL)               */
};
/* step 3: per entry and head, token by token in fp32, by `mode`.
 * state [rows, H, dk, dv] fp32 is read (zero when the entry starts at position 0) and written back; head h reads q/k head
 * h / (H / KH).  o fp32 [M, H dv]. */
int b200p_delta_scan(const float* qn, const float* kn, const float* v, const float* beta, const float* decay, float* state,
                     const int32_t* cu, const int32_t* rows, const int32_t* lengths, float* o, int nb, int H, int KH, int dk,
                     int dv, int mode, void* stream);
/* step 4: out[t, h, :] (dtype, row stride ld_out) = out_scale * o / sqrt(mean_dv(o^2) + eps) * norm_w * act(gate[t, h, :]);
 * gate fp32 with row stride ldg; gate_act 0 silu, 1 sigmoid.  H == 1 norms the dv values of a row as one group. */
int b200p_delta_out(const float* o, const float* gate, int64_t ldg, const float* norm_w, void* out, int64_t ld_out, int64_t M,
                    int H, int dv, float eps, int gate_act, float out_scale, int dtype, void* stream);
/* Inputs of the plain decayed accumulation (B200P_SCAN_ACCUMULATE): proj fp32 [M, ldp] = [q | k (H x dk each) | v (H x dv)];
 * q, k, v = silu of them (fp32); decay[t, h] = head_decay[h]. */
int b200p_linear_attn_prep(const float* proj, int64_t ldp, const float* head_decay, float* q, float* k, float* v, float* decay,
                           int64_t M, int H, int dk, int dv, void* stream);

/* Attention without a rotation, with grouped heads, a distance bias and a sink.  Step 1: proj fp32 [M, ldp] holds q (H x dk) at
 * col_q, k (G x dk) at col_k, v (G x dv) at col_v.  q_out fp32 [M, H dk] = rms_norm(q) * wq * scale * temperature, temperature
 * = 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) at position p; rms_norm(k) * wk and v go to the caches
 * [rows, G, Tcap, dk] / [rows, G, Tcap, dv] (dtype) at (t_row, t_pos).  wq / wk NULL: no norm. */
int b200p_sink_attn_prep(const float* proj, int64_t ldp, int64_t col_q, int64_t col_k, int64_t col_v, const float* wq,
                         const float* wk, float eps, float scale, float temp_coef, float temp_every, float* q_out, void* kcache,
                         void* vcache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos, int64_t M, int H, int G, int dk,
                         int dv, int dtype, void* stream);
/* step 2: token t at position p of row r sees j <= p; score_j = q . k_j - slope_h (p - j), slope_h = 2^(slope_log2 (h+1) / H)
 * (slope_log2 == 0: no bias); fp32 softmax whose denominator also holds exp(sink[h]) (sink NULL: none);
 * out[t, h, :] (dtype, row stride ld_out) = out_scale * sum_j p_j v_j.  Query head h reads key/value head h / (H / G).
 * With the ragged description (cu, rows, nb entries, the longest of max_n tokens; cu may be NULL) prompts of 16-bit models with
 * key / value sizes of 64 or 128 run on the tensor-core tile kernel, and so do decode steps (max_n == 1, at most 16 query heads
 * per key/value head) when `workspace` (fp32, 16-byte aligned) holds their partial sums; everything else takes the per-token
 * kernel. */
int b200p_sink_attn(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                    const int32_t* t_pos, const int32_t* cu, const int32_t* rows, int nb, int max_n, const float* sink,
                    float slope_log2, void* out, int64_t ld_out, float out_scale, int64_t M, int H, int G, int dk, int dv,
                    int dtype, void* workspace, size_t workspace_bytes, void* stream);
int b200p_sink_attn_tiles_supported(int dk, int dv, int dtype);
/* room for the partial sums of a decode step of nb entries split over the most CTAs the kernel uses (less room: fewer splits) */
size_t b200p_sink_attn_workspace_bytes(int64_t nb, int H, int dv);

/* Routed experts.  logits fp32 [M, ldl] (+ bias [E] or NULL): ids / wts [M, top] = the `top` largest and the softmax over those;
 * seg [E + 1] = offsets of every expert's rows among the M * top slots; slot_of [M * top] the slot of choice k of token t;
 * token_of [M * top] the token of a slot. */
int b200p_moe_route(const float* logits, int64_t ldl, const float* bias, int32_t* ids, float* wts, int32_t* seg, int32_t* slot_of,
                    int32_t* token_of, int64_t M, int E, int top, void* stream);
/* xs[s, :] = x[token_of[s], :], rows of W elements in `dtype` */
int b200p_moe_gather(const void* x, const int32_t* token_of, void* xs, int64_t slots, int64_t W, int dtype, void* stream);
/* The same outputs from sigmoid scores s = sigmoid(logits): experts are picked by s + correction (NULL: none) among the experts of
 * the `keep` best of `count` equal groups of neighbouring experts (a group's score = the sum of its two largest picking scores);
 * wts = the picked experts' s divided by their sum (+ 1e-20), times `scale`.  count == 1 or keep == count: no group limit. */
int b200p_moe_route_sigmoid(const float* logits, int64_t ldl, const float* correction, int32_t* ids, float* wts, int32_t* seg,
                            int32_t* slot_of, int32_t* token_of, int64_t M, int E, int top, int count, int keep, float scale,
                            void* stream);
/* The same outputs from plain sigmoid scores: the `top` largest s = sigmoid(logits) are picked (ties to the smaller index) and
 * wts are those scores as they are, not renormalised. */
int b200p_moe_route_scores(const float* logits, int64_t ldl, int32_t* ids, float* wts, int32_t* seg, int32_t* slot_of,
                           int32_t* token_of, int64_t M, int E, int top, void* stream);
/* xs[slot_of[t, k], :] = wts[t, k] * x[t, :] (fp32 product rounded to `dtype`): routing weights that multiply the experts' inputs */
int b200p_moe_scatter_scaled(const void* x, const int32_t* slot_of, const float* wts, void* xs, int64_t M, int64_t W, int top,
                             int dtype, void* stream);
/* y[t, :] = (shared_y ? g[t] * shared_y[t, :] : 0) + sum_k wts[t, k] * ye[slot_of[t, k], :], all fp32 (wts NULL: weights of one);
 * g[t] = sigmoid(shared_gate[t * ldg]) (shared_gate NULL: 1) */
int b200p_moe_combine(const float* ye, const int32_t* slot_of, const float* wts, const float* shared_y, const float* shared_gate,
                      int64_t ldg, float* y, int64_t M, int64_t W, int top, void* stream);

/* Selective state-space layer around b200p_delta_scan (B200P_SCAN_ACCUMULATE with KH = groups, dk = state).  proj fp32 [M, ldp]
 * holds the channels x (H dv) | B (groups state) | C (groups state) from column col_x on and dt (H) at col_dt.  The channels pass a
 * causal convolution over the sequence (conv_w [C, taps], the last tap the current token's; conv_b [C] or NULL; conv_state
 * [rows, taps-1, C] carries the inputs of earlier steps: commit it afterwards with b200p_delta_conv_commit on the same columns)
 * and silu.  dt = softplus(dt + dt_bias); decay [M, H] = exp(-exp(A_log) dt); xs [M, H dv] = x; v = dt x; kn [M, groups state] = B;
 * qn = C.  All fp32. */
int b200p_ssm_prep(const float* proj, int64_t ldp, int64_t col_x, int64_t col_dt, const float* conv_w, const float* conv_b,
                   const float* conv_state, const float* A_log, const float* dt_bias, const int32_t* t_row, const int32_t* t_pos,
                   const int32_t* t_off, float* xs, float* v, float* kn, float* qn, float* decay, int64_t M, int H, int dv,
                   int groups, int state, int taps, void* stream);
/* y = (o + D[h] xs) * silu(z) (z fp32, row stride ldz; D NULL: no skip term); each of `parts` equal runs of the H dv channels is
 * divided by sqrt(mean(y^2) + eps) over the run; out (dtype, row stride ld_out) = that * norm_w[channel]. */
int b200p_ssm_out(const float* o, const float* xs, const float* z, int64_t ldz, const float* D, const float* norm_w, void* out,
                  int64_t ld_out, int64_t M, int H, int dv, int parts, float eps, int dtype, void* stream);

/* Rotated attention with `maps` (1 or 2) score maps per head.  Step 1: proj fp32 [M, ldp] holds q (H x maps x d) at col_q, k
 * (G x maps x d) at col_k, v (G x dv) at col_v.  In every vector of d the pairs (2i, 2i+1), i < rot_dims / 2, turn by the angle
 * position * rates[i] (rates fp32, on the device); q_out fp32 [M, H maps d] = that * scale; keys and values go to the caches
 * [rows, G, Tcap, maps d] / [rows, G, Tcap, dv] (dtype) at (t_row, t_pos). */
int b200p_rope_attn_prep(const float* proj, int64_t ldp, int64_t col_q, int64_t col_k, int64_t col_v, const float* rates,
                         int rot_dims, float scale, float* q_out, void* kcache, void* vcache, int64_t Tcap, const int32_t* t_row,
                         const int32_t* t_pos, int64_t M, int H, int G, int maps, int d, int dv, int dtype, void* stream);
/* step 2: token t at position p sees j <= p with floor(j / chunk) == floor(p / chunk) (chunk <= 0: all j <= p).  Every map m is a
 * fp32 softmax attention a_m of its own over the same values; o = a_1 (maps == 1) or a_1 - lambda a_2; with eps >= 0 o is divided
 * by sqrt(mean_dv(o^2) + eps); out[t, h, :] (dtype, row stride ld_out) = post * o.  Query head h reads key/value head h / (H / G).
 * cu, rows, nb, max_n describe the ragged batch like b200p_sink_attn; 16-bit caches with d and dv of 32, 64 or 128 run on the
 * tensor-core tile kernel (decode steps when `workspace` holds their partial sums), everything else on the per-token kernel. */
int b200p_diff_attn(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos,
                    const int32_t* cu, const int32_t* rows, int nb, int max_n, int64_t chunk, int maps, float lambda, float eps,
                    float post, void* out, int64_t ld_out, int64_t M, int H, int G, int d, int dv, int dtype, void* workspace,
                    size_t workspace_bytes, void* stream);
size_t b200p_diff_attn_workspace_bytes(int64_t nb, int H, int maps, int dv);
/* y[i] *= s for n fp32 values (the logit scale of designs that have one) */
int b200p_scale(float* y, int64_t n, float s, void* stream);

/* Latent attention, step 1.  proj fp32 [M, ldp] = [down-projected query (q_rank) | down-projected key/value (kv_rank)].
 * cq_out [M, q_rank] (dtype) = rms_norm(query part) * wq; the key/value part, rms_norm * wkv, is written to
 * cache[t_row, t_pos, :] (cache [rows, Tcap, kv_rank] in `dtype`).  kv_rank == 0: a layer that reads another layer's cache. */
int b200p_latent_prep(const float* proj, int64_t ldp, int q_rank, int kv_rank, const float* wq, const float* wkv, float eps,
                      void* cq_out, void* cache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos, int64_t M, int dtype,
                      void* stream);
/* step 2: H heads attend over the ONE latent per position (keys and values both): q fp32 [M, H, R] are the queries already
 * carried into the latent space; token t at position p sees positions j with 0 <= p - j < window (window <= 0: all j <= p);
 * fp32 softmax of q . c_j * scale; out [M, H, R] (dtype) = sum_j p_j c_j.  R <= 1024. */
int b200p_latent_attn(const float* q, const void* cache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos, void* out,
                      int64_t M, int H, int R, int64_t window, float scale, int dtype, void* stream);
/* The same attention on the tensor cores: tiles of 16 consecutive tokens of one entry and one head (max_n = the longest
 * entry's token count), or, when max_n == 1 (a decode step), tiles of 16 heads of each entry's one token; 16-bit types,
 * R % 32 == 0, R <= 512 (b200p_latent_attn_tiles_supported says whether a call
 * qualifies).  q and p are rounded to the storage type for the products; max, sum and the accumulators are fp32. */
int b200p_latent_attn_tiles_supported(int R, int dtype);
/* 16-row tiles (heads of a prompt tile, or blocks of 16 heads of a decode step) that one CTA of the tile kernel serves from one
 * staged copy of the keys: 1..4, or 0 for the built-in choice. */
int b200p_latent_attn_set_groups(int groups);
/* CTAs of a thread-block cluster that share the keys of one decode tile (each a run of 64-key chunks, merged through distributed
 * shared memory): 2, 4 or 8, 1 for one CTA per tile, 0 for the built-in choice (about two CTAs per SM). */
int b200p_latent_attn_set_splits(int splits);
/* Chunk buffers of the tile kernel: 2 = the next 64 latents are in flight while the current ones are multiplied, 1 = one buffer,
 * 0 = the built-in choice (2 where two CTAs per SM still fit beside the buffers). */
int b200p_latent_attn_set_buffers(int buffers);
int b200p_latent_attn_tiles(const float* q, const void* cache, int64_t Tcap, const int32_t* cu, const int32_t* rows,
                            const int32_t* t_pos, void* out, int nb, int max_n, int H, int R, int64_t window, float scale,
                            int dtype, void* stream);


/* Latent attention whose keys also have a rotated part shared by all heads.  Step 1 as b200p_latent_prep with
 * proj = [query (q_rank) | key/value (kv_rank) | rotated key part (rot_dim)]; the cache row ([rows, Tcap, row], row >= kv_rank +
 * rot_dim) becomes [rms-normed latent * wkv | rotated part | zeros]: the pairs (2i, 2i+1) of the rotated part turn by the angle
 * position * rates[i] (fp32) and are multiplied by mag. */
int b200p_latent_rope_prep(const float* proj, int64_t ldp, int q_rank, int kv_rank, int rot_dim, int row, const float* wq,
                           const float* wkv, float eps, const float* rates, float mag, void* cq_out, void* cache, int64_t Tcap,
                           const int32_t* t_row, const int32_t* t_pos, int64_t M, int dtype, void* stream);
/* The queries' rotated part: q [M, H, dim + rot_dim] (dtype); the last rot_dim values of every head turn like the keys' and go,
 * fp32, to q_lat [M, H, row] columns [kv_rank, kv_rank + rot_dim); the columns behind them become zero.  (The columns before
 * them are the query carried into the latent space by a product of the caller's.)  b200p_latent_attn over rows of `row`
 * values then scores q_lat . cache row = unrotated part + rotated part. */
int b200p_latent_q_rope(const void* q, int H, int dim, int rot_dim, int kv_rank, int row, const float* rates, float mag,
                        const int32_t* t_pos, float* q_lat, int64_t M, int dtype, void* stream);

/* Windowed attention with capped scores for designs without rotation.  Step 1: proj fp32 [M, ldp] holds q (H x dk) | k (G x dk)
 * from column col_q; both pass a causal convolution over time (conv_w [taps, (H + G) dk], tap by tap, the last tap the current token's;
 * conv_state [rows, taps-1, (H + G) dk] carries the inputs of earlier steps: commit it afterwards with b200p_delta_conv_commit on the
 * same columns; taps == 1: one factor per channel).  q_out fp32 [M, H dk] = that * scale; the keys go to kcache [rows, G, Tcap, dk]. */
int b200p_window_attn_prep(const float* proj, int64_t ldp, int64_t col_q, const float* conv_w, const float* conv_state, int taps,
                           float scale, float* q_out, void* kcache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos,
                           const int32_t* t_off, int64_t M, int H, int G, int dk, int dtype, void* stream);
/* Step 2: score s = q . k; softcap > 0: s <- softcap tanh(s / softcap); r1, r2 (fp32 [H], or both NULL): s <- s - r1[h] ln(1 +
 * r2[h] (p - j)); the token at position p sees j with 0 <= p - j < window (window 0: every j <= p); fp32 softmax; out[t, h, :]
 * (dtype, row stride ld_out) = sum_j p_j v_j * sigmoid(gate[t * ldg + h dv + c]) (gate fp32, NULL: no gate).  vcache may be kcache
 * (values that are the keys).  The ragged description, the workspace and the choice of kernels are b200p_sink_attn's; the
 * tensor-core tiles take dk == dv of 64 or 128. */
int b200p_window_attn(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                      const int32_t* t_pos, const int32_t* cu, const int32_t* rows, int nb, int max_n, float softcap,
                      const float* r1, const float* r2, int64_t window, const float* gate, int64_t ldg, void* out, int64_t ld_out,
                      int64_t M, int H, int G, int dk, int dv, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Several copies of the residual stream.  xs fp32 [M, streams, W].  One pass over a token closes a sublayer and opens the next:
 *   x'_r = sum_s mix[s, r] x_s + out[r] y   (mix [streams, streams] indexed [from, to], out [streams]; both NULL: x' = x;
 *                                            src [M, W] given: every old copy is src, the start of a model)
 *   sum_out [M, W] (or NULL) = sum_r x'_r
 *   u = sum_r in[r] x'_r;  n = tanh(alpha[0] u) w + b  (w NULL: n = u; b NULL: no offset);  n_out [M, W] (or NULL) = n
 * With x_out (dtype [M, W]) the step is a decode step, one token per entry, and the pass also adds the causal convolution over time
 * of n: x = n + sum_j conv_w[j, :] n_(t - taps + 1 + j) (conv_w fp32 [taps, W], tap by tap) from conv_state [rows, taps-1, W] (inputs
 * before position 0 count as zero),
 * then shifts n into conv_state.  streams <= 8, taps <= 16. */
int b200p_hyper_step(float* xs, const float* y, const float* src, const float* mix, const float* out, const float* in,
                     const float* alpha, const float* w, const float* b, float* n_out, float* sum_out, int64_t M, int streams,
                     int64_t W, const float* conv_w, float* conv_state, const int32_t* t_row, const int32_t* t_pos, int taps,
                     void* x_out, int dtype, void* stream);
/* The same convolution for steps of several tokens per entry: x_out (dtype) = n + conv(n) over the portion's rows of n [M, W] and,
 * before the portion, conv_state (commit it afterwards with b200p_delta_conv_commit on n); conv_w fp32 [taps, W] as above. */
int b200p_canon_conv(const float* n, const float* conv_w, const float* conv_state, const int32_t* t_row, const int32_t* t_pos,
                     const int32_t* t_off, void* x_out, int64_t M, int64_t W, int taps, int dtype, void* stream);
/* x_out (dtype [M, W]) = tanh(alpha[0] h) w + b: the norm without statistics, on given rows */
int b200p_tanh_norm(const float* h, const float* alpha, const float* w, const float* b, void* x_out, int64_t M, int64_t W,
                    int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200P_H */

// Dense 16-bit GEMM on tcgen05: y[M,N] = x[M,K] . w[N,K]^T (+ batch), both operands in shared memory, accumulators in TMEM.
//
//   A = x tile  [128 tokens x 64 k]  K-major, SWIZZLE_128B, filled by TMA          (the M side of the MMA)
//   B = w tile  [BN rows    x 64 k]  K-major, SWIZZLE_128B, filled by TMA          (the N side; BN = 256, 128 or 64)
//   D = [128 x BN] fp32 in TMEM, two buffers: the epilogue of one tile overlaps the main loop of the next
//
// Persistent: CTA c takes tiles c, c + grid, ...; tiles are numbered with the token tile fastest, so the CTAs that run at the
// same time share one weight tile through L2 and the activations (a few tens of MB) stay L2-resident across weight tiles.
//
// warp roles (192 threads):
//   warp 0      TMA producer: x and w tiles of one 64-wide k-block per ring stage (3-d tensor maps: k, row, batch index)
//   warp 1      MMA issuer (one elected lane): four tcgen05.mma (M=128, N=BN, K=16) per stage, tcgen05.commit frees the
//               stage; owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld (thread = token row, 32 columns at a time) -> store / store fp32 / clamped gated unit
//
// Decode batches (17..64 tokens) swap the operands: the weight tile is the 128-row M side, the tokens are the narrow N side
// (BN = 32 or 64), because the MMA reads all 128 rows of its A operand from shared memory whatever they hold, and with the
// tokens there that read (not HBM) bounded the weight stream.  The accumulator then holds y transposed (lane = output column,
// TMEM column = token) and the epilogue stores it back transposed, a warp writing 32 consecutive outputs of one token.  Where
// the weight matrix has too few 128-row tiles to fill the GPU (narrow outputs with long K), K is split over several CTAs that
// add their partial sums into the zeroed fp32 output with red.global.add.
//
// Rows, columns and k outside the tensors are zero-filled by the TMA unit and masked in the epilogue.  Every mbarrier wait is
// bounded: a wait that runs out raises a device flag (reported by the next launch) and the CTA leaves through the common exit,
// which frees its TMEM.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace b200p {

int sm_count();

constexpr int GT_BM = 128, GT_BK = 64, GT_THREADS = 192, GT_EPI_WARP0 = 2;
constexpr int GT_A_BYTES = GT_BM * GT_BK * 2;

__device__ int g_gemm_tc_fault;                   // 0, or 1 + the role that gave up waiting

struct GemmTcParams {
  void* y;
  int64_t M, N, K, ldy, sy;
  int tiles_m, tiles_n, num_tiles, num_kb;
  int splits, kb_per_split;      // K split over `splits` CTAs per output tile (transposed fp32 store only)
  int trans;                     // operands swapped: accumulator row = output column, accumulator column = token
  int epi, vec_ok;
  float limit;
  // grouped products (not with trans): batch index z owns the rows [seg[z], seg[z+1]) of x and y; tiles past a group's rows are
  // skipped by every role alike; seg (device, groups + 1 offsets) is copied to shared memory first
  const int32_t* seg;
  int groups;
};
constexpr int GT_MAX_GROUPS = 1024;

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, 16-bit inputs, fp32 accumulation
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accum)
      : "memory");
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// 32 consecutive accumulator columns of one token row -> y
template <typename T>
__device__ __forceinline__ void gemm_tc_store32(const GemmTcParams& p, int64_t row_off, int64_t n0, const float (&v)[32]) {
  if (p.epi == B200P_GEMM_STORE_F32) {
    float* dst = reinterpret_cast<float*>(p.y) + row_off + n0;
    if (p.vec_ok && n0 + 32 <= p.N) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (n0 + i < p.N) dst[i] = v[i];
    }
  } else if (!gemm_epi_is_glu(p.epi)) {
    float a[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) a[i] = gemm_store_act(v[i], p.epi);
    T* dst = reinterpret_cast<T*>(p.y) + row_off + n0;
    if (p.vec_ok && n0 + 32 <= p.N) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 u;
        u.x = pack2<T>(a[i], a[i + 1]);
        u.y = pack2<T>(a[i + 2], a[i + 3]);
        u.z = pack2<T>(a[i + 4], a[i + 5]);
        u.w = pack2<T>(a[i + 6], a[i + 7]);
        *reinterpret_cast<uint4*>(dst + i) = u;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (n0 + i < p.N) dst[i] = Tr<T>::from_f(a[i]);
    }
  } else {  // gated units: columns 2i / 2i+1 are gate_i / up_i
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) a[i] = glu_unit(v[2 * i], v[2 * i + 1], p.epi, p.limit);
    T* dst = reinterpret_cast<T*>(p.y) + row_off + (n0 >> 1);
    if (p.vec_ok && n0 + 32 <= p.N) {
#pragma unroll
      for (int i = 0; i < 16; i += 8) {
        uint4 u;
        u.x = pack2<T>(a[i], a[i + 1]);
        u.y = pack2<T>(a[i + 2], a[i + 3]);
        u.z = pack2<T>(a[i + 4], a[i + 5]);
        u.w = pack2<T>(a[i + 6], a[i + 7]);
        *reinterpret_cast<uint4*>(dst + i) = u;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (n0 + 2 * i + 1 < p.N) dst[i] = Tr<T>::from_f(a[i]);
    }
  }
}

// Swapped operands: this thread owns output column `n` (a weight row) and holds it for 32 consecutive tokens from `tok0`.
// p.M counts output columns and p.N tokens here.  Gate / up pairs sit in neighbouring lanes.
template <typename T>
__device__ __forceinline__ void gemm_tc_store32_trans(const GemmTcParams& p, int64_t z_off, int64_t n, int64_t tok0, const float (&v)[32]) {
  if (gemm_epi_is_glu(p.epi)) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], 1);
      if (!(threadIdx.x & 1) && n + 1 < p.M && tok0 + i < p.N)
        reinterpret_cast<T*>(p.y)[z_off + (tok0 + i) * p.ldy + (n >> 1)] = Tr<T>::from_f(glu_unit(v[i], other, p.epi, p.limit));
    }
    return;
  }
  if (n >= p.M) return;
  if (p.epi == B200P_GEMM_STORE_F32) {
    float* dst = reinterpret_cast<float*>(p.y) + z_off + n;
    if (p.splits > 1) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (tok0 + i < p.N) atomicAdd(dst + (tok0 + i) * p.ldy, v[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (tok0 + i < p.N) dst[(tok0 + i) * p.ldy] = v[i];
    }
  } else {
    T* dst = reinterpret_cast<T*>(p.y) + z_off + n;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (tok0 + i < p.N) dst[(tok0 + i) * p.ldy] = Tr<T>::from_f(gemm_store_act(v[i], p.epi));
  }
}

struct GemmTcShared {            // lives behind the ring stages (8-byte aligned)
  uint64_t full[10], empty[10], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  volatile int abort;
  int seg[GT_MAX_GROUPS + 1];
};

// rows of group z that tile mt covers: first row in x / y and how many rows the group has; false when the tile is past them
__device__ __forceinline__ bool gemm_tc_group_tile(const GemmTcParams& p, const GemmTcShared* sh, int z, int mt, int& first, int& len) {
  first = 0;
  len = (int)p.M;
  if (!p.seg) return true;
  first = sh->seg[z];
  len = sh->seg[z + 1] - first;
  return mt * GT_BM < len;
}

// bounded wait: gives up after about a second, or as soon as another role of the CTA has given up
__device__ __forceinline__ bool gemm_tc_wait(uint32_t bar, uint32_t parity, GemmTcShared* sh, int role) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if (sh->abort) return false;
    if (clock64() - t0 > 2000000000ll) {
      sh->abort = 1;
      atomicCAS(&g_gemm_tc_fault, 0, 1 + role);
      return false;
    }
  }
}

template <typename T, int BN, int STAGES>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmw, const GemmTcParams p) {
  constexpr int B_BYTES = BN * GT_BK * 2, STAGE_BYTES = GT_A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;           // 64 .. 512: a power of two >= 32
  static_assert(STAGES <= 10 && (BN == 32 || BN == 64 || BN == 128 || BN == 256), "ring / tile shape");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;    // SWIZZLE_128B tiles start on 1024-byte boundaries
  GemmTcShared* sh = reinterpret_cast<GemmTcShared*>(smem_raw + (base - raw) + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&sh->acc_full[a]), 1);
      mbar_init(smem_u32(&sh->acc_empty[a]), 4);   // one arrival per epilogue warp
    }
    sh->abort = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmx);
    tma_prefetch_desc(&tmw);
  }
  if (warp == 1) tmem_alloc(smem_u32(&sh->tmem_base), TMEM_COLS);
  if (p.seg)
    for (int i = threadIdx.x; i <= p.groups; i += blockDim.x) sh->seg[i] = p.seg[i];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const int per_batch = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        const int ts = t / p.splits, kb0 = (t - ts * p.splits) * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        const int z = ts / per_batch, r = ts - z * per_batch;
        const int nt = r / p.tiles_m, mt = r - nt * p.tiles_m;
        int first, len;
        if (!gemm_tc_group_tile(p, sh, z, mt, first, len)) continue;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!(ok = gemm_tc_wait(smem_u32(&sh->empty[stage]), phase ^ 1u, sh, 0))) break;
          const uint32_t bar = smem_u32(&sh->full[stage]);
          const uint32_t dst = base + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(bar, STAGE_BYTES);
          tma_load_3d(dst, &tmx, kb * GT_BK, first + mt * GT_BM, p.seg ? 0 : z, bar);
          tma_load_3d(dst + GT_A_BYTES, &tmw, kb * GT_BK, nt * BN, z, bar);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(GT_BM >> 4) << 24);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        if (p.seg) {
          const int ts = t / p.splits, z = ts / per_batch, r = ts - z * per_batch;
          int first, len;
          if (!gemm_tc_group_tile(p, sh, z, r % p.tiles_m, first, len)) continue;
        }
        if (!(ok = gemm_tc_wait(smem_u32(&sh->acc_empty[acc]), acc_phase ^ 1u, sh, 1))) break;
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(acc * BN);
        const int kb0 = (t % p.splits) * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!(ok = gemm_tc_wait(smem_u32(&sh->full[stage]), phase, sh, 1))) break;
          tc_fence_after();
          const uint64_t ad = make_desc_sw128(base + stage * STAGE_BYTES);
          const uint64_t bd = make_desc_sw128(base + stage * STAGE_BYTES + GT_A_BYTES);
#pragma unroll
          for (int k = 0; k < GT_BK / 16; ++k)     // 16 k = 32 bytes = 2 descriptor units inside the swizzle atom
            umma_f16_ss(d, ad + 2u * k, bd + 2u * k, idesc, ((kb - kb0) | k) ? 1u : 0u);
          umma_commit(smem_u32(&sh->empty[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&sh->acc_full[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    const int lg = warp & 3;                       // the TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
      const int ts = t / p.splits;
      const int z = ts / per_batch, r = ts - z * per_batch;
      const int nt = r / p.tiles_m, mt = r - nt * p.tiles_m;
      int first, len;
      if (!gemm_tc_group_tile(p, sh, z, mt, first, len)) continue;
      if (!gemm_tc_wait(smem_u32(&sh->acc_full[acc]), acc_phase, sh, 2)) break;
      tc_fence_after();
      const int64_t row = (int64_t)mt * GT_BM + lg * 32 + lane;               // within the batch index's (group's) rows
      const int64_t row_off = p.seg ? (first + row) * p.ldy : (int64_t)z * p.sy + row * p.ldy;
      const uint32_t tsrc = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        const int64_t n0 = (int64_t)nt * BN + c;
        if (n0 >= p.N) break;                      // warp-uniform
        float v[32];
        tmem_ld16(tsrc + c, *reinterpret_cast<float(*)[16]>(&v[0]));
        tmem_ld16(tsrc + c + 16, *reinterpret_cast<float(*)[16]>(&v[16]));
        tmem_ld_wait();
        if (p.trans) gemm_tc_store32_trans<T>(p, (int64_t)z * p.sy, row, n0, v);
        else if (row < len) gemm_tc_store32<T>(p, row_off, n0, v);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------ host
static TcEncodeFn gemm_tc_encode_fn() {
  static TcEncodeFn fn = nullptr;
  if (!fn) {
    void* q = nullptr;
    cudaDriverEntryPointQueryResult r;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess && r == cudaDriverEntryPointSuccess)
      fn = (TcEncodeFn)q;
  }
  return fn;
}

// [batch][rows][K] 16-bit tensor, box = 64 k x box_rows rows of one batch index, SWIZZLE_128B
static bool gemm_tc_map(TcEncodeFn enc, CUtensorMap* tm, CUtensorMapDataType dt, const void* base, int64_t K, int64_t rows,
                        int64_t batch, int64_t ld, int64_t stride, int box_rows) {
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? stride : ld * rows) * 2};
  cuuint32_t box[3] = {(cuuint32_t)GT_BK, (cuuint32_t)box_rows, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  return enc(tm, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int BN, int STAGES>
static int gemm_tc_run(const CUtensorMap& tmx, const CUtensorMap& tmw, GemmTcParams p, cudaStream_t st) {
  constexpr size_t smem = 1024 + (size_t)STAGES * (GT_A_BYTES + BN * GT_BK * 2) + sizeof(GemmTcShared);
  auto kern = gemm_tc_kernel<T, BN, STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm_tc_kernel)");
    attr_set = true;
  }
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  kern<<<grid, GT_THREADS, smem, st>>>(tmx, tmw, p);
  B200P_LAUNCH_CHECK("gemm_tc_kernel");
  return B200P_OK;
}

// Up to 64 tokens: weights on the M side, tokens on the N side, transposed store, K split where the output is narrow.
template <typename T>
static int gemm_tc_launch_decode(TcEncodeFn enc, const T* x, const T* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw,
                                 int64_t ldy, int64_t batch, int64_t sx, int64_t sw, int64_t sy, int epi, float limit, cudaStream_t st) {
  const CUtensorMapDataType dt = std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int bn = M <= 32 ? 32 : 64;
  CUtensorMap tma, tmb;                            // A = weights (128-row boxes), B = tokens (bn-row boxes)
  if (!gemm_tc_map(enc, &tma, dt, w, K, N, batch, ldw, sw, GT_BM)) return 1;
  if (!gemm_tc_map(enc, &tmb, dt, x, K, M, batch, ldx, sx, bn)) return 1;
  GemmTcParams p;
  p.y = y;
  p.M = N; p.N = M; p.K = K; p.ldy = ldy; p.sy = sy;
  p.tiles_m = (int)((N + GT_BM - 1) / GT_BM);
  p.tiles_n = 1;
  p.num_kb = (int)((K + GT_BK - 1) / GT_BK);
  const int64_t tiles = (int64_t)p.tiles_m * batch;
  if (tiles >= (1ll << 24)) return 1;
  // few weight tiles and a long K: split K so that about one CTA per SM streams weights, at least 4 k-blocks each
  int splits = 1;
  if (epi == B200P_GEMM_STORE_F32 && batch == 1 && ldy == N && tiles * 2 <= sm_count()) {
    splits = (int)min((int64_t)(sm_count() / tiles), (int64_t)(p.num_kb / 4));
    if (splits < 1) splits = 1;
  }
  p.kb_per_split = (p.num_kb + splits - 1) / splits;
  p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;          // no empty split
  p.num_tiles = (int)(tiles * p.splits);
  p.trans = 1;
  p.seg = nullptr;
  p.groups = 0;
  p.epi = epi;
  p.limit = limit;
  p.vec_ok = 0;
  if (p.splits > 1) {
    cudaError_t e = cudaMemsetAsync(y, 0, (size_t)M * N * sizeof(float), st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(split-K output)");
  }
  if (bn == 32) return gemm_tc_run<T, 32, 10>(tma, tmb, p, st);
  return gemm_tc_run<T, 64, 8>(tma, tmb, p, st);
}

// Returns B200P_OK, an error, or 1 when the shape is not one this kernel takes (the caller then runs the mma.sync kernel).
template <typename T>
int gemm_tc_launch(const T* x, const T* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy,
                   int64_t batch, int64_t sx, int64_t sw, int64_t sy, int epi, float limit, cudaStream_t st) {
  if (K < GT_BK || M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return 1;
  TcEncodeFn enc = gemm_tc_encode_fn();
  if (!enc) return 1;
  if (M <= 64) return gemm_tc_launch_decode<T>(enc, x, w, y, M, N, K, ldx, ldw, ldy, batch, sx, sw, sy, epi, limit, st);
  const int tiles_m = (int)((M + GT_BM - 1) / GT_BM);
  // widest weight tile that still gives every SM about two tiles
  const int64_t want = 2ll * sm_count();
  int bn = 256;
  if (N <= 64 || tiles_m * ((N + 127) / 128) * batch < want) bn = 64;
  else if (N <= 128 || tiles_m * ((N + 255) / 256) * batch < want) bn = 128;
  const CUtensorMapDataType dt = std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tmx, tmw;
  if (!gemm_tc_map(enc, &tmx, dt, x, K, M, batch, ldx, sx, GT_BM)) return 1;
  if (!gemm_tc_map(enc, &tmw, dt, w, K, N, batch, ldw, sw, bn)) return 1;
  GemmTcParams p;
  p.y = y;
  p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.sy = sy;
  p.tiles_m = tiles_m;
  p.tiles_n = (int)((N + bn - 1) / bn);
  const int64_t nt = (int64_t)p.tiles_m * p.tiles_n * batch;
  if (nt >= (1ll << 31)) return 1;
  p.num_tiles = (int)nt;
  p.num_kb = (int)((K + GT_BK - 1) / GT_BK);
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.trans = 0;
  p.seg = nullptr;
  p.groups = 0;
  p.epi = epi;
  p.limit = limit;
  const int64_t eb = epi == B200P_GEMM_STORE_F32 ? 4 : 2;
  p.vec_ok = aligned(y, 16) && (ldy * eb) % 16 == 0 && (sy * eb) % 16 == 0;
  if (bn == 256) return gemm_tc_run<T, 256, 4>(tmx, tmw, p, st);
  if (bn == 128) return gemm_tc_run<T, 128, 6>(tmx, tmw, p, st);
  return gemm_tc_run<T, 64, 8>(tmx, tmw, p, st);
}

// Grouped product: x [total_rows, K] holds the groups' rows back to back (group z: rows [seg[z], seg[z+1]), at most max_rows of
// them), w [groups][N][K].  The tile list covers max_rows rows for every group; tiles past a group's rows cost a shared-memory
// read.  A tile's 128-row box may reach into the next group's rows (or past the tensor, which reads zeros): those accumulator
// rows are not stored.
template <typename T>
int gemm_tc_launch_grouped(const T* x, const T* w, void* y, const int32_t* seg, int64_t total_rows, int64_t max_rows, int64_t N,
                           int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int64_t groups, int64_t sw, int epi, float limit,
                           cudaStream_t st) {
  if (K < GT_BK || total_rows >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31) || groups > GT_MAX_GROUPS) return 1;
  TcEncodeFn enc = gemm_tc_encode_fn();
  if (!enc) return 1;
  const int bn = N <= 64 ? 64 : N <= 128 ? 128 : 256;
  const CUtensorMapDataType dt = std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tmx, tmw;
  if (!gemm_tc_map(enc, &tmx, dt, x, K, total_rows, 1, ldx, 0, GT_BM)) return 1;
  if (!gemm_tc_map(enc, &tmw, dt, w, K, N, groups, ldw, sw, bn)) return 1;
  GemmTcParams p;
  p.y = y;
  p.M = max_rows; p.N = N; p.K = K; p.ldy = ldy; p.sy = 0;
  p.tiles_m = (int)((max_rows + GT_BM - 1) / GT_BM);
  p.tiles_n = (int)((N + bn - 1) / bn);
  const int64_t nt = (int64_t)p.tiles_m * p.tiles_n * groups;
  if (nt >= (1ll << 31)) return 1;
  p.num_tiles = (int)nt;
  p.num_kb = (int)((K + GT_BK - 1) / GT_BK);
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.trans = 0;
  p.seg = seg;
  p.groups = (int)groups;
  p.epi = epi;
  p.limit = limit;
  const int64_t eb = epi == B200P_GEMM_STORE_F32 ? 4 : 2;
  p.vec_ok = aligned(y, 16) && (ldy * eb) % 16 == 0;
  if (bn == 256) return gemm_tc_run<T, 256, 4>(tmx, tmw, p, st);
  if (bn == 128) return gemm_tc_run<T, 128, 6>(tmx, tmw, p, st);
  return gemm_tc_run<T, 64, 8>(tmx, tmw, p, st);
}
template int gemm_tc_launch_grouped<__half>(const __half*, const __half*, void*, const int32_t*, int64_t, int64_t, int64_t, int64_t, int64_t,
                                            int64_t, int64_t, int64_t, int64_t, int, float, cudaStream_t);
template int gemm_tc_launch_grouped<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*, void*, const int32_t*, int64_t, int64_t,
                                                   int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, float, cudaStream_t);

template int gemm_tc_launch<__half>(const __half*, const __half*, void*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                                    int64_t, int64_t, int64_t, int64_t, int, float, cudaStream_t);
template int gemm_tc_launch<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*, void*, int64_t, int64_t, int64_t, int64_t,
                                           int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, float, cudaStream_t);

}  // namespace b200p

// 0, or 1 + the role (0 loader, 1 MMA issuer, 2 epilogue) of the first wait of a tcgen05 dense GEMM that ran out; reading
// clears it.  Synchronises the device.
extern "C" int b200p_gemm_tc_fault(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, b200p::g_gemm_tc_fault, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(b200p::g_gemm_tc_fault, &zero, sizeof(int));
  return v;
}

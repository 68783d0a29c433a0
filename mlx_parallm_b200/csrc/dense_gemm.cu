// Dense (unquantised) linear layers: y[M,N] = x[M,K] . w[N,K]^T with fp32 accumulation, optionally batched over a leading
// index (one weight block per attention head).  Five kernels behind b200p_gemm:
//   gemm_tc_kernel     16-bit operands, tcgen05 / TMA / TMEM (dense_gemm_tc.cu)                             (9 rows and more)   
//   gemm_mma_kernel    16-bit operands, mma.sync m16n8k16 over cp.async-staged tiles, two tile shapes      (K < 64, or on request)
//   gemm_stream_kernel 16-bit operands, weights streamed from global memory straight into MMA fragments    (9..64 rows where tcgen05 declines)
//   gemv_rows_kernel   16-bit operands, a warp per pair of weight rows, 128-bit streaming                  (up to 8 rows)
//   gemm_simt_kernel   any operand type and any shape or alignment; true fp32 FMA in ascending k for float32 models
// Epilogues: store in the storage type, store fp32, and the clamped gated unit of b200p.h (gate / up rows interleaved).
#include <type_traits>

#include "common.cuh"
#include "mma_util.cuh"

namespace b200p {

// dense_gemm_tc.cu: B200P_OK, an error, or 1 = "not a shape for the tcgen05 kernel"
template <typename T>
int gemm_tc_launch(const T* x, const T* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy,
                   int64_t batch, int64_t sx, int64_t sw, int64_t sy, int epi, float limit, cudaStream_t st);
template <typename T>
int gemm_tc_launch_grouped(const T* x, const T* w, void* y, const int32_t* seg, int64_t total_rows, int64_t max_rows, int64_t N,
                           int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int64_t groups, int64_t sw, int epi, float limit,
                           cudaStream_t st);
// 0: tcgen05 from 9 rows up (its decode variant streams the weights 1.0-2.3x faster than gemm_stream_kernel at 16 rows, 1.1-2.6x at
//    32, 1.6-4.4x at 64), the mma.sync kernels where it declines; 1: mma.sync kernels only; 2: the same as 0
static int g_gemm_path = 0;

// ---- epilogue -------------------------------------------------------------------------------------------------------
// value pair (even column n, odd column n+1) of one output row
template <typename T>
__device__ __forceinline__ void gemm_store_pair(void* y, int64_t row_off, int64_t n, int64_t N, float v0, float v1, int epi,
                                                float limit) {
  if (epi == B200P_GEMM_STORE_F32) {
    float* p = reinterpret_cast<float*>(y) + row_off;
    if (n < N) p[n] = v0;
    if (n + 1 < N) p[n + 1] = v1;
  } else if (!gemm_epi_is_glu(epi)) {
    T* p = reinterpret_cast<T*>(y) + row_off;
    if (n < N) p[n] = Tr<T>::from_f(gemm_store_act(v0, epi));
    if (n + 1 < N) p[n + 1] = Tr<T>::from_f(gemm_store_act(v1, epi));
  } else {  // gated units: v0 = gate, v1 = up of hidden unit n / 2
    if (n + 1 < N) reinterpret_cast<T*>(y)[row_off + (n >> 1)] = Tr<T>::from_f(glu_unit(v0, v1, epi, limit));
  }
}

// Grouped calls (a mixture of experts: group z owns the rows [seg[z], seg[z+1]) of x and y and the z-th weight block): the row
// count and the row offsets of a CTA's product come from the device array instead of the launch, so the launch is the same
// whatever the routing (and can sit in a captured graph).  Without `seg` the products are `batch` equal ones at fixed strides.
#define GEMM_GROUP_ROWS(seg, z, M, x, ldx, sx, ybase, ldy, sy) \
  int64_t ybase;                                                \
  if (seg) {                                                    \
    const int64_t s0__ = seg[z];                                \
    M = seg[z + 1] - s0__;                                      \
    x += s0__ * ldx;                                            \
    ybase = s0__ * ldy;                                         \
  } else {                                                      \
    x += z * sx;                                                \
    ybase = z * sy;                                             \
  }

// ---- generic kernel ---------------------------------------------------------------------------------------------------
constexpr int GS_BM = 64, GS_BN = 64, GS_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ y, int64_t M, int64_t N, int64_t K,
                 int64_t ldx, int64_t ldw, int64_t ldy, int64_t sx, int64_t sw, int64_t sy, int epi, float limit,
                 const int32_t* __restrict__ seg) {
  __shared__ float xs[GS_BK][GS_BM + 4];
  __shared__ float ws[GS_BK][GS_BN + 4];
  const int64_t z = blockIdx.z;
  GEMM_GROUP_ROWS(seg, z, M, x, ldx, sx, ybase, ldy, sy);
  w += z * sw;
  const int64_t m0 = (int64_t)blockIdx.y * GS_BM, n0 = (int64_t)blockIdx.x * GS_BN;
  if (m0 >= M) return;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // 4 x 4 outputs: rows ty*4.., columns tx*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int64_t k0 = 0; k0 < K; k0 += GS_BK) {
    for (int idx = threadIdx.x; idx < GS_BM * GS_BK; idx += 256) {
      const int r = idx / GS_BK, c = idx % GS_BK;
      const int64_t m = m0 + r, k = k0 + c;
      xs[c][r] = (m < M && k < K) ? Tr<T>::to_f(x[m * ldx + k]) : 0.f;
      const int64_t n = n0 + r;
      ws[c][r] = (n < N && k < K) ? Tr<T>::to_f(w[n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < GS_BK; ++c) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[c][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[c][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= M) continue;
    const int64_t off = ybase + m * ldy;
#pragma unroll
    for (int j = 0; j < 4; j += 2) gemm_store_pair<T>(y, off, n0 + tx * 4 + j, N, acc[i][j], acc[i][j + 1], epi, limit);
  }
}

// ---- tensor-core tile kernel (16-bit operands) ---------------------------------------------------------------------------
// WM x WN warps, each a WTM x WTN output block (multiples of 16), k tiles of BK staged by cp.async STAGES deep.  Two shapes
// are instantiated: 128 x 128 (warp blocks of 64 x 64: four MMAs per ldmatrix) for prompts and 64 x 64 when that grid would
// not fill the GPU.
constexpr int GM_PAD = 8;

template <typename T, int WM, int WN, int WTM, int WTN, int BK, int STAGES>
__global__ void __launch_bounds__(WM * WN * 32)
gemm_mma_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ y, int64_t M, int64_t N, int64_t K,
                int64_t ldx, int64_t ldw, int64_t ldy, int64_t sx, int64_t sw, int64_t sy, int epi, float limit,
                const int32_t* __restrict__ seg) {
  constexpr int BM = WM * WTM, BN = WN * WTN, NT = WM * WN * 32, LDS = BK + GM_PAD, MI = WTM / 16, NJ = WTN / 8;
  static_assert(WTM % 16 == 0 && WTN % 16 == 0 && BK % 16 == 0, "warp blocks are made of 16 x 16 pieces");
  extern __shared__ __align__(128) uint8_t smem_raw[];
  T* xs = reinterpret_cast<T*>(smem_raw);                       // [STAGES][BM][LDS]
  T* ws = xs + STAGES * BM * LDS;                               // [STAGES][BN][LDS]
  const int64_t z = blockIdx.z;
  GEMM_GROUP_ROWS(seg, z, M, x, ldx, sx, ybase, ldy, sy);
  w += z * sw;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  if (m0 >= M) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp / WN, wn = warp % WN;
  const int nk = (int)((K + BK - 1) / BK);

  auto issue = [&](int kt, int stage) {
    const int64_t k0 = (int64_t)kt * BK;
    T* xd = xs + stage * BM * LDS;
    T* wd = ws + stage * BN * LDS;
    for (int idx = threadIdx.x; idx < BM * (BK / 8); idx += NT) {
      const int r = idx / (BK / 8), c = (idx % (BK / 8)) * 8;
      const bool ok = (m0 + r < M) && (k0 + c < K);
      cp_async16((uint32_t)__cvta_generic_to_shared(xd + r * LDS + c), ok ? (const void*)(x + (m0 + r) * ldx + k0 + c) : (const void*)x, ok);
    }
    for (int idx = threadIdx.x; idx < BN * (BK / 8); idx += NT) {
      const int r = idx / (BK / 8), c = (idx % (BK / 8)) * 8;
      const bool ok = (n0 + r < N) && (k0 + c < K);
      cp_async16((uint32_t)__cvta_generic_to_shared(wd + r * LDS + c), ok ? (const void*)(w + (n0 + r) * ldw + k0 + c) : (const void*)w, ok);
    }
  };

  float acc[MI][NJ][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) issue(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (kt + STAGES - 1 < nk) issue(kt + STAGES - 1, (kt + STAGES - 1) % STAGES);
    cp_async_commit();
    const T* xt = xs + (kt % STAGES) * BM * LDS;
    const T* wt = ws + (kt % STAGES) * BN * LDS;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t a[MI][4], b[NJ / 2][4];
#pragma unroll
      for (int i = 0; i < MI; ++i)
        ldsm_x4((uint32_t)__cvta_generic_to_shared(xt + (wm * WTM + i * 16 + (lane & 15)) * LDS + kk + (lane >> 4) * 8), a[i]);
#pragma unroll
      for (int j = 0; j < NJ / 2; ++j)
        ldsm_x4((uint32_t)__cvta_generic_to_shared(wt + (wn * WTN + j * 16 + (lane & 7) + (lane >> 4) * 8) * LDS + kk + ((lane >> 3) & 1) * 8),
                b[j]);
#pragma unroll
      for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j) mma16816<T>(acc[i][j], a[i], b[j >> 1][(j & 1) * 2], b[j >> 1][(j & 1) * 2 + 1]);
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int64_t m = m0 + wm * WTM + i * 16 + (lane >> 2) + hf * 8;
      if (m >= M) continue;
      const int64_t off = ybase + m * ldy;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        gemm_store_pair<T>(y, off, n0 + wn * WTN + j * 8 + (lane & 3) * 2, N, acc[i][j][hf * 2], acc[i][j][hf * 2 + 1], epi, limit);
    }
}

template <typename T, int WM, int WN, int WTM, int WTN, int BK, int STAGES>
static int gemm_mma_launch(const T* x, const T* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy,
                           int64_t batch, int64_t sx, int64_t sw, int64_t sy, int epi, float limit, cudaStream_t st,
                           const int32_t* seg = nullptr) {
  constexpr int BM = WM * WTM, BN = WN * WTN;
  constexpr size_t smem = (size_t)STAGES * (BM + BN) * (BK + GM_PAD) * sizeof(T);
  auto kern = gemm_mma_kernel<T, WM, WN, WTM, WTN, BK, STAGES>;
  if (smem > 48 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm_mma_kernel)");
      attr_set = true;
    }
  }
  dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM), (unsigned)batch);
  kern<<<grid, WM * WN * 32, smem, st>>>(x, w, y, M, N, K, ldx, ldw, ldy, sx, sw, sy, epi, limit, seg);
  B200P_LAUNCH_CHECK("gemm_mma_kernel");
  return B200P_OK;
}

// ---- few rows (decode): the weights stream once, every warp owns two weight rows ---------------------------------------------
constexpr int GEMV_MAX_M = 8;

template <typename T, int MR>
__global__ void __launch_bounds__(256)
gemv_rows_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ y, int M, int64_t N, int64_t K, int64_t ldx,
                 int64_t ldw, int64_t ldy, int64_t sx, int64_t sw, int64_t sy, int epi, float limit) {
  const int64_t z = blockIdx.z;
  x += z * sx;
  w += z * sw;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n = ((int64_t)blockIdx.x * 8 + warp) * 2;
  if (n >= N) return;
  const bool two = n + 1 < N;
  float a0[MR], a1[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) a0[m] = a1[m] = 0.f;
  const T* w0 = w + n * ldw;
  const T* w1 = w + (two ? n + 1 : n) * ldw;
  for (int64_t k = (int64_t)lane * 8; k < K; k += 256) {
    const uint4 u0 = ldg_stream(w0 + k), u1 = ldg_stream(w1 + k);
    const T* p0 = reinterpret_cast<const T*>(&u0);
    const T* p1 = reinterpret_cast<const T*>(&u1);
    float f0[8], f1[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      f0[e] = Tr<T>::to_f(p0[e]);
      f1[e] = Tr<T>::to_f(p1[e]);
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      if (m < M) {
        const uint4 ux = *reinterpret_cast<const uint4*>(x + (int64_t)m * ldx + k);
        const T* px = reinterpret_cast<const T*>(&ux);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xv = Tr<T>::to_f(px[e]);
          a0[m] = fmaf(xv, f0[e], a0[m]);
          a1[m] = fmaf(xv, f1[e], a1[m]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MR; ++m) {
    a0[m] = warp_sum(a0[m]);
    a1[m] = warp_sum(a1[m]);
  }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MR; ++m)
      if (m < M) gemm_store_pair<T>(y, z * sy + (int64_t)m * ldy, n, N, a0[m], a1[m], epi, limit);
  }
}

// ---- decode batches (9..64 rows): weights stream straight from global memory into MMA fragments ----------------------------
// A CTA owns 16 weight rows (two n8 tiles) and splits K over its 8 warps (2 n-tiles x 4 k-slices); a warp walks its slice 32
// elements at a time: every lane loads 16 contiguous bytes of "its" weight row (row lane/4, the quarter lane%4 of the 32) and
// the same 16 bytes of its activation rows, and uses them as the k pairs of two m16n8k16 MMAs.  The MMA sums over k in whatever
// order the pairs are presented, as long as A and B present the same one, so no shared memory, ldmatrix or transposition is
// needed and every row is read in 64-byte pieces.  The four k-slices are summed through shared memory in a fixed order.
constexpr int GK_SLICES = 4, GK_THREADS = 256;

template <typename T, int MT>     // MT m16 tiles: rows <= 16 * MT
__global__ void __launch_bounds__(GK_THREADS)
gemm_stream_kernel(const T* __restrict__ x, const T* __restrict__ w, void* __restrict__ y, int M, int64_t N, int64_t K, int64_t ldx,
                   int64_t ldw, int64_t ldy, int64_t sx, int64_t sw, int64_t sy, int epi, float limit,
                   const int32_t* __restrict__ seg) {
  __shared__ float red[GK_SLICES][2][MT][32][4];
  const int64_t z = blockIdx.z;
  GEMM_GROUP_ROWS(seg, z, M, x, ldx, sx, ybase, ldy, sy);
  if (M <= 0) return;                                            // a group nobody was routed to: its weights are not read
  w += z * sw;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = warp & 1, ks = warp >> 1;
  const int64_t n_row = (int64_t)blockIdx.x * 16 + nt * 8 + (lane >> 2);
  const bool n_ok = n_row < N;
  const T* wp = w + (n_ok ? n_row : 0) * ldw + (lane & 3) * 8;
  const T* xp[MT][2];
  bool x_ok[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int m = i * 16 + (lane >> 2) + hf * 8;
      x_ok[i][hf] = m < M;
      xp[i][hf] = x + (int64_t)(x_ok[i][hf] ? m : 0) * ldx + (lane & 3) * 8;
    }
  float acc[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  // slice ks takes the 32-element blocks ks, ks + 4, ...: neighbouring warps read neighbouring 64-byte pieces of a row
#pragma unroll 4
  for (int64_t k = (int64_t)ks * 32; k < K; k += 32 * GK_SLICES) {
    const bool k_ok = k + (lane & 3) * 8 < K;                    // K % 8 == 0: a 16-byte piece is inside or outside
    uint4 b = make_uint4(0, 0, 0, 0);
    if (n_ok && k_ok) b = ldg_stream(wp + k);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      uint4 a0 = make_uint4(0, 0, 0, 0), a1 = make_uint4(0, 0, 0, 0);
      if (x_ok[i][0] && k_ok) a0 = *reinterpret_cast<const uint4*>(xp[i][0] + k);
      if (x_ok[i][1] && k_ok) a1 = *reinterpret_cast<const uint4*>(xp[i][1] + k);
      const uint32_t f0[4] = {a0.x, a1.x, a0.y, a1.y}, f1[4] = {a0.z, a1.z, a0.w, a1.w};
      mma16816<T>(acc[i], f0, b.x, b.y);
      mma16816<T>(acc[i], f1, b.z, b.w);
    }
  }
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[ks][nt][i][lane][e] = acc[i][e];
  __syncthreads();
  if (ks != 0) return;
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = ((red[0][nt][i][lane][e] + red[1][nt][i][lane][e]) + red[2][nt][i][lane][e]) + red[3][nt][i][lane][e];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int m = i * 16 + (lane >> 2) + hf * 8;
      if (m < M)
        gemm_store_pair<T>(y, ybase + (int64_t)m * ldy, (int64_t)blockIdx.x * 16 + nt * 8 + (lane & 3) * 2, N, v[hf * 2], v[hf * 2 + 1],
                           epi, limit);
    }
  }
}

template <typename T>
static int gemm_dispatch(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw,
                         int64_t ldy, int64_t batch, int64_t sx, int64_t sw, int64_t sy, int epi, float limit, bool fast_ok,
                         cudaStream_t st) {
  const T* xp = (const T*)x;
  const T* wp = (const T*)w;
  if (fast_ok && M <= GEMV_MAX_M) {
    dim3 grid((unsigned)((N + 15) / 16), 1, (unsigned)batch);
    if (M <= 2) gemv_rows_kernel<T, 2><<<grid, 256, 0, st>>>(xp, wp, y, (int)M, N, K, ldx, ldw, ldy, sx, sw, sy, epi, limit);
    else if (M <= 4) gemv_rows_kernel<T, 4><<<grid, 256, 0, st>>>(xp, wp, y, (int)M, N, K, ldx, ldw, ldy, sx, sw, sy, epi, limit);
    else gemv_rows_kernel<T, 8><<<grid, 256, 0, st>>>(xp, wp, y, (int)M, N, K, ldx, ldw, ldy, sx, sw, sy, epi, limit);
    B200P_LAUNCH_CHECK("gemv_rows_kernel");
    return B200P_OK;
  }
  if (fast_ok) {
    if constexpr (!std::is_same<T, float>::value) {
      if (M <= 64 && g_gemm_path != 1) {
        const int rc = gemm_tc_launch<T>(xp, wp, y, M, N, K, ldx, ldw, ldy, batch, sx, sw, sy, epi, limit, st);
        if (rc != 1) return rc;
      }
    }
    if (M <= 64) {
      dim3 grid((unsigned)((N + 15) / 16), 1, (unsigned)batch);
      if (M <= 16) gemm_stream_kernel<T, 1><<<grid, GK_THREADS, 0, st>>>(xp, wp, y, (int)M, N, K, ldx, ldw, ldy, sx, sw, sy, epi, limit, nullptr);
      else if (M <= 32) gemm_stream_kernel<T, 2><<<grid, GK_THREADS, 0, st>>>(xp, wp, y, (int)M, N, K, ldx, ldw, ldy, sx, sw, sy, epi, limit, nullptr);
      else gemm_stream_kernel<T, 4><<<grid, GK_THREADS, 0, st>>>(xp, wp, y, (int)M, N, K, ldx, ldw, ldy, sx, sw, sy, epi, limit, nullptr);
      B200P_LAUNCH_CHECK("gemm_stream_kernel");
      return B200P_OK;
    }
    if constexpr (!std::is_same<T, float>::value) {
      if (g_gemm_path != 1) {
        const int rc = gemm_tc_launch<T>(xp, wp, y, M, N, K, ldx, ldw, ldy, batch, sx, sw, sy, epi, limit, st);
        if (rc != 1) return rc;
      }
    }
    // mma.sync: 128 x 128 tiles once that grid covers most of the GPU's SMs, 64 x 64 below
    const int64_t big = ((M + 127) / 128) * ((N + 127) / 128) * batch;
    if (big >= 96) return gemm_mma_launch<T, 2, 2, 64, 64, 32, 4>(xp, wp, y, M, N, K, ldx, ldw, ldy, batch, sx, sw, sy, epi, limit, st);
    return gemm_mma_launch<T, 2, 2, 32, 32, 32, 3>(xp, wp, y, M, N, K, ldx, ldw, ldy, batch, sx, sw, sy, epi, limit, st);
  }
  dim3 grid((unsigned)((N + GS_BN - 1) / GS_BN), (unsigned)((M + GS_BM - 1) / GS_BM), (unsigned)batch);
  gemm_simt_kernel<T><<<grid, 256, 0, st>>>(xp, wp, y, M, N, K, ldx, ldw, ldy, sx, sw, sy, epi, limit, nullptr);
  B200P_LAUNCH_CHECK("gemm_simt_kernel");
  return B200P_OK;
}

// groups of at most max_rows rows each: the row-streaming kernel while a group fits its 64 rows, 64 x 64 tiles beyond
template <typename T>
static int gemm_grouped_dispatch(const void* x, const void* w, void* y, const int32_t* seg, int64_t total_rows, int64_t max_rows, int64_t N, int64_t K,
                                 int64_t ldx, int64_t ldw, int64_t ldy, int64_t groups, int64_t sw, int epi, float limit, bool fast_ok,
                                 cudaStream_t st) {
  const T* xp = (const T*)x;
  const T* wp = (const T*)w;
  if (fast_ok && max_rows <= 64) {
    dim3 grid((unsigned)((N + 15) / 16), 1, (unsigned)groups);
    if (max_rows <= 16) gemm_stream_kernel<T, 1><<<grid, GK_THREADS, 0, st>>>(xp, wp, y, 0, N, K, ldx, ldw, ldy, 0, sw, 0, epi, limit, seg);
    else if (max_rows <= 32) gemm_stream_kernel<T, 2><<<grid, GK_THREADS, 0, st>>>(xp, wp, y, 0, N, K, ldx, ldw, ldy, 0, sw, 0, epi, limit, seg);
    else gemm_stream_kernel<T, 4><<<grid, GK_THREADS, 0, st>>>(xp, wp, y, 0, N, K, ldx, ldw, ldy, 0, sw, 0, epi, limit, seg);
    B200P_LAUNCH_CHECK("gemm_stream_kernel");
    return B200P_OK;
  }
  if (fast_ok) {
    if constexpr (!std::is_same<T, float>::value) {
      if (g_gemm_path != 1) {
        const int rc = gemm_tc_launch_grouped<T>(xp, wp, y, seg, total_rows, max_rows, N, K, ldx, ldw, ldy, groups, sw, epi, limit, st);
        if (rc != 1) return rc;
      }
    }
    return gemm_mma_launch<T, 2, 2, 32, 32, 32, 3>(xp, wp, y, max_rows, N, K, ldx, ldw, ldy, groups, 0, sw, 0, epi, limit, st, seg);
  }
  dim3 grid((unsigned)((N + GS_BN - 1) / GS_BN), (unsigned)((max_rows + GS_BM - 1) / GS_BM), (unsigned)groups);
  gemm_simt_kernel<T><<<grid, 256, 0, st>>>(xp, wp, y, max_rows, N, K, ldx, ldw, ldy, 0, sw, 0, epi, limit, seg);
  B200P_LAUNCH_CHECK("gemm_simt_kernel");
  return B200P_OK;
}

}  // namespace b200p

extern "C" int b200p_gemm_grouped(const void* x, const void* w, void* y, const int32_t* seg, int64_t total_rows, int64_t max_rows, int64_t N, int64_t K,
                                  int64_t ldx, int64_t ldw, int64_t ldy, int64_t groups, int64_t stride_w, int dtype, int epilogue,
                                  float limit, void* stream) {
  using namespace b200p;
  B200P_REQUIRE(x && w && y && seg, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(total_rows >= max_rows, B200P_ERR_ARG, "x has fewer rows than a group may have");
  B200P_REQUIRE(max_rows >= 0 && N > 0 && K > 0 && groups > 0 && groups < 65536 && ldx >= K && ldw >= K, B200P_ERR_ARG, "bad GEMM shape");
  B200P_REQUIRE(epilogue >= B200P_GEMM_STORE && epilogue <= B200P_GEMM_RELU_SQ, B200P_ERR_ARG, "unknown epilogue %d", epilogue);
  B200P_REQUIRE(epilogue < B200P_GEMM_GLU_CLAMP || epilogue > B200P_GEMM_GLU_SILU || N % 2 == 0, B200P_ERR_ARG, "the gated epilogue needs gate / up row pairs");
  B200P_REQUIRE((max_rows + 63) / 64 < 65536, B200P_ERR_ARG, "grid too large");
  if (max_rows == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool fast_ok = dtype != B200P_F32 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && stride_w % 8 == 0 && aligned(x, 16) &&
                       aligned(w, 16);
  switch (dtype) {
    case B200P_F32:
      return gemm_grouped_dispatch<float>(x, w, y, seg, total_rows, max_rows, N, K, ldx, ldw, ldy, groups, stride_w, epilogue, limit, false, st);
    case B200P_F16:
      return gemm_grouped_dispatch<__half>(x, w, y, seg, total_rows, max_rows, N, K, ldx, ldw, ldy, groups, stride_w, epilogue, limit, fast_ok, st);
    case B200P_BF16:
      return gemm_grouped_dispatch<__nv_bfloat16>(x, w, y, seg, total_rows, max_rows, N, K, ldx, ldw, ldy, groups, stride_w, epilogue, limit,
                                                  fast_ok, st);
    default:
      set_error("bad dtype %d", dtype);
      return B200P_ERR_ARG;
  }
}

extern "C" int b200p_gemm_set_path(int path) {
  b200p::g_gemm_path = (path == 1 || path == 2) ? path : 0;
  return B200P_OK;
}

extern "C" int b200p_gemm(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw,
                          int64_t ldy, int64_t batch, int64_t stride_x, int64_t stride_w, int64_t stride_y, int dtype,
                          int epilogue, float limit, void* stream) {
  using namespace b200p;
  B200P_REQUIRE(x && w && y, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(M >= 0 && N > 0 && K > 0 && batch > 0 && ldx >= K && ldw >= K, B200P_ERR_ARG, "bad GEMM shape");
  B200P_REQUIRE(epilogue >= B200P_GEMM_STORE && epilogue <= B200P_GEMM_RELU_SQ, B200P_ERR_ARG, "unknown epilogue %d", epilogue);
  B200P_REQUIRE(epilogue < B200P_GEMM_GLU_CLAMP || epilogue > B200P_GEMM_GLU_SILU || N % 2 == 0, B200P_ERR_ARG, "the gated epilogue needs gate / up row pairs");
  B200P_REQUIRE((M + 63) / 64 < 65536 && batch < 65536, B200P_ERR_ARG, "grid too large");
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // the 16-bit fast kernels move 16-byte pieces of rows: every row start and every k step must be 16-byte aligned
  const bool fast_ok = dtype != B200P_F32 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && stride_x % 8 == 0 &&
                       stride_w % 8 == 0 && aligned(x, 16) && aligned(w, 16);
  switch (dtype) {
    case B200P_F32:
      return gemm_dispatch<float>(x, w, y, M, N, K, ldx, ldw, ldy, batch, stride_x, stride_w, stride_y, epilogue, limit, false, st);
    case B200P_F16:
      return gemm_dispatch<__half>(x, w, y, M, N, K, ldx, ldw, ldy, batch, stride_x, stride_w, stride_y, epilogue, limit, fast_ok, st);
    case B200P_BF16:
      return gemm_dispatch<__nv_bfloat16>(x, w, y, M, N, K, ldx, ldw, ldy, batch, stride_x, stride_w, stride_y, epilogue, limit,
                                          fast_ok, st);
    default:
      set_error("bad dtype %d", dtype);
      return B200P_ERR_ARG;
  }
}

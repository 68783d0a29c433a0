// Rotated, chunk-masked attention with one or two score maps per head, over a ragged batch.
// Every query head carries `maps` (1 or 2) query vectors of d and every key/value head as many key vectors; each map is a
// softmax attention of its own over the SAME values.  With two maps the head's output is the difference
//   o = a_1 - lambda a_2                     ("differential" attention: the second map cancels what both attend to)
// which is then divided by its root mean square over the value size (when eps >= 0) and multiplied by `post`.
// Position i sees j <= i inside its own chunk of `chunk` positions (floor(i / chunk) == floor(j / chunk); chunk <= 0: every
// j <= i).  Chunks are counted from the sequence's first position, so how a prompt was cut into steps does not matter.
//   rope_attn_prep_kernel  pairwise rotation of the first rot_dims dimensions of every query / key vector (dimension 2i with
//                          2i+1, angle = position * rate_i), scale on q; keys and values into the caches           (per token)
//   diff_attn_kernel       one token x the query heads of one key/value head, fp32 throughout, any sizes          (per token)
//   diff_attn_tile_kernel  mma.sync tiles over 64-key blocks for 16-bit caches: 32 tokens of a prompt for one head (two warps
//                          per map), or the heads of a key/value head for one decoded token                          (16-bit)
#include "common.cuh"
#include "mma_util.cuh"

namespace b200p {

// vectors 0 .. nq-1 are the queries (written fp32, scaled), nq .. nq+nk-1 the keys (written to the cache: vector kv of a
// token lands at [row, kv / per_g, pos, (kv % per_g) * d ..], per_g = nk / G vectors side by side per key/value head)
template <typename T>
__global__ void rope_attn_prep_kernel(const float* __restrict__ proj, int64_t ldp, int64_t col_q, int64_t col_k, int64_t col_v,
                                      const float* __restrict__ rates, int rot_dims, float scale, float* __restrict__ q_out,
                                      T* __restrict__ kcache, T* __restrict__ vcache, int64_t Tcap,
                                      const int32_t* __restrict__ t_row, const int32_t* __restrict__ t_pos, int nq, int nk, int G,
                                      int d, int dv) {
  const int64_t t = blockIdx.x;
  const float* pt = proj + t * ldp;
  const int64_t pos = t_pos[t], row = t_row[t];
  const bool in_cache = pos < Tcap;                  // the host sizes the cache first; never write outside it
  const int per_g = nk / G, half = d / 2 + (d & 1), n_rot = rot_dims / 2;
  // one thread per pair of neighbouring dimensions (the last one alone when d is odd)
  for (int idx = threadIdx.x; idx < (nq + nk) * half; idx += blockDim.x) {
    const int vec = idx / half, i = idx % half;
    const bool is_q = vec < nq;
    const float* src = is_q ? pt + col_q + (int64_t)vec * d : pt + col_k + (int64_t)(vec - nq) * d;
    const bool pair = 2 * i + 1 < d;
    float a = src[2 * i], b = pair ? src[2 * i + 1] : 0.f;
    if (i < n_rot && pair) {
      float s, c;
      sincosf((float)pos * rates[i], &s, &c);
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = ra;
      b = rb;
    }
    if (is_q) {
      float* dst = q_out + (t * nq + vec) * d + 2 * i;
      dst[0] = a * scale;
      if (pair) dst[1] = b * scale;
    } else if (in_cache) {
      const int kv = vec - nq;
      T* dst = kcache + ((row * G + kv / per_g) * Tcap + pos) * (int64_t)(per_g * d) + (kv % per_g) * d + 2 * i;
      dst[0] = Tr<T>::from_f(a);
      if (pair) dst[1] = Tr<T>::from_f(b);
    }
  }
  if (in_cache) {
    for (int c = threadIdx.x; c < G * dv; c += blockDim.x) {
      const int g = c / dv, i = c % dv;
      vcache[((row * G + g) * Tcap + pos) * dv + i] = Tr<T>::from_f(pt[col_v + c]);
    }
  }
}

constexpr int DA_KEYS = 32;        // keys per staged block: one per lane in the score phase
constexpr int DA_MAX_HEADS = 8;    // query heads (warps) per CTA
constexpr int DA_MAX_VL = 16;      // value elements per lane: dv <= 512

// first key position that position `pos` sees
__device__ __forceinline__ int64_t chunk_start(int64_t pos, int64_t chunk) { return chunk > 0 ? pos / chunk * chunk : 0; }

// CTA = (token t, key/value head g, block of up to 8 of its query heads); warp = query head, both maps at once.
template <typename T, int MAPS>
__global__ void __launch_bounds__(DA_MAX_HEADS * 32)
diff_attn_kernel(const float* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache, int64_t Tcap,
                 const int32_t* __restrict__ t_row, const int32_t* __restrict__ t_pos, int64_t chunk, float lambda, float eps,
                 float post, T* __restrict__ out, int64_t ld_out, int H, int G, int d, int dv) {
  extern __shared__ float da_sm[];
  const int KD = MAPS * d, KS = KD + 1;                            // padded row: lane j reads row j without bank conflicts
  float* ks = da_sm;                                               // [DA_KEYS][KS]
  float* vs = ks + DA_KEYS * KS;                                   // [DA_KEYS][dv]
  float* qs = vs + DA_KEYS * dv;                                   // [warps][KD]
  const int64_t t = blockIdx.x;
  const int g = blockIdx.y, per = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int hl = blockIdx.z * nw + warp;                           // head inside the group
  const bool head_ok = hl < per;
  const int h = g * per + hl;
  const int64_t pos = t_pos[t];
  const T* kb = kcache + ((int64_t)t_row[t] * G + g) * Tcap * KD;
  const T* vb = vcache + ((int64_t)t_row[t] * G + g) * Tcap * dv;
  if (head_ok)
    for (int i = lane; i < KD; i += 32) qs[warp * KD + i] = q[(t * H + h) * KD + i];
  float acc[MAPS][DA_MAX_VL], mx[MAPS], den[MAPS];
#pragma unroll
  for (int m = 0; m < MAPS; ++m) {
    mx[m] = -INFINITY;
    den[m] = 0.f;
#pragma unroll
    for (int i = 0; i < DA_MAX_VL; ++i) acc[m][i] = 0.f;
  }
  for (int64_t j0 = chunk_start(pos, chunk); j0 <= pos; j0 += DA_KEYS) {
    const int nk = (int)min((int64_t)DA_KEYS, pos + 1 - j0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nk * KD; idx += blockDim.x) {
      const int kk = idx / KD, i = idx % KD;
      ks[kk * KS + i] = Tr<T>::to_f(kb[(j0 + kk) * KD + i]);
    }
    for (int idx = threadIdx.x; idx < nk * dv; idx += blockDim.x) vs[idx] = Tr<T>::to_f(vb[j0 * dv + idx]);
    __syncthreads();
    if (!head_ok) continue;
    float p[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
      float s = -INFINITY;
      if (lane < nk) {
        const float* kr = ks + lane * KS + m * d;
        const float* qr = qs + warp * KD + m * d;
        float dot = 0.f;
        for (int i = 0; i < d; ++i) dot = fmaf(qr[i], kr[i], dot);
        s = dot;
      }
      const float nmx = fmaxf(mx[m], warp_max(s));                 // finite: the block's first key is visible
      const float corr = expf(mx[m] - nmx);                        // 0 on the first block (mx = -inf)
      p[m] = lane < nk ? expf(s - nmx) : 0.f;
      den[m] = den[m] * corr + warp_sum(p[m]);
      mx[m] = nmx;
#pragma unroll
      for (int i = 0; i < DA_MAX_VL; ++i) acc[m][i] *= corr;
    }
    for (int kk = 0; kk < nk; ++kk) {
      const float* vr = vs + kk * dv;
      float pk[MAPS];
#pragma unroll
      for (int m = 0; m < MAPS; ++m) pk[m] = __shfl_sync(0xffffffffu, p[m], kk);
#pragma unroll
      for (int i = 0; i < DA_MAX_VL; ++i) {
        const int c = i * 32 + lane;
        if (c < dv) {
          const float vv = vr[c];
#pragma unroll
          for (int m = 0; m < MAPS; ++m) acc[m][i] = fmaf(pk[m], vv, acc[m][i]);
        }
      }
    }
  }
  if (!head_ok) return;
  float o[DA_MAX_VL], ss = 0.f;
  const float inv0 = 1.f / den[0], inv1 = MAPS == 2 ? lambda / den[MAPS - 1] : 0.f;
#pragma unroll
  for (int i = 0; i < DA_MAX_VL; ++i) {
    o[i] = acc[0][i] * inv0;
    if (MAPS == 2) o[i] -= acc[MAPS - 1][i] * inv1;
    if (i * 32 + lane < dv) ss = fmaf(o[i], o[i], ss);
  }
  float mul = post;
  if (eps >= 0.f) mul *= 1.f / sqrtf(warp_sum(ss) / (float)dv + eps);
#pragma unroll
  for (int i = 0; i < DA_MAX_VL; ++i) {
    const int c = i * 32 + lane;
    if (c < dv) out[t * ld_out + (int64_t)h * dv + c] = Tr<T>::from_f(o[i] * mul);
  }
}

template <typename T>
static int diff_attn_generic(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                             const int32_t* t_pos, int64_t chunk, int maps, float lambda, float eps, float post, void* out,
                             int64_t ld_out, int64_t M, int H, int G, int d, int dv, cudaStream_t st) {
  const int per = H / G, nw = per < DA_MAX_HEADS ? per : DA_MAX_HEADS;
  const size_t smem = ((size_t)DA_KEYS * (maps * d + 1) + (size_t)DA_KEYS * dv + (size_t)nw * maps * d) * sizeof(float);
  auto kern = maps == 2 ? diff_attn_kernel<T, 2> : diff_attn_kernel<T, 1>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(diff_attn_kernel)");
  }
  dim3 grid((unsigned)M, (unsigned)G, (unsigned)((per + nw - 1) / nw));
  kern<<<grid, nw * 32, smem, st>>>(q, (const T*)kcache, (const T*)vcache, Tcap, t_row, t_pos, chunk, lambda, eps, post, (T*)out, ld_out,
                                    H, G, d, dv);
  B200P_LAUNCH_CHECK("diff_attn_kernel");
  return B200P_OK;
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_rope_attn_prep(const float* proj, int64_t ldp, int64_t col_q, int64_t col_k, int64_t col_v, const float* rates,
                                    int rot_dims, float scale, float* q_out, void* kcache, void* vcache, int64_t Tcap,
                                    const int32_t* t_row, const int32_t* t_pos, int64_t M, int H, int G, int maps, int d, int dv,
                                    int dtype, void* stream) {
  B200P_REQUIRE(proj && q_out && kcache && vcache && t_row && t_pos, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0 && (maps == 1 || maps == 2), B200P_ERR_ARG, "bad head geometry");
  B200P_REQUIRE(rot_dims >= 0 && rot_dims <= d && rot_dims % 2 == 0 && (rot_dims == 0 || rates), B200P_ERR_ARG,
                "rotated dimensions: an even count up to the vector size, with their rates");
  if (M == 0) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (rope_attn_prep_kernel<T><<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(
      proj, ldp, col_q, col_k, col_v, rates, rot_dims, scale, q_out, (T*)kcache, (T*)vcache, Tcap, t_row, t_pos, H * maps, G * maps, G,
      d, dv)));
  B200P_LAUNCH_CHECK("rope_attn_prep_kernel");
  return B200P_OK;
}

extern "C" int b200p_diff_attn(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                               const int32_t* t_pos, const int32_t* cu, const int32_t* rows, int nb, int max_n, int64_t chunk,
                               int maps, float lambda, float eps, float post, void* out, int64_t ld_out, int64_t M, int H, int G,
                               int d, int dv, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  B200P_REQUIRE(q && kcache && vcache && t_row && t_pos && out, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && G > 0 && H % G == 0 && G < 65536 && d > 0 && dv > 0 && (maps == 1 || maps == 2), B200P_ERR_ARG,
                "bad head geometry");
  B200P_REQUIRE(dv <= 32 * DA_MAX_VL && maps * d <= 1024, B200P_ERR_ARG, "value size above %d or key size above 1024 is not built",
                32 * DA_MAX_VL);
  B200P_REQUIRE(ld_out >= (int64_t)H * dv, B200P_ERR_ARG, "output rows are shorter than the heads");
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  (void)cu; (void)rows; (void)nb; (void)max_n; (void)workspace; (void)workspace_bytes;
  switch (dtype) {
    case B200P_F32: return diff_attn_generic<float>(q, kcache, vcache, Tcap, t_row, t_pos, chunk, maps, lambda, eps, post, out, ld_out, M, H, G, d, dv, st);
    case B200P_F16: return diff_attn_generic<__half>(q, kcache, vcache, Tcap, t_row, t_pos, chunk, maps, lambda, eps, post, out, ld_out, M, H, G, d, dv, st);
    case B200P_BF16: return diff_attn_generic<__nv_bfloat16>(q, kcache, vcache, Tcap, t_row, t_pos, chunk, maps, lambda, eps, post, out, ld_out, M, H, G, d, dv, st);
    default: set_error("bad dtype %d", dtype); return B200P_ERR_ARG;
  }
}

extern "C" size_t b200p_diff_attn_workspace_bytes(int64_t nb, int H, int maps, int dv) {
  (void)nb; (void)H; (void)maps; (void)dv;
  return 0;
}

// Attention over a shared low-rank latent: every position stores ONE vector c (rank R) that serves as key and value of all
// heads; the per-head key and value up-projections are folded into the query (before) and the output (after) by b200p_gemm,
// so the cache is read as it is stored.  A sliding window bounds the visible positions.
//   latent_prep_kernel   rms norms of the two down-projections; the key/value latent goes into the cache
//   latent_attn_kernel   one CTA per token and group of heads; keys staged 32 at a time in shared memory; online fp32 softmax
//                        (decode steps, float32 models, ranks off the tensor-core shapes)
//   latent_attn_tile_kernel  16-bit models: up to four tiles of 16 query rows per CTA (prompts: 16 consecutive tokens of one
//                        sequence for one head each; decode steps: 16 heads each of the one new token), mma.sync m16n8k16 for
//                        q.c and p.c over 64-key chunks staged once for both products and for all the CTA's tiles
#include <cooperative_groups.h>

#include "common.cuh"
#include "mma_util.cuh"

namespace b200p {

template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ proj, int64_t ldp, int q_rank, int kv_rank,
                                   const float* __restrict__ wq, const float* __restrict__ wkv, float eps, T* __restrict__ cq_out,
                                   T* __restrict__ cache, int64_t Tcap, const int32_t* __restrict__ t_row,
                                   const int32_t* __restrict__ t_pos) {
  __shared__ float red[2];
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;     // warp 0: query part, warp 1: key/value part
  const float* src = proj + t * ldp + (warp == 0 ? 0 : q_rank);
  const int n = warp == 0 ? q_rank : kv_rank;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncwarp();
  if (n == 0) return;
  const float inv = 1.f / sqrtf(red[warp] / (float)n + eps);
  if (warp == 0) {
    for (int i = lane; i < n; i += 32) cq_out[t * q_rank + i] = Tr<T>::from_f(src[i] * inv * wq[i]);
  } else {
    const int64_t pos = t_pos[t];
    if (pos >= Tcap) return;                                       // the host sizes the cache first; never write outside it
    T* dst = cache + ((int64_t)t_row[t] * Tcap + pos) * kv_rank;
    for (int i = lane; i < n; i += 32) dst[i] = Tr<T>::from_f(src[i] * inv * wkv[i]);
  }
}

// The same two norms for designs whose keys also have a rotated part that all heads share: proj = [query (q_rank) | key/value
// (kv_rank) | rotated key part (rot_dim)].  The cache row is [normed latent | rotated part | zeros up to `row`]: the pairs
// (2i, 2i+1) of the last part turn by the angle position * rates[i] (fp32, accurate sine and cosine) and are multiplied by `mag`.
template <typename T>
__global__ void latent_rope_prep_kernel(const float* __restrict__ proj, int64_t ldp, int q_rank, int kv_rank, int rot_dim, int row,
                                        const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                                        const float* __restrict__ rates, float mag, T* __restrict__ cq_out, T* __restrict__ cache,
                                        int64_t Tcap, const int32_t* __restrict__ t_row, const int32_t* __restrict__ t_pos) {
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;     // warp 0: query part, warp 1: key/value part, warp 2: rotated part
  const int64_t pos = t_pos[t];
  T* dst = cache + ((int64_t)t_row[t] * Tcap + pos) * row;
  if (warp == 2) {
    if (pos >= Tcap) return;                                       // the host sizes the cache first; never write outside it
    const float* src = proj + t * ldp + q_rank + kv_rank;
    for (int i = lane; i < rot_dim / 2; i += 32) {
      float sn, cs;
      sincosf((float)pos * rates[i], &sn, &cs);
      sn *= mag; cs *= mag;
      const float u = src[2 * i], v = src[2 * i + 1];
      dst[kv_rank + 2 * i] = Tr<T>::from_f(u * cs - v * sn);
      dst[kv_rank + 2 * i + 1] = Tr<T>::from_f(v * cs + u * sn);
    }
    for (int i = kv_rank + rot_dim + lane; i < row; i += 32) dst[i] = Tr<T>::from_f(0.f);
    return;
  }
  const float* src = proj + t * ldp + (warp == 0 ? 0 : q_rank);
  const int n = warp == 0 ? q_rank : kv_rank;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) ss = fmaf(src[i], src[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  if (warp == 0) {
    for (int i = lane; i < n; i += 32) cq_out[t * q_rank + i] = Tr<T>::from_f(src[i] * inv * wq[i]);
  } else {
    if (pos >= Tcap) return;
    for (int i = lane; i < n; i += 32) dst[i] = Tr<T>::from_f(src[i] * inv * wkv[i]);
  }
}

// The rotated part of the queries, q [M, H, dim + rot_dim] in the storage type: its last rot_dim values turn like the keys' and
// go, fp32, behind the latent-space part of the head's query row, q_lat [M, H, row] columns [kv_rank, kv_rank + rot_dim); the
// columns up to `row` become zero.
template <typename T>
__global__ void latent_q_rope_kernel(const T* __restrict__ q, int H, int dim, int rot_dim, int kv_rank, int row,
                                     const float* __restrict__ rates, float mag, const int32_t* __restrict__ t_pos,
                                     float* __restrict__ q_lat) {
  const int64_t t = blockIdx.x;
  const float pos = (float)t_pos[t];
  const int half = rot_dim / 2, tail = row - kv_rank - rot_dim;
  for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    float sn, cs;
    sincosf(pos * rates[i], &sn, &cs);
    sn *= mag; cs *= mag;
    const T* src = q + (t * H + h) * (int64_t)(dim + rot_dim) + dim;
    const float u = Tr<T>::to_f(src[2 * i]), v = Tr<T>::to_f(src[2 * i + 1]);
    float* dst = q_lat + (t * H + h) * (int64_t)row + kv_rank;
    dst[2 * i] = u * cs - v * sn;
    dst[2 * i + 1] = v * cs + u * sn;
  }
  for (int idx = threadIdx.x; idx < H * tail; idx += blockDim.x)
    q_lat[(t * H + idx / tail) * (int64_t)row + kv_rank + rot_dim + idx % tail] = 0.f;
}

constexpr int LA_KEYS = 32;       // keys per staged chunk: one per lane in the score phase
constexpr int LA_MAX_HEADS = 8;   // heads (warps) per CTA
constexpr int LA_MAX_RL = 32;     // latent elements per lane in the output phase: R <= 1024

template <typename T>
__global__ void __launch_bounds__(LA_MAX_HEADS * 32)
latent_attn_kernel(const float* __restrict__ q, const T* __restrict__ cache, int64_t Tcap, const int32_t* __restrict__ t_row,
                   const int32_t* __restrict__ t_pos, T* __restrict__ out, int H, int R, int64_t window, float scale) {
  extern __shared__ float sm[];
  const int RS = R + 1;                                            // padded row: lane j reads row j without bank conflicts
  float* cs = sm;                                                  // [LA_KEYS][RS]
  float* qs = sm + LA_KEYS * RS;                                   // [warps][R]
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int h = blockIdx.y * nw + warp;
  const bool head_ok = h < H;
  const int64_t pos = t_pos[t];
  const int64_t lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const T* cbase = cache + (int64_t)t_row[t] * Tcap * R;
  if (head_ok)
    for (int r = lane; r < R; r += 32) qs[warp * R + r] = q[(t * H + h) * R + r];
  float acc[LA_MAX_RL];
#pragma unroll
  for (int i = 0; i < LA_MAX_RL; ++i) acc[i] = 0.f;
  float mx = -INFINITY, den = 0.f;
  for (int64_t j0 = lo; j0 <= pos; j0 += LA_KEYS) {
    const int nk = (int)min((int64_t)LA_KEYS, pos + 1 - j0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nk * R; idx += blockDim.x) {
      const int kk = idx / R, r = idx % R;
      cs[kk * RS + r] = Tr<T>::to_f(cbase[(j0 + kk) * R + r]);
    }
    __syncthreads();
    if (!head_ok) continue;
    float s = -INFINITY;
    if (lane < nk) {
      const float* cr = cs + lane * RS;
      const float* qr = qs + warp * R;
      float d = 0.f;
      for (int r = 0; r < R; ++r) d = fmaf(qr[r], cr[r], d);
      s = d * scale;
    }
    const float cmx = warp_max(s);
    const float nmx = fmaxf(mx, cmx);
    const float corr = expf(mx - nmx);                             // 0 on the first chunk (mx = -inf)
    const float p = lane < nk ? expf(s - nmx) : 0.f;
    den = den * corr + warp_sum(p);
    mx = nmx;
#pragma unroll
    for (int i = 0; i < LA_MAX_RL; ++i) acc[i] *= corr;
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const float* cr = cs + kk * RS;
#pragma unroll
      for (int i = 0; i < LA_MAX_RL; ++i) {
        const int r = i * 32 + lane;
        if (r < R) acc[i] = fmaf(pk, cr[r], acc[i]);
      }
    }
  }
  if (!head_ok) return;
  const float inv = 1.f / den;
#pragma unroll
  for (int i = 0; i < LA_MAX_RL; ++i) {
    const int r = i * 32 + lane;
    if (r < R) out[(t * H + h) * R + r] = Tr<T>::from_f(acc[i] * inv);
  }
}


// ---- prompts on the tensor cores -----------------------------------------------------------------------------------------
// CTA = (tile of 16 tokens of entry e, G heads), G groups of 4 warps; group g owns one head.  All heads read the same latent
// cache, so a chunk of 64 positions is staged ONCE per CTA (cp.async; one copy serves keys and values of all G heads): the
// L2 -> shared traffic per head falls by G, which is what bounded the one-head tile.  Per chunk, in every group:
//   S   warp w: scores of its 16 keys, q [16, R] x c[16 keys, R]^T                     -> shared S [16, 64] fp32, masked
//   P   8 threads per row: running max / sum in fp32, p = exp(s - max) as 16-bit       -> shared P [16, 64]
//   O   warp w: columns [w R/4, (w+1) R/4) of o [16, R] += P x c[64 keys, its columns]   (accumulators rescaled first)
constexpr int LT_ROWS = 16, LT_KEYS = 64, LT_THREADS = 128, LT_MAX_NT = 16;      // R <= 512, R % 32 == 0
constexpr int LT_WIDE_NT = 20;     // a second instantiation with more accumulators: 512 < R <= 640 (a 512-value latent plus a rotated part)
constexpr int LT_MAX_GROUPS = 4;

int sm_count();

template <typename T, int G, int MAXNT>
__global__ void __launch_bounds__(LT_THREADS * G)
latent_attn_tile_kernel(const float* __restrict__ q, const T* __restrict__ cache, int64_t Tcap, const int32_t* __restrict__ cu,
                        const int32_t* __restrict__ rows, const int32_t* __restrict__ t_pos, T* __restrict__ out, int H, int R,
                        int64_t window, float scale, int by_head, int splits, int nbuf) {
  extern __shared__ __align__(128) uint8_t lt_smem[];
  // splits > 1 (decode only): the CTAs of a thread-block cluster (gridDim.x = cluster size = splits) share the keys of one tile
  // between them, a run of 64-key chunks each, and CTA 0 merges their partial sums through distributed shared memory
  // by_head == 0: rows of a group's tile are 16 consecutive tokens of entry e = blockIdx.z, for ONE head (prompts)
  // by_head == 1: rows are 16 consecutive heads of the ONE token of entry e (decode: every head reads the same keys)
  const int e = blockIdx.z;
  const int grp = threadIdx.x / LT_THREADS, tl = threadIdx.x % LT_THREADS;
  const int h = by_head ? (blockIdx.y * G + grp) * LT_ROWS : blockIdx.y * G + grp;
  const int t0 = by_head ? cu[e] : cu[e] + blockIdx.x * LT_ROWS;
  if ((by_head ? cu[e + 1] - cu[e] : cu[e + 1] - t0) <= 0) return;             // the same for every thread of the CTA
  const bool active = h < H;                                     // a group past the last head only helps to stage the chunks
  const int nrow = !active ? 0 : by_head ? min(LT_ROWS, H - h) : min(LT_ROWS, cu[e + 1] - t0);               // live rows
  const int tstep = by_head ? 0 : 1, hstep = by_head ? 1 : 0;   // row r is token t0 + r * tstep, head h + r * hstep
  const int LDC = R + 8;                                         // padded rows: ldmatrix reads 8 rows without bank conflicts
  T* cs0 = reinterpret_cast<T*>(lt_smem);                        // nbuf x [64][LDC], shared by the groups; with two buffers the
                                                                 // next chunk is in flight while this one is multiplied
  const size_t group_bytes = (size_t)(LT_ROWS * LDC + LT_ROWS * 72) * sizeof(T) + (LT_ROWS * 68 + 3 * LT_ROWS) * sizeof(float);
  T* qs = reinterpret_cast<T*>(lt_smem + (size_t)nbuf * LT_KEYS * LDC * sizeof(T) + grp * group_bytes);             // [16][LDC]
  T* ps = qs + LT_ROWS * LDC;                                    // [16][72]
  float* ss = reinterpret_cast<float*>(ps + LT_ROWS * 72);       // [16][68]
  float* row_m = ss + LT_ROWS * 68;                              // running max, sum, and this chunk's rescale factor
  float* row_l = row_m + LT_ROWS;
  float* row_c = row_l + LT_ROWS;
  const int warp = tl >> 5, lane = tl & 31;                     // warp inside the group
  const int64_t p0 = t_pos[t0];                                  // positions of the tile's rows are p0, p0 + 1, ...
  const int64_t plast = by_head ? p0 : p0 + min(LT_ROWS, cu[e + 1] - t0) - 1;
  const int64_t kmin = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
  const T* cbase = cache + (int64_t)rows[e] * Tcap * R;
#pragma unroll 4
  for (int idx = tl; idx < LT_ROWS * (R / 4); idx += LT_THREADS) {       // R is a multiple of 32: rows of q are 16-byte aligned
    const int r = idx / (R / 4), c = (idx % (R / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < nrow) v = *reinterpret_cast<const float4*>(q + ((int64_t)(t0 + r * tstep) * H + h + r * hstep) * R + c);
    *reinterpret_cast<uint2*>(qs + r * LDC + c) = make_uint2(pack2<T>(v.x, v.y), pack2<T>(v.z, v.w));
  }
  if (tl < LT_ROWS) { row_m[tl] = -INFINITY; row_l[tl] = 0.f; }
  const int ntw = R / 32;                                        // 8-column tiles of o per warp
  float o[MAXNT][4];
#pragma unroll
  for (int i = 0; i < MAXNT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int chunks_per_row = R / 8;
  int64_t jbeg = kmin, jend = plast;                             // this CTA's keys, inclusive
  if (splits > 1) {
    const int64_t nchunks = (plast - kmin) / LT_KEYS + 1, per = (nchunks + splits - 1) / splits;
    jbeg = kmin + (int64_t)blockIdx.x * per * LT_KEYS;
    jend = min(plast, jbeg + per * LT_KEYS - 1);
  }
  auto stage_chunk = [&](int64_t j0, T* dst) {                  // 64 latents from position j0 on (zero-filled past plast)
    for (int idx = threadIdx.x; idx < LT_KEYS * chunks_per_row; idx += LT_THREADS * G) {
      const int kk = idx / chunks_per_row, c = (idx % chunks_per_row) * 8;
      const bool ok = j0 + kk <= plast;
      cp_async16((uint32_t)__cvta_generic_to_shared(dst + kk * LDC + c), ok ? (const void*)(cbase + (j0 + kk) * R + c) : (const void*)cbase, ok);
    }
    cp_async_commit();
  };
  if (nbuf > 1 && jbeg <= jend) stage_chunk(jbeg, cs0);
  int buf = 0;
  for (int64_t j0 = jbeg; j0 <= jend; j0 += LT_KEYS) {
    T* cs = cs0 + (size_t)buf * LT_KEYS * LDC;
    if (nbuf > 1) {
      cp_async_wait<0>();
      __syncthreads();                                           // this chunk has landed; the previous chunk's products are done
      if (j0 + LT_KEYS <= jend) stage_chunk(j0 + LT_KEYS, cs0 + (size_t)(buf ^ 1) * LT_KEYS * LDC);
      buf ^= 1;
    } else {
      __syncthreads();                                           // the previous chunk's products are done with cs / ss / ps
      stage_chunk(j0, cs);
      cp_async_wait<0>();
      __syncthreads();
    }
    if (active) {   // ---- S
      float sc[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
      for (int kk = 0; kk < R; kk += 16) {
        uint32_t a[4], b[4];
        ldsm_x4((uint32_t)__cvta_generic_to_shared(qs + (lane & 15) * LDC + kk + (lane >> 4) * 8), a);
        ldsm_x4((uint32_t)__cvta_generic_to_shared(cs + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * LDC + kk + ((lane >> 3) & 1) * 8), b);
        mma16816<T>(sc[0], a, b[0], b[1]);
        mma16816<T>(sc[1], a, b[2], b[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int el = 0; el < 4; ++el) {
          const int r = (lane >> 2) + (el >> 1) * 8;
          const int kc = warp * 16 + nt * 8 + (lane & 3) * 2 + (el & 1);
          const int64_t key = j0 + kc, pr = p0 + r * tstep;
          const bool vis = r < nrow && key <= pr && (window <= 0 || pr - key < window);
          ss[r * 68 + kc] = vis ? sc[nt][el] * scale : -INFINITY;
        }
    }
    __syncthreads();
    if (active) {   // ---- P: thread = (row, eighth of the chunk)
      const int r = tl >> 3, seg = tl & 7;
      float v[8], mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) { v[i] = ss[r * 68 + seg * 8 + i]; mx = fmaxf(mx, v[i]); }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float mo = row_m[r], mn = fmaxf(mo, mx);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float pv = mn == -INFINITY ? 0.f : __expf(v[i] - mn);      // masked scores are -inf: exp gives 0
        sum += pv;
        ps[r * 72 + seg * 8 + i] = Tr<T>::from_f(pv);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      __syncwarp();                                              // every lane of the row has read row_m before it changes
      if (seg == 0) {
        const float corr = mn == -INFINITY ? 1.f : __expf(mo - mn);      // mo = -inf on the first visible chunk: 0
        row_c[r] = corr;
        row_l[r] = row_l[r] * corr + sum;
        row_m[r] = mn;
      }
    }
    __syncthreads();
    if (active) {   // ---- O
      const float c0 = row_c[lane >> 2], c1 = row_c[(lane >> 2) + 8];
#pragma unroll
      for (int i = 0; i < MAXNT; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
#pragma unroll
      for (int kk = 0; kk < LT_KEYS; kk += 16) {
        uint32_t a[4];
        ldsm_x4((uint32_t)__cvta_generic_to_shared(ps + (lane & 15) * 72 + kk + (lane >> 4) * 8), a);
#pragma unroll
        for (int jp = 0; jp < MAXNT / 2; ++jp) {
          if (2 * jp < ntw) {
            uint32_t b[4];
            ldsm_x4_trans((uint32_t)__cvta_generic_to_shared(cs + (kk + (lane & 15)) * LDC + warp * (R / 4) + jp * 16 + (lane >> 4) * 8), b);
            mma16816<T>(o[2 * jp], a, b[0], b[1]);
            mma16816<T>(o[2 * jp + 1], a, b[2], b[3]);
          }
        }
      }
    }
  }
  __syncthreads();
  if (splits > 1) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    float* po = reinterpret_cast<float*>(cs0);                    // [16][R] unnormalised partial sums (the chunk buffer is free now)
#pragma unroll
    for (int i = 0; i < MAXNT; ++i) {
      if (i < ntw) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int r = (lane >> 2) + hf * 8, c = warp * (R / 4) + i * 8 + (lane & 3) * 2;
          po[r * R + c] = o[i][hf * 2];
          po[r * R + c + 1] = o[i][hf * 2 + 1];
        }
      }
    }
    cluster.sync();
    {   // every CTA of the cluster merges its own slice of the columns, R / splits wide, for all rows
      const int r = tl >> 3, seg = tl & 7;                       // eight threads per row
      const int cw = R / splits, c0 = (int)cluster.block_rank() * cw;
      if (r < nrow) {
        float ms[8], ls[8], m = -INFINITY, l = 0.f;
#pragma unroll
        for (int s_ = 0; s_ < 8; ++s_) {
          if (s_ < splits) {
            ms[s_] = cluster.map_shared_rank(row_m, s_)[r];
            ls[s_] = cluster.map_shared_rank(row_l, s_)[r];
            m = fmaxf(m, ms[s_]);
          }
        }
#pragma unroll
        for (int s_ = 0; s_ < 8; ++s_) {
          if (s_ < splits) {
            ms[s_] = ms[s_] == -INFINITY ? 0.f : __expf(ms[s_] - m);     // a CTA whose run of keys was empty or all masked: 0
            l += ls[s_] * ms[s_];
          }
        }
        const float inv = 1.f / l;
        T* dst = out + ((int64_t)(t0 + r * tstep) * H + h + r * hstep) * R;
#pragma unroll 2
        for (int c = c0 + seg; c < c0 + cw; c += 8) {
          float part[8];
#pragma unroll
          for (int s_ = 0; s_ < 8; ++s_) part[s_] = s_ < splits ? cluster.map_shared_rank(po, s_)[r * R + c] : 0.f;
          float acc = 0.f;
#pragma unroll
          for (int s_ = 0; s_ < 8; ++s_) acc = fmaf(part[s_], s_ < splits ? ms[s_] : 0.f, acc);
          dst[c] = Tr<T>::from_f(acc * inv);
        }
      }
    }
    cluster.sync();                                              // a CTA's shared memory lives until the others have read it
    return;
  }
#pragma unroll
  for (int i = 0; i < MAXNT; ++i) {
    if (i < ntw) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int r = (lane >> 2) + hf * 8;
        if (r < nrow) {
          const float inv = 1.f / row_l[r];
          const int c = warp * (R / 4) + i * 8 + (lane & 3) * 2;
          *reinterpret_cast<uint32_t*>(out + ((int64_t)(t0 + r * tstep) * H + h + r * hstep) * R + c) =
              pack2<T>(o[i][hf * 2] * inv, o[i][hf * 2 + 1] * inv);
        }
      }
    }
  }
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_latent_prep(const float* proj, int64_t ldp, int q_rank, int kv_rank, const float* wq, const float* wkv,
                                 float eps, void* cq_out, void* cache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos,
                                 int64_t M, int dtype, void* stream) {
  B200P_REQUIRE(proj && wq && cq_out && q_rank > 0 && kv_rank >= 0, B200P_ERR_ARG, "null pointer or bad rank");
  B200P_REQUIRE(kv_rank == 0 || (wkv && cache && t_row && t_pos && Tcap > 0), B200P_ERR_ARG, "the key/value latent needs its cache");
  if (M == 0) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (latent_prep_kernel<T><<<(unsigned)M, 64, 0, (cudaStream_t)stream>>>(
      proj, ldp, q_rank, kv_rank, wq, wkv, eps, (T*)cq_out, (T*)cache, Tcap, t_row, t_pos)));
  B200P_LAUNCH_CHECK("latent_prep_kernel");
  return B200P_OK;
}

extern "C" int b200p_latent_rope_prep(const float* proj, int64_t ldp, int q_rank, int kv_rank, int rot_dim, int row, const float* wq,
                                      const float* wkv, float eps, const float* rates, float mag, void* cq_out, void* cache,
                                      int64_t Tcap, const int32_t* t_row, const int32_t* t_pos, int64_t M, int dtype, void* stream) {
  B200P_REQUIRE(proj && wq && wkv && cq_out && cache && t_row && t_pos, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(q_rank > 0 && kv_rank > 0 && rot_dim >= 0 && rot_dim % 2 == 0 && row >= kv_rank + rot_dim && Tcap > 0, B200P_ERR_ARG,
                "bad ranks: an even rotated part and a cache row that holds latent and rotated part");
  B200P_REQUIRE(rot_dim == 0 || rates, B200P_ERR_ARG, "the rotated part needs its rates");
  if (M == 0) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (latent_rope_prep_kernel<T><<<(unsigned)M, 96, 0, (cudaStream_t)stream>>>(
      proj, ldp, q_rank, kv_rank, rot_dim, row, wq, wkv, eps, rates, mag, (T*)cq_out, (T*)cache, Tcap, t_row, t_pos)));
  B200P_LAUNCH_CHECK("latent_rope_prep_kernel");
  return B200P_OK;
}

extern "C" int b200p_latent_q_rope(const void* q, int H, int dim, int rot_dim, int kv_rank, int row, const float* rates, float mag,
                                   const int32_t* t_pos, float* q_lat, int64_t M, int dtype, void* stream) {
  B200P_REQUIRE(q && t_pos && q_lat && (rot_dim == 0 || rates), B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && dim >= 0 && rot_dim >= 0 && rot_dim % 2 == 0 && row >= kv_rank + rot_dim, B200P_ERR_ARG, "bad sizes");
  if (M == 0 || row == kv_rank) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (latent_q_rope_kernel<T><<<(unsigned)M, 128, 0, (cudaStream_t)stream>>>(
      (const T*)q, H, dim, rot_dim, kv_rank, row, rates, mag, t_pos, q_lat)));
  B200P_LAUNCH_CHECK("latent_q_rope_kernel");
  return B200P_OK;
}

template <typename T>
static int latent_attn_launch(const float* q, const void* cache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos, void* out,
                              int64_t M, int H, int R, int64_t window, float scale, cudaStream_t st) {
  const int nw = H < LA_MAX_HEADS ? H : LA_MAX_HEADS;
  const size_t smem = ((size_t)LA_KEYS * (R + 1) + (size_t)nw * R) * sizeof(float);
  auto kern = latent_attn_kernel<T>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(latent_attn_kernel)");
  }
  dim3 grid((unsigned)M, (unsigned)((H + nw - 1) / nw));
  kern<<<grid, nw * 32, smem, st>>>(q, (const T*)cache, Tcap, t_row, t_pos, (T*)out, H, R, window, scale);
  B200P_LAUNCH_CHECK("latent_attn_kernel");
  return B200P_OK;
}

extern "C" int b200p_latent_attn(const float* q, const void* cache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos,
                                 void* out, int64_t M, int H, int R, int64_t window, float scale, int dtype, void* stream) {
  B200P_REQUIRE(q && cache && t_row && t_pos && out, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && R > 0 && R <= 32 * LA_MAX_RL, B200P_ERR_ARG, "latent rank must be in [1, %d]", 32 * LA_MAX_RL);
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case B200P_F32: return latent_attn_launch<float>(q, cache, Tcap, t_row, t_pos, out, M, H, R, window, scale, st);
    case B200P_F16: return latent_attn_launch<__half>(q, cache, Tcap, t_row, t_pos, out, M, H, R, window, scale, st);
    case B200P_BF16: return latent_attn_launch<__nv_bfloat16>(q, cache, Tcap, t_row, t_pos, out, M, H, R, window, scale, st);
    default: set_error("bad dtype %d", dtype); return B200P_ERR_ARG;
  }
}

static int g_lt_groups = 0;     // 0: chosen per launch; 1..4: forced (b200p_latent_attn_set_groups)
static int g_lt_nbuf = 0;       // chunk buffers of the tile kernel: 0 = chosen per launch, 1 or 2 forced (b200p_latent_attn_set_buffers)
static int g_lt_splits = 0;     // decode: 0 = chosen per launch; 1 = one CTA per tile; 2, 4, 8 = forced (b200p_latent_attn_set_splits)

template <typename T, int MAXNT>
static int latent_attn_tile_launch(const float* q, const void* cache, int64_t Tcap, const int32_t* cu, const int32_t* rows,
                                   const int32_t* t_pos, void* out, int nb, int max_n, int H, int R, int64_t window, float scale,
                                   cudaStream_t st) {
  const int by_head = max_n == 1 ? 1 : 0;       // one token per entry: tile over the heads instead of over the tokens
  const int units = by_head ? (H + LT_ROWS - 1) / LT_ROWS : H;                   // 16-row tiles that share one set of keys
  // Two tiles per CTA halve the L2 -> shared traffic per head and win on prompts from rank 128 up (1.1x at rank 256, 1.8x at
  // rank 512); four leave one CTA per SM (registers) and lose the overlap between CTAs again.  Decode steps gain nothing.
  // Above rank 512 one CTA per SM is all that fits: four tiles on one staged copy then beat two (5.7 -> 4.3 ms at rank 576).
  int G = g_lt_groups > 0 ? g_lt_groups : (by_head || R < 128) ? 1 : R > 32 * LT_MAX_NT ? 4 : 2;
  if (G > units) G = units;
  if (G == 3) G = 2;
  const size_t group_bytes = ((size_t)LT_ROWS * (R + 8) + LT_ROWS * 72) * sizeof(T) + (LT_ROWS * 68 + 3 * LT_ROWS) * sizeof(float);
  // two chunk buffers where two CTAs per SM still fit beside them (ranks up to 256); above, the second CTA hides more latency
  // than the second buffer (measured on prompts and on decode steps)
  const size_t chunk_bytes = (size_t)LT_KEYS * (R + 8) * sizeof(T);
  const int nbuf = g_lt_nbuf > 0 ? g_lt_nbuf : 2 * (2 * chunk_bytes + G * group_bytes) <= 220 * 1024 ? 2 : 1;
  const size_t smem = nbuf * chunk_bytes + G * group_bytes;
  auto kern = G == 1 ? latent_attn_tile_kernel<T, 1, MAXNT> : G == 2 ? latent_attn_tile_kernel<T, 2, MAXNT> : latent_attn_tile_kernel<T, 4, MAXNT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(latent_attn_tile_kernel)");
  }
  // Decode steps have few tiles (entries x heads / 16), each a serial walk over the window: a cluster of up to 8 CTAs shares the
  // chunks of one tile so that about two CTAs per SM stream the cache
  int splits = 1;
  if (by_head && G == 1 && g_lt_splits != 1) {
    const int64_t tiles = (int64_t)nb * units, span = window > 0 ? window : Tcap;
    const int64_t chunks = (span + LT_KEYS - 1) / LT_KEYS + 1;
    int64_t want = g_lt_splits > 1 ? g_lt_splits : (2ll * sm_count() + tiles - 1) / tiles;
    want = want < chunks ? want : chunks;
    splits = want >= 8 ? 8 : want >= 4 ? 4 : want >= 2 ? 2 : 1;
  }
  dim3 grid(by_head ? (unsigned)splits : (unsigned)((max_n + LT_ROWS - 1) / LT_ROWS), (unsigned)((units + G - 1) / G), (unsigned)nb);
  if (splits > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(LT_THREADS * G);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)splits;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, q, (const T*)cache, Tcap, cu, rows, t_pos, (T*)out, H, R, window, scale, by_head, splits, nbuf);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(latent_attn_tile_kernel)");
  } else {
    kern<<<grid, LT_THREADS * G, smem, st>>>(q, (const T*)cache, Tcap, cu, rows, t_pos, (T*)out, H, R, window, scale, by_head, 1, nbuf);
  }
  B200P_LAUNCH_CHECK("latent_attn_tile_kernel");
  return B200P_OK;
}

extern "C" int b200p_latent_attn_set_groups(int groups) {
  g_lt_groups = groups < 0 ? 0 : groups > LT_MAX_GROUPS ? LT_MAX_GROUPS : groups;
  return B200P_OK;
}

extern "C" int b200p_latent_attn_set_buffers(int buffers) {
  g_lt_nbuf = buffers == 1 || buffers == 2 ? buffers : 0;
  return B200P_OK;
}

extern "C" int b200p_latent_attn_set_splits(int splits) {
  g_lt_splits = splits < 0 ? 0 : splits > 8 ? 8 : splits;
  return B200P_OK;
}

extern "C" int b200p_latent_attn_tiles_supported(int R, int dtype) {
  return (dtype == B200P_F16 || dtype == B200P_BF16) && R % 32 == 0 && R <= 32 * LT_WIDE_NT ? 1 : 0;
}

extern "C" int b200p_latent_attn_tiles(const float* q, const void* cache, int64_t Tcap, const int32_t* cu, const int32_t* rows,
                                       const int32_t* t_pos, void* out, int nb, int max_n, int H, int R, int64_t window,
                                       float scale, int dtype, void* stream) {
  B200P_REQUIRE(q && cache && cu && rows && t_pos && out, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(b200p_latent_attn_tiles_supported(R, dtype), B200P_ERR_ARG, "the tile kernel needs a 16-bit type and a rank that is a multiple of 32, at most %d", 32 * LT_WIDE_NT);
  B200P_REQUIRE(nb > 0 && nb < 65536 && H > 0 && H < 65536 && max_n > 0, B200P_ERR_ARG, "bad batch geometry");
  B200P_REQUIRE(aligned(cache, 16) && aligned(q, 16) && aligned(out, 4), B200P_ERR_ALIGN, "cache and q must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  if (R > 32 * LT_MAX_NT) {
    if (dtype == B200P_F16) return latent_attn_tile_launch<__half, LT_WIDE_NT>(q, cache, Tcap, cu, rows, t_pos, out, nb, max_n, H, R, window, scale, st);
    return latent_attn_tile_launch<__nv_bfloat16, LT_WIDE_NT>(q, cache, Tcap, cu, rows, t_pos, out, nb, max_n, H, R, window, scale, st);
  }
  if (dtype == B200P_F16) return latent_attn_tile_launch<__half, LT_MAX_NT>(q, cache, Tcap, cu, rows, t_pos, out, nb, max_n, H, R, window, scale, st);
  return latent_attn_tile_launch<__nv_bfloat16, LT_MAX_NT>(q, cache, Tcap, cu, rows, t_pos, out, nb, max_n, H, R, window, scale, st);
}

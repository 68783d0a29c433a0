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

// ---- 16-bit caches on the tensor cores ----------------------------------------------------------------------------------------
// K / V tiles of 64 keys stream global -> shared with cp.async (two stages, XOR-swizzled 16-byte pieces); a key row holds the
// vectors of both maps side by side, so one staged tile serves both.  S = Q K^T and O += P V run on mma.sync m16n8k16 with the
// fp32 online softmax in registers, in base-2 units.  A warp owns 16 query rows of ONE map:
//   prompts (DECODE = false)  4 warps = 2 row blocks x 2 maps: 32 consecutive tokens of entry blockIdx.z for head blockIdx.y;
//                             the second map's warps hand lambda a_2 over through shared memory and the first map's warps
//                             finish the head: a_1 - lambda a_2, the division by the root mean square, the store;
//   decode (DECODE = true)    2 warps = 2 maps; the 16 rows are the query heads of key/value head blockIdx.y for the single
//                             token of entry blockIdx.z, and the CTA takes the blockIdx.x-th share of the key tiles: it writes
//                             unnormalised partial sums (o, running max, sum) that diff_attn_merge_kernel combines.
// A row whose chunk begins after a tile's last key sees nothing of that tile: its running maximum stays -inf and the
// exponentials are taken against 0 instead, which leaves sums and accumulators at zero.
constexpr int DT_KT = 64, DT_STAGES = 2, DT_QT = 32;
constexpr float DA_LOG2E = 1.4426950408889634f;
constexpr int DIFF_ATTN_MAX_SPLITS = 16;
constexpr int DIFF_ATTN_TILES_MIN_TOKENS = 4;   // shorter portions take the per-token kernel

// 16-byte piece `ch` of row `key` sits at piece swz(key, ch) of the row: rows of 8 pieces and more rotate by the row number, rows of
// 4 pieces (64 bytes, two rows per 128-byte line) by half of it, so the 8 rows of an ldmatrix fall into different banks
template <int CH>
__device__ __forceinline__ int swz(int key, int ch) { return CH >= 8 ? (ch ^ (key & 7)) : (ch ^ ((key >> 1) & 3)); }

template <typename T, int D, int DV, bool DECODE>
__global__ void __launch_bounds__(DECODE ? 64 : 128)
diff_attn_tile_kernel(const float* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc, int64_t Tcap,
                      const int32_t* __restrict__ cu, const int32_t* __restrict__ rows, const int32_t* __restrict__ t_pos,
                      int64_t chunk, float lambda, float eps, float post, T* __restrict__ out, int64_t ld_out, int H, int G,
                      float* __restrict__ part_o, float* __restrict__ part_ms) {
  constexpr int NT = DECODE ? 64 : 128;
  constexpr int KD = 2 * D;                                         // elements of a key row: both maps
  constexpr int KROW = KD * 2, VROW = DV * 2;                       // bytes per staged row
  constexpr int K_BYTES = DT_KT * KROW, V_BYTES = DT_KT * VROW, STAGE_BYTES = K_BYTES + V_BYTES;
  constexpr int KCH = KD / 8, VCH = DV / 8;                         // 16-byte pieces per row
  extern __shared__ __align__(128) uint8_t dt_smem[];
  const int e = blockIdx.z;
  const int t_first = cu[e], n_e = cu[e + 1] - t_first;
  const int q0 = DECODE ? 0 : blockIdx.x * DT_QT;
  if (q0 >= n_e) return;                                            // the same for every thread of the CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int map = warp & 1, rb = warp >> 1;
  const int quad_row = lane >> 2, qc = lane & 3;
  const int per = H / G;
  const int g = DECODE ? blockIdx.y : blockIdx.y / per;
  const int p_first = t_pos[t_first];                               // positions of an entry's tokens are consecutive
  const int l0 = q0 + rb * 16 + quad_row, l1 = l0 + 8;              // this thread's two rows: tokens (prompts) or heads (decode)
  const int n_rows = DECODE ? per : n_e;
  const int lc0 = min(l0, n_rows - 1), lc1 = min(l1, n_rows - 1);   // rows past the end compute a valid row, not stored
  const int h0 = DECODE ? g * per + lc0 : blockIdx.y, h1 = DECODE ? g * per + lc1 : blockIdx.y;
  const int tk0 = DECODE ? t_first : t_first + lc0, tk1 = DECODE ? t_first : t_first + lc1;
  const int pos0 = DECODE ? p_first : p_first + lc0, pos1 = DECODE ? p_first : p_first + lc1;
  const int lo0 = (int)chunk_start(pos0, chunk), lo1 = (int)chunk_start(pos1, chunk);     // first key each row sees
  const int kend = DECODE ? p_first + 1 : p_first + min(n_e, q0 + DT_QT);                 // keys any row of this CTA may see
  const int kbegin = (int)chunk_start(p_first + q0, chunk);
  const int t_begin = kbegin / DT_KT, t_end = (kend + DT_KT - 1) / DT_KT;
  int tile_lo = t_begin, tile_hi = t_end;
  if (DECODE) {
    const int share = (t_end - t_begin + gridDim.x - 1) / gridDim.x;
    tile_lo = t_begin + blockIdx.x * share;
    tile_hi = min(t_end, tile_lo + share);
  }

  uint32_t qf[D / 16][4];
  {
    const float* p0 = q + ((int64_t)tk0 * H + h0) * KD + map * D;
    const float* p1 = q + ((int64_t)tk1 * H + h1) * KD + map * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const float2 a0 = *reinterpret_cast<const float2*>(p0 + ks * 16 + 2 * qc), a1 = *reinterpret_cast<const float2*>(p1 + ks * 16 + 2 * qc);
      const float2 b0 = *reinterpret_cast<const float2*>(p0 + ks * 16 + 8 + 2 * qc), b1 = *reinterpret_cast<const float2*>(p1 + ks * 16 + 8 + 2 * qc);
      qf[ks][0] = pack2<T>(a0.x, a0.y);
      qf[ks][1] = pack2<T>(a1.x, a1.y);
      qf[ks][2] = pack2<T>(b0.x, b0.y);
      qf[ks][3] = pack2<T>(b1.x, b1.y);
    }
  }
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dt_smem);
  const int64_t row = rows[e];
  const T* kbase = kc + (row * G + g) * Tcap * KD;
  const T* vbase = vc + (row * G + g) * Tcap * DV;
  auto issue_tile = [&](int tile, int stage) {
    const uint32_t ks = sbase + stage * STAGE_BYTES, vs = ks + K_BYTES;
    const int key0 = tile * DT_KT;
#pragma unroll
    for (int i = 0; i < DT_KT * KCH / NT; ++i) {
      const int idx = i * NT + threadIdx.x;
      const int key = idx / KCH, ch = idx % KCH;
      const bool ok = key0 + key < kend;
      cp_async16(ks + (uint32_t)(key * KROW + (swz<KCH>(key, ch) << 4)), kbase + (int64_t)(key0 + (ok ? key : 0)) * KD + ch * 8, ok);
    }
#pragma unroll
    for (int i = 0; i < DT_KT * VCH / NT; ++i) {
      const int idx = i * NT + threadIdx.x;
      const int key = idx / VCH, ch = idx % VCH;
      const bool ok = key0 + key < kend;
      cp_async16(vs + (uint32_t)(key * VROW + (swz<VCH>(key, ch) << 4)), vbase + (int64_t)(key0 + (ok ? key : 0)) * DV + ch * 8, ok);
    }
  };

  float o[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, s0 = 0.f, s1 = 0.f;

  if (tile_lo < tile_hi) issue_tile(tile_lo, 0);
  cp_async_commit();
  for (int it = tile_lo; it < tile_hi; ++it) {
    const int stage = (it - tile_lo) & 1;
    if (it + 1 < tile_hi) issue_tile(it + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t ks = sbase + stage * STAGE_BYTES, vs = ks + K_BYTES;
    const int key0 = it * DT_KT;
    const int mat = lane >> 3, r = lane & 7;
    float sc[DT_KT / 8][4];
#pragma unroll
    for (int nt = 0; nt < DT_KT / 8; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
    for (int np = 0; np < DT_KT / 16; ++np) {
      const int key = 16 * np + r + 8 * (mat >> 1);
#pragma unroll
      for (int kstep = 0; kstep < D / 16; ++kstep) {
        const int ch = map * (D / 8) + 2 * kstep + (mat & 1);
        uint32_t bf[4];
        ldsm_x4(ks + (uint32_t)(key * KROW + (swz<KCH>(key, ch) << 4)), bf);
        mma16816<T>(sc[2 * np], qf[kstep], bf[0], bf[1]);
        mma16816<T>(sc[2 * np + 1], qf[kstep], bf[2], bf[3]);
      }
    }
    float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < DT_KT / 8; ++nt) {
      const int kcol = key0 + 8 * nt + 2 * qc;
      sc[nt][0] = (kcol <= pos0 && kcol >= lo0) ? sc[nt][0] * DA_LOG2E : -INFINITY;
      sc[nt][1] = (kcol + 1 <= pos0 && kcol + 1 >= lo0) ? sc[nt][1] * DA_LOG2E : -INFINITY;
      sc[nt][2] = (kcol <= pos1 && kcol >= lo1) ? sc[nt][2] * DA_LOG2E : -INFINITY;
      sc[nt][3] = (kcol + 1 <= pos1 && kcol + 1 >= lo1) ? sc[nt][3] * DA_LOG2E : -INFINITY;
      t0 = fmaxf(t0, fmaxf(sc[nt][0], sc[nt][1]));
      t1 = fmaxf(t1, fmaxf(sc[nt][2], sc[nt][3]));
    }
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1)); t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    const float mn0 = fmaxf(m0, t0), mn1 = fmaxf(m1, t1);
    const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;      // nothing seen yet: all terms 0
    const float corr0 = exp2f(m0 - ref0), corr1 = exp2f(m1 - ref1);
    m0 = mn0; m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < DT_KT / 8; ++nt) {
      sc[nt][0] = exp2f(sc[nt][0] - ref0); sc[nt][1] = exp2f(sc[nt][1] - ref0);
      sc[nt][2] = exp2f(sc[nt][2] - ref1); sc[nt][3] = exp2f(sc[nt][3] - ref1);
      ps0 += sc[nt][0] + sc[nt][1];
      ps1 += sc[nt][2] + sc[nt][3];
    }
    s0 = s0 * corr0 + ps0;
    s1 = s1 * corr1 + ps1;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) { o[j][0] *= corr0; o[j][1] *= corr0; o[j][2] *= corr1; o[j][3] *= corr1; }
#pragma unroll
    for (int kk = 0; kk < DT_KT / 16; ++kk) {
      uint32_t pf[4];
      pf[0] = pack2<T>(sc[2 * kk][0], sc[2 * kk][1]);
      pf[1] = pack2<T>(sc[2 * kk][2], sc[2 * kk][3]);
      pf[2] = pack2<T>(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
      pf[3] = pack2<T>(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
      const int key = 16 * kk + r + 8 * (mat & 1);
#pragma unroll
      for (int jp = 0; jp < DV / 16; ++jp) {
        const int ch = 2 * jp + (mat >> 1);
        uint32_t bf[4];
        ldsm_x4_trans(vs + (uint32_t)(key * VROW + (swz<VCH>(key, ch) << 4)), bf);
        mma16816<T>(o[2 * jp], pf, bf[0], bf[1]);
        mma16816<T>(o[2 * jp + 1], pf, bf[2], bf[3]);
      }
    }
    __syncthreads();                                 // this stage is refilled by the next iteration's prefetch
  }
  cp_async_wait<0>();
  s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
  if constexpr (DECODE) {
    const int64_t b0 = (((int64_t)e * H + h0) * 2 + map) * gridDim.x + blockIdx.x, b1 = (((int64_t)e * H + h1) * 2 + map) * gridDim.x + blockIdx.x;
    if (qc == 0) {
      if (l0 < per) { part_ms[b0 * 2] = m0; part_ms[b0 * 2 + 1] = s0; }       // a share without tiles leaves (-inf, 0)
      if (l1 < per) { part_ms[b1 * 2] = m1; part_ms[b1 * 2 + 1] = s1; }
    }
    if (tile_lo >= tile_hi) return;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
      const int c = 8 * j + 2 * qc;
      if (l0 < per) *reinterpret_cast<float2*>(part_o + b0 * DV + c) = make_float2(o[j][0], o[j][1]);
      if (l1 < per) *reinterpret_cast<float2*>(part_o + b1 * DV + c) = make_float2(o[j][2], o[j][3]);
    }
    return;
  } else {
    // every row of a prompt tile sees at least its own key: the sums are positive.  The staged tiles are done with (the loop
    // ended on a barrier): their room carries lambda a_2 from the second map's warps to the first map's.
    float* xch = reinterpret_cast<float*>(dt_smem) + rb * 16 * (DV + 2);
    const float inv0 = 1.f / s0, inv1 = 1.f / s1;
    if (map == 1) {
#pragma unroll
      for (int j = 0; j < DV / 8; ++j) {
        const int c = 8 * j + 2 * qc;
        *reinterpret_cast<float2*>(xch + quad_row * (DV + 2) + c) = make_float2(o[j][0] * inv0 * lambda, o[j][1] * inv0 * lambda);
        *reinterpret_cast<float2*>(xch + (quad_row + 8) * (DV + 2) + c) = make_float2(o[j][2] * inv1 * lambda, o[j][3] * inv1 * lambda);
      }
    }
    __syncthreads();
    if (map == 1) return;
    float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
      const int c = 8 * j + 2 * qc;
      const float2 x0 = *reinterpret_cast<const float2*>(xch + quad_row * (DV + 2) + c);
      const float2 x1 = *reinterpret_cast<const float2*>(xch + (quad_row + 8) * (DV + 2) + c);
      o[j][0] = o[j][0] * inv0 - x0.x; o[j][1] = o[j][1] * inv0 - x0.y;
      o[j][2] = o[j][2] * inv1 - x1.x; o[j][3] = o[j][3] * inv1 - x1.y;
      ss0 += o[j][0] * o[j][0] + o[j][1] * o[j][1];
      ss1 += o[j][2] * o[j][2] + o[j][3] * o[j][3];
    }
    float mul0 = post, mul1 = post;
    if (eps >= 0.f) {
      ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
      ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
      mul0 *= 1.f / sqrtf(ss0 / (float)DV + eps);
      mul1 *= 1.f / sqrtf(ss1 / (float)DV + eps);
    }
    T* o0 = out + (int64_t)tk0 * ld_out + (int64_t)h0 * DV;
    T* o1 = out + (int64_t)tk1 * ld_out + (int64_t)h1 * DV;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
      const int c = 8 * j + 2 * qc;
      if (l0 < n_e) *reinterpret_cast<uint32_t*>(o0 + c) = pack2<T>(o[j][0] * mul0, o[j][1] * mul0);
      if (l1 < n_e) *reinterpret_cast<uint32_t*>(o1 + c) = pack2<T>(o[j][2] * mul1, o[j][3] * mul1);
    }
  }
}

// per (entry, head): a_m = (sum_s o_s 2^(m_s - m)) / (sum_s l_s 2^(m_s - m)) for both maps, then the head's output as above
template <typename T>
__global__ void diff_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ms,
                                       const int32_t* __restrict__ cu, float lambda, float eps, float post, T* __restrict__ out,
                                       int64_t ld_out, int H, int dv, int splits) {
  __shared__ float red[4];
  const int e = blockIdx.x, h = blockIdx.y;
  if (cu[e + 1] - cu[e] <= 0) return;
  float mx[2], inv[2];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp) {
    const int64_t base = (((int64_t)e * H + h) * 2 + mp) * splits;
    float m = -INFINITY, den = 0.f;
    for (int sidx = 0; sidx < splits; ++sidx) m = fmaxf(m, part_ms[(base + sidx) * 2]);
    for (int sidx = 0; sidx < splits; ++sidx) {
      const float ms = part_ms[(base + sidx) * 2];
      if (ms != -INFINITY) den += part_ms[(base + sidx) * 2 + 1] * exp2f(ms - m);
    }
    mx[mp] = m;
    inv[mp] = (mp == 0 ? 1.f : lambda) / den;
  }
  float ss = 0.f, mine = 0.f;                        // one value per thread: dv <= blockDim.x
  const int c = threadIdx.x;
  if (c < dv) {
    float a[2];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
      const int64_t base = (((int64_t)e * H + h) * 2 + mp) * splits;
      float acc = 0.f;
      for (int sidx = 0; sidx < splits; ++sidx) {
        const float ms = part_ms[(base + sidx) * 2];
        if (ms != -INFINITY) acc = fmaf(part_o[(base + sidx) * dv + c], exp2f(ms - mx[mp]), acc);
      }
      a[mp] = acc * inv[mp];
    }
    mine = a[0] - a[1];
    ss = mine * mine;
  }
  float mul = post;
  if (eps >= 0.f) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
    mul *= 1.f / sqrtf(tot / (float)dv + eps);
  }
  if (c < dv) out[(int64_t)cu[e] * ld_out + (int64_t)h * dv + c] = Tr<T>::from_f(mine * mul);
}

template <typename T, int D, int DV>
static int diff_attn_tiles_launch(const float* q, const void* kc, const void* vc, int64_t Tcap, const int32_t* cu, const int32_t* rows,
                                  const int32_t* t_pos, int64_t chunk, float lambda, float eps, float post, void* out, int64_t ld_out,
                                  int nb, int max_n, int H, int G, float* ws, size_t ws_bytes, cudaStream_t st) {
  constexpr int stage_bytes = DT_STAGES * DT_KT * (2 * D + DV) * 2, xch_bytes = 2 * 16 * (DV + 2) * 4;
  constexpr int smem = stage_bytes > xch_bytes ? stage_bytes : xch_bytes;
  if (max_n == 1) {
    // decode: shares of the key tiles per (entry, key/value head), as many as keep several CTAs per SM busy and the workspace holds
    auto kern = diff_attn_tile_kernel<T, D, DV, true>;
    static bool attr_set = false;
    if (smem > 48 * 1024 && !attr_set) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(diff_attn_tile_kernel)");
      attr_set = true;
    }
    const size_t per_split = (size_t)nb * H * 2 * (DV + 2) * sizeof(float);
    int splits = (int)((8 * 148 + (int64_t)nb * G - 1) / ((int64_t)nb * G));
    splits = splits < 1 ? 1 : splits > DIFF_ATTN_MAX_SPLITS ? DIFF_ATTN_MAX_SPLITS : splits;
    if ((size_t)splits * per_split > ws_bytes) splits = (int)(ws_bytes / per_split);
    if (splits < 1) return 1;                                     // no room for partial sums: the caller takes the per-token kernel
    float* part_o = ws;
    float* part_ms = ws + (size_t)nb * H * 2 * splits * DV;
    dim3 grid((unsigned)splits, (unsigned)G, (unsigned)nb);
    kern<<<grid, 64, smem, st>>>(q, (const T*)kc, (const T*)vc, Tcap, cu, rows, t_pos, chunk, lambda, eps, post, (T*)out, ld_out, H, G,
                                 part_o, part_ms);
    B200P_LAUNCH_CHECK("diff_attn_tile_kernel");
    diff_attn_merge_kernel<T><<<dim3((unsigned)nb, (unsigned)H), DV >= 128 ? 128 : DV >= 64 ? 64 : 32, 0, st>>>(
        part_o, part_ms, cu, lambda, eps, post, (T*)out, ld_out, H, DV, splits);
    B200P_LAUNCH_CHECK("diff_attn_merge_kernel");
    return B200P_OK;
  }
  auto kern = diff_attn_tile_kernel<T, D, DV, false>;
  if (smem > 48 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(diff_attn_tile_kernel)");
      attr_set = true;
    }
  }
  dim3 grid((unsigned)((max_n + DT_QT - 1) / DT_QT), (unsigned)H, (unsigned)nb);
  kern<<<grid, 128, smem, st>>>(q, (const T*)kc, (const T*)vc, Tcap, cu, rows, t_pos, chunk, lambda, eps, post, (T*)out, ld_out, H, G,
                                nullptr, nullptr);
  B200P_LAUNCH_CHECK("diff_attn_tile_kernel");
  return B200P_OK;
}

// whether the tile kernel takes these sizes (16-bit caches, two maps, vector and value sizes of 32, 64 or 128)
static bool diff_attn_tiles_ok(int maps, int d, int dv, int dtype) {
  return (dtype == B200P_F16 || dtype == B200P_BF16) && maps == 2 && (d == 32 || d == 64 || d == 128) && (dv == 32 || dv == 64 || dv == 128);
}

template <typename T>
static int diff_attn_tiles(const float* q, const void* kc, const void* vc, int64_t Tcap, const int32_t* cu, const int32_t* rows,
                           const int32_t* t_pos, int64_t chunk, float lambda, float eps, float post, void* out, int64_t ld_out, int nb,
                           int max_n, int H, int G, int d, int dv, float* ws, size_t ws_bytes, cudaStream_t st) {
#define DT_CASE(D_, DV_) \
  if (d == D_ && dv == DV_) \
    return diff_attn_tiles_launch<T, D_, DV_>(q, kc, vc, Tcap, cu, rows, t_pos, chunk, lambda, eps, post, out, ld_out, nb, max_n, H, G, ws, ws_bytes, st)
  DT_CASE(32, 32); DT_CASE(32, 64); DT_CASE(32, 128);
  DT_CASE(64, 32); DT_CASE(64, 64); DT_CASE(64, 128);
  DT_CASE(128, 32); DT_CASE(128, 64); DT_CASE(128, 128);
#undef DT_CASE
  set_error("tile attention: unsupported sizes");
  return B200P_ERR_ARG;
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
  // prompts (entries of several tokens, described by cu / rows) of 16-bit models run on the tensor-core tile kernel, and so do
  // decode steps (one token per entry) whose heads per key/value head fit a 16-row tile, given room for partial sums
  const bool prompts = max_n >= DIFF_ATTN_TILES_MIN_TOKENS;
  const bool decode = max_n == 1 && H / G <= 16 && workspace && aligned(workspace, 16);
  if (cu && rows && nb > 0 && (prompts || decode) && diff_attn_tiles_ok(maps, d, dv, dtype) && ld_out % 2 == 0 && aligned(kcache, 16) &&
      aligned(vcache, 16) && aligned(out, 4) && aligned(q, 8) && nb < 65536 && H < 65536) {
    const int rc = dtype == B200P_F16
        ? diff_attn_tiles<__half>(q, kcache, vcache, Tcap, cu, rows, t_pos, chunk, lambda, eps, post, out, ld_out, nb, max_n, H, G, d, dv,
                                  (float*)workspace, workspace_bytes, st)
        : diff_attn_tiles<__nv_bfloat16>(q, kcache, vcache, Tcap, cu, rows, t_pos, chunk, lambda, eps, post, out, ld_out, nb, max_n, H, G, d,
                                         dv, (float*)workspace, workspace_bytes, st);
    if (rc != 1) return rc;
  }
  switch (dtype) {
    case B200P_F32: return diff_attn_generic<float>(q, kcache, vcache, Tcap, t_row, t_pos, chunk, maps, lambda, eps, post, out, ld_out, M, H, G, d, dv, st);
    case B200P_F16: return diff_attn_generic<__half>(q, kcache, vcache, Tcap, t_row, t_pos, chunk, maps, lambda, eps, post, out, ld_out, M, H, G, d, dv, st);
    case B200P_BF16: return diff_attn_generic<__nv_bfloat16>(q, kcache, vcache, Tcap, t_row, t_pos, chunk, maps, lambda, eps, post, out, ld_out, M, H, G, d, dv, st);
    default: set_error("bad dtype %d", dtype); return B200P_ERR_ARG;
  }
}

extern "C" size_t b200p_diff_attn_workspace_bytes(int64_t nb, int H, int maps, int dv) {
  return (size_t)nb * H * maps * DIFF_ATTN_MAX_SPLITS * (dv + 2) * sizeof(float);
}

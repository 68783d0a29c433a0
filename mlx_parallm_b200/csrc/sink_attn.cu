// Causal attention over a ragged batch for designs without a positional rotation: grouped query heads, separate key and value
// sizes, rms-normed queries and keys, a query temperature that depends on the position, a bias linear in the distance
// (score - slope_h (i - j)) and a learned per-head "sink": one extra term exp(sink_h) in the softmax denominator that adds
// nothing to the output, so it only takes probability mass away from the keys.
//   sink_attn_prep_kernel   norms, temperature and scale on q; normed k and v into the cache at (row, position)     (per token)
//   sink_attn_kernel        one token x the query heads of one key/value head, fp32 throughout, any sizes           (per token)
//   sink_attn_tile_kernel   16 query rows per warp on mma.sync over 64-key tiles: 64 tokens of a prompt for one head, or the
//                           heads of a key/value head for one decoded token with the keys split over CTAs              (16-bit caches)
//   sink_attn_merge_kernel  the decode step's partial sums and the sink                                               (per token, head)
// The softmax starts from the sink: running maximum = sink, running sum = 1 (the sink's own term), accumulator = 0; every key
// then joins by the usual online update, so a query that sees few keys is damped exactly as the definition says.
// Every option is a parameter: no norm (weights NULL), no temperature (coef 0), no bias (slope_log2 0), no sink (NULL).
// A second family of options (ScoreRule; b200p_window_attn) serves designs that cap their scores, cap tanh(s / cap), take a
// logarithmic distance penalty r1_h ln(1 + r2_h (i - j)) off them, see a sliding window 0 <= i - j < window, and gate the
// heads' outputs with a sigmoid:
//   window_attn_prep_kernel  a short causal convolution over time on the q and k projections (carried inputs like the delta
//                            rule's), q scaled into fp32, k into the cache                                          (per token)
#include "common.cuh"
#include "mma_util.cuh"

namespace b200p {

// What happens to a score s = q . k (q already scaled) of the query at position p and the key at position j, and to the output.
struct ScoreRule {
  float cap;            // > 0: s <- cap tanh(s / cap)
  const float* r1;      // per head: s <- s - r1[h] ln(1 + r2[h] (p - j)); NULL: none
  const float* r2;
  int window;           // > 0: only keys with 0 <= p - j < window are seen
  const float* gate;    // fp32 [M, ldg]: out[t, h, c] *= sigmoid(gate[t, h dv + c]); NULL: none
  int64_t ldg;
  int table;            // prompts on the tile kernel: entries of the per-CTA penalty table in shared memory (0: computed per score)
};

__device__ __forceinline__ float ruled_score(float s, const ScoreRule& rule, float r1, float r2, float dist) {
  if (rule.cap > 0.f) s = rule.cap * tanhf(s / rule.cap);
  if (rule.r1) s -= r1 * log1pf(r2 * dist);
  return s;
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
// The same rule on the special-function unit, for the 16-bit tile kernel whose probabilities are rounded to 16 bits anyway:
// tanh x = 1 - 2 / (1 + e^2x) (absolute error near 1e-7, so cap tanh(s / cap) is off by about cap * 1e-7), ln through lg2.
// The penalty of a distance comes from `tab` (filled once per CTA: a prompt tile serves one head) where there is one.
// Five instructions for the cap: cap tanh(s / cap) = cap - 2 cap / (1 + 2^(s 2 log2(e) / cap)) with the constants formed once.
__device__ __forceinline__ float ex2_approx(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcp_approx(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float ruled_score_fast(float s, const ScoreRule& rule, float k_exp, float cap2, float r1, float r2, int dist,
                                                  const float* tab) {
  if (rule.cap > 0.f) s = fmaf(-cap2, rcp_approx(1.f + ex2_approx(s * k_exp)), rule.cap);
  if (tab) s -= tab[dist];
  else if (rule.r1) s -= r1 * __logf(fmaf(r2, (float)dist, 1.f));
  return s;
}
__device__ __forceinline__ float sigmoid_fast(float z) { return __fdividef(1.f, 1.f + __expf(-z)); }

// slope of head h: 2^(slope_log2 * (h + 1) / H); slope_log2 = 0 means no bias
__device__ __forceinline__ float head_slope(float slope_log2, int h, int H) {
  return slope_log2 == 0.f ? 0.f : exp2f(slope_log2 * (float)(h + 1) / (float)H);
}

template <typename T>
__global__ void sink_attn_prep_kernel(const float* __restrict__ proj, int64_t ldp, int64_t col_q, int64_t col_k, int64_t col_v,
                                      const float* __restrict__ wq, const float* __restrict__ wk, float eps, float scale,
                                      float temp_coef, float temp_every, float* __restrict__ q_out, T* __restrict__ kcache,
                                      T* __restrict__ vcache, int64_t Tcap, const int32_t* __restrict__ t_row,
                                      const int32_t* __restrict__ t_pos, int H, int G, int dk, int dv) {
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float* pt = proj + t * ldp;
  const int64_t pos = t_pos[t], row = t_row[t];
  float qmul = scale;
  if (temp_coef != 0.f) qmul *= 1.f + temp_coef * logf(floorf((float)(pos + 1) / temp_every) + 1.f);
  const bool in_cache = pos < Tcap;                                // the host sizes the cache first; never write outside it
  for (int hd = warp; hd < H + G; hd += nw) {                      // query heads, then key heads
    const bool is_q = hd < H;
    const float* src = is_q ? pt + col_q + (int64_t)hd * dk : pt + col_k + (int64_t)(hd - H) * dk;
    const float* w = is_q ? wq : wk;
    float inv = 1.f;
    if (w) {
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) ss = fmaf(src[i], src[i], ss);
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / (float)dk + eps);
    }
    if (is_q) {
      float* dst = q_out + (t * H + hd) * dk;
      for (int i = lane; i < dk; i += 32) dst[i] = src[i] * inv * (w ? w[i] : 1.f) * qmul;
    } else if (in_cache) {
      T* dst = kcache + ((row * G + (hd - H)) * Tcap + pos) * dk;
      for (int i = lane; i < dk; i += 32) dst[i] = Tr<T>::from_f(src[i] * inv * (w ? w[i] : 1.f));
    }
  }
  if (in_cache) {
    for (int c = threadIdx.x; c < G * dv; c += blockDim.x) {
      const int g = c / dv, i = c % dv;
      vcache[((row * G + g) * Tcap + pos) * dv + i] = Tr<T>::from_f(pt[col_v + c]);
    }
  }
}

constexpr int SINK_ATTN_TILES_MIN_TOKENS = 4;   // shorter portions (and decode steps) take the per-token kernel
constexpr int SA_KEYS = 32;        // keys per staged chunk: one per lane in the score phase
constexpr int SA_MAX_HEADS = 8;    // query heads (warps) per CTA
constexpr int SA_MAX_VL = 16;      // value elements per lane: dv <= 512

// CTA = (token t, key/value head g, block of up to 8 of its query heads); warp = query head.
template <typename T>
__global__ void __launch_bounds__(SA_MAX_HEADS * 32)
sink_attn_kernel(const float* __restrict__ q, const T* __restrict__ kcache, const T* __restrict__ vcache, int64_t Tcap,
                 const int32_t* __restrict__ t_row, const int32_t* __restrict__ t_pos, const float* __restrict__ sink,
                 float slope_log2, T* __restrict__ out, int64_t ld_out, float out_scale, int H, int G, int dk, int dv,
                 ScoreRule rule) {
  extern __shared__ float sa_sm[];
  const int KS = dk + 1;                                           // padded row: lane j reads row j without bank conflicts
  float* ks = sa_sm;                                               // [SA_KEYS][KS]
  float* vs = ks + SA_KEYS * KS;                                   // [SA_KEYS][dv]
  float* qs = vs + SA_KEYS * dv;                                   // [warps][dk]
  const int64_t t = blockIdx.x;
  const int g = blockIdx.y, per = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int hl = blockIdx.z * nw + warp;                           // head inside the group
  const bool head_ok = hl < per;
  const int h = g * per + hl;
  const int64_t pos = t_pos[t];
  const T* kb = kcache + ((int64_t)t_row[t] * G + g) * Tcap * dk;
  const T* vb = vcache + ((int64_t)t_row[t] * G + g) * Tcap * dv;
  if (head_ok)
    for (int i = lane; i < dk; i += 32) qs[warp * dk + i] = q[(t * H + h) * dk + i];
  const float slope = head_ok ? head_slope(slope_log2, h, H) : 0.f;
  float acc[SA_MAX_VL];
#pragma unroll
  for (int i = 0; i < SA_MAX_VL; ++i) acc[i] = 0.f;
  float mx = (head_ok && sink) ? sink[h] : -INFINITY;
  float den = (head_ok && sink) ? 1.f : 0.f;
  const float r1 = (head_ok && rule.r1) ? rule.r1[h] : 0.f, r2 = (head_ok && rule.r1) ? rule.r2[h] : 0.f;
  const int64_t first = (rule.window > 0 && pos - rule.window + 1 > 0) ? pos - rule.window + 1 : 0;
  for (int64_t j0 = first; j0 <= pos; j0 += SA_KEYS) {
    const int nk = (int)min((int64_t)SA_KEYS, pos + 1 - j0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nk * dk; idx += blockDim.x) {
      const int kk = idx / dk, i = idx % dk;
      ks[kk * KS + i] = Tr<T>::to_f(kb[(j0 + kk) * dk + i]);
    }
    for (int idx = threadIdx.x; idx < nk * dv; idx += blockDim.x) vs[idx] = Tr<T>::to_f(vb[j0 * dv + idx]);
    __syncthreads();
    if (!head_ok) continue;
    float s = -INFINITY;
    if (lane < nk) {
      const float* kr = ks + lane * KS;
      const float* qr = qs + warp * dk;
      float d = 0.f;
      for (int i = 0; i < dk; ++i) d = fmaf(qr[i], kr[i], d);
      s = ruled_score(d, rule, r1, r2, (float)(pos - (j0 + lane))) - slope * (float)(pos - (j0 + lane));
    }
    const float nmx = fmaxf(mx, warp_max(s));
    const float corr = expf(mx - nmx);                             // 0 on the first chunk without a sink (mx = -inf)
    const float p = lane < nk ? expf(s - nmx) : 0.f;
    den = den * corr + warp_sum(p);
    mx = nmx;
#pragma unroll
    for (int i = 0; i < SA_MAX_VL; ++i) acc[i] *= corr;
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const float* vr = vs + kk * dv;
#pragma unroll
      for (int i = 0; i < SA_MAX_VL; ++i) {
        const int c = i * 32 + lane;
        if (c < dv) acc[i] = fmaf(pk, vr[c], acc[i]);
      }
    }
  }
  if (!head_ok) return;
  const float inv = out_scale / den;
#pragma unroll
  for (int i = 0; i < SA_MAX_VL; ++i) {
    const int c = i * 32 + lane;
    if (c < dv) {
      const float gz = rule.gate ? sigmoid_f(rule.gate[t * rule.ldg + (int64_t)h * dv + c]) : 1.f;
      out[t * ld_out + (int64_t)h * dv + c] = Tr<T>::from_f(acc[i] * inv * gz);
    }
  }
}

// q and k of the windowed attention: projections [q (H dk) | k (G dk)] from column col_q of proj pass a causal convolution over
// time (conv_w [taps, C], tap by tap, the last tap the current token's; conv_state [rows, taps-1, C] the inputs of earlier steps, zeros before the
// sequence's start); q_out = that * scale (fp32), the keys go to the cache.
template <typename T, int V>
__global__ void window_attn_prep_kernel(const float* __restrict__ proj, int64_t ldp, int64_t col_q, const float* __restrict__ conv_w,
                                        const float* __restrict__ conv_state, int taps, float scale, float* __restrict__ q_out,
                                        T* __restrict__ kcache, int64_t Tcap, const int32_t* __restrict__ t_row,
                                        const int32_t* __restrict__ t_pos, const int32_t* __restrict__ t_off, int H, int G, int dk) {
  const int64_t t = blockIdx.x;
  const int C = (H + G) * dk, Cq = H * dk;
  const int row = t_row[t], pos = t_pos[t], off = t_off[t];
  const float* pt = proj + t * ldp + col_q;
  // V neighbouring channels per thread (V == 4: 16-byte accesses; the channels of a thread then lie in one head)
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * V; c < C; c += gridDim.y * blockDim.x * V) {
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
    for (int j = 0; j < taps; ++j) {                 // tap j multiplies the input d = taps-1-j tokens back
      const int d = taps - 1 - j;
      if (d > pos) continue;                         // before the sequence
      const float* in = d <= off ? pt + c - (int64_t)d * ldp : conv_state + ((int64_t)row * (taps - 1) + (taps - 1 + off - d)) * C + c;
      const float* wt = conv_w + (int64_t)j * C + c;
      if constexpr (V == 4) {
        const float4 a = *reinterpret_cast<const float4*>(in), w4 = *reinterpret_cast<const float4*>(wt);
        acc[0] = fmaf(w4.x, a.x, acc[0]); acc[1] = fmaf(w4.y, a.y, acc[1]); acc[2] = fmaf(w4.z, a.z, acc[2]); acc[3] = fmaf(w4.w, a.w, acc[3]);
      } else {
        acc[0] = fmaf(wt[0], in[0], acc[0]);
      }
    }
    if (c < Cq) {
      if constexpr (V == 4) *reinterpret_cast<float4*>(q_out + t * Cq + c) = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
      else q_out[t * Cq + c] = acc[0] * scale;
    } else if (pos < Tcap) {                         // the host sizes the cache first; never write outside it
      const int g = (c - Cq) / dk, i = (c - Cq) % dk;
      T* dst = kcache + (((int64_t)row * G + g) * Tcap + pos) * dk + i;
#pragma unroll
      for (int k = 0; k < V; ++k) dst[k] = Tr<T>::from_f(acc[k]);
    }
  }
}

// ---- prompts on the tensor cores ------------------------------------------------------------------------------------------
// CTA = 64 consecutive tokens of one entry x one query head: 4 warps x 16 query rows.  K / V tiles of 64 keys stream
// global -> shared with cp.async (two stages, XOR-swizzled 16-byte chunks, shared by the four warps); S = Q K^T and O += P V
// run on mma.sync m16n8k16 with the fp32 online softmax in registers, in base-2 units: the distance bias is added to the
// scores as -slope log2(e) (p - j), and the running maximum / sum start from the sink (max = sink log2(e), sum = 1).
constexpr int ST_WARPS = 4, ST_THREADS = ST_WARPS * 32, ST_QT = 16 * ST_WARPS, ST_KT = 64, ST_STAGES = 2;
constexpr float LOG2E = 1.4426950408889634f;

// DECODE = false: 4 warps, rows = 64 consecutive tokens of entry blockIdx.z for head blockIdx.y (tile blockIdx.x of the entry).
// DECODE = true: ONE warp per CTA; its 16 rows are the query heads of key/value head blockIdx.y for the single token of entry
// blockIdx.z, and the CTA takes the blockIdx.x-th share of the key tiles (gridDim.x shares): it writes unnormalised partial
// sums (o, running max, sum; no sink) that sink_attn_merge_kernel combines.  The keys are then read once for all heads of a
// group, by many small CTAs at a time.
// RULED = true: the scores also pass the ScoreRule (cap, logarithmic penalty, window: tiles before the window of the CTA's first
// row are skipped, a row whose window has not begun keeps max = -inf and adds nothing) and the output its gate.
template <typename T, int DK, int DV, bool DECODE, bool RULED>
__global__ void __launch_bounds__(DECODE ? 32 : ST_THREADS, (RULED && !DECODE) ? 3 : 1)
sink_attn_tile_kernel(const float* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc, int64_t Tcap,
                      const int32_t* __restrict__ cu, const int32_t* __restrict__ rows, const int32_t* __restrict__ t_pos,
                      const float* __restrict__ sink, float slope_log2, T* __restrict__ out, int64_t ld_out, float out_scale,
                      int H, int G, float* __restrict__ part_o, float* __restrict__ part_ms, ScoreRule rule) {
  constexpr int NT = DECODE ? 32 : ST_THREADS;
  constexpr int KROW = DK * 2, VROW = DV * 2;                       // bytes per staged row
  constexpr int K_BYTES = ST_KT * KROW, V_BYTES = ST_KT * VROW, STAGE_BYTES = K_BYTES + V_BYTES;
  constexpr int KCH = DK / 8, VCH = DV / 8;                         // 16-byte chunks per row
  extern __shared__ __align__(128) uint8_t st_smem[];
  const int e = blockIdx.z;
  const int t_first = cu[e], n_e = cu[e + 1] - t_first;
  const int q0 = DECODE ? 0 : blockIdx.x * ST_QT;
  if (q0 >= n_e) return;                                            // the same for every thread of the CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad_row = lane >> 2, qc = lane & 3;
  const int per = H / G;
  const int g = DECODE ? blockIdx.y : blockIdx.y / per;
  const int p_first = t_pos[t_first];                               // positions of an entry's tokens are consecutive
  const int l0 = q0 + warp * 16 + quad_row, l1 = l0 + 8;            // this thread's two rows: tokens (prompts) or heads (decode)
  const int n_rows = DECODE ? per : n_e;
  const int lc0 = min(l0, n_rows - 1), lc1 = min(l1, n_rows - 1);   // rows past the end compute a valid row, not stored
  const int h0 = DECODE ? g * per + lc0 : blockIdx.y, h1 = DECODE ? g * per + lc1 : blockIdx.y;
  const int tk0 = DECODE ? t_first : t_first + lc0, tk1 = DECODE ? t_first : t_first + lc1;
  const int pos0 = DECODE ? p_first : p_first + lc0, pos1 = DECODE ? p_first : p_first + lc1;
  const int kend = DECODE ? p_first + 1 : p_first + min(n_e, q0 + ST_QT);     // keys any row of this CTA may see
  const int n_all = (kend + ST_KT - 1) / ST_KT;
  int tile_lo = 0, tile_hi = n_all;
  if (RULED && rule.window > 0) {                                   // the first key the CTA's first row sees
    const int first = (DECODE ? p_first : p_first + q0) - rule.window + 1;
    tile_lo = first > 0 ? first / ST_KT : 0;
  }
  if (DECODE) {
    const int share = (n_all - tile_lo + gridDim.x - 1) / gridDim.x;
    tile_lo += blockIdx.x * share;
    tile_hi = min(n_all, tile_lo + share);
  }
  float r1_0 = 0.f, r2_0 = 0.f, r1_1 = 0.f, r2_1 = 0.f;
  if (RULED && rule.r1) { r1_0 = rule.r1[h0]; r2_0 = rule.r2[h0]; r1_1 = rule.r1[h1]; r2_1 = rule.r2[h1]; }
  const float k_exp = (RULED && rule.cap > 0.f) ? 2.f * LOG2E / rule.cap : 0.f, cap2 = 2.f * rule.cap;
  // values that are the keys (one buffer, equal sizes): the staged key tile serves both products, no value tile is loaded and a
  // stage is half as large (the launcher sizes the shared memory accordingly)
  const bool same_kv = RULED && DK == DV && kc == vc;
  const int stage_bytes = same_kv ? K_BYTES : STAGE_BYTES;
  const float* ptab = nullptr;
  if (RULED && !DECODE && rule.r1 && rule.table > 0) {
    // every distance a visible pair of this CTA can have (below the window) once, instead of a logarithm per score
    float* tab = reinterpret_cast<float*>(st_smem + ST_STAGES * stage_bytes);
    for (int i = threadIdx.x; i < rule.table; i += NT) tab[i] = r1_0 * log1pf(r2_0 * (float)i);
    ptab = tab;                                                     // read after the first tile's __syncthreads
  }
  const float slope2_0 = head_slope(slope_log2, h0, H) * LOG2E, slope2_1 = head_slope(slope_log2, h1, H) * LOG2E;

  uint32_t qf[DK / 16][4];
  {
    const float* p0 = q + ((int64_t)tk0 * H + h0) * DK;
    const float* p1 = q + ((int64_t)tk1 * H + h1) * DK;
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) {
      const float2 a0 = *reinterpret_cast<const float2*>(p0 + ks * 16 + 2 * qc), a1 = *reinterpret_cast<const float2*>(p1 + ks * 16 + 2 * qc);
      const float2 b0 = *reinterpret_cast<const float2*>(p0 + ks * 16 + 8 + 2 * qc), b1 = *reinterpret_cast<const float2*>(p1 + ks * 16 + 8 + 2 * qc);
      qf[ks][0] = pack2<T>(a0.x, a0.y);
      qf[ks][1] = pack2<T>(a1.x, a1.y);
      qf[ks][2] = pack2<T>(b0.x, b0.y);
      qf[ks][3] = pack2<T>(b1.x, b1.y);
    }
  }
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(st_smem);
  const int64_t row = rows[e];
  const T* kbase = kc + (row * G + g) * Tcap * DK;
  const T* vbase = vc + (row * G + g) * Tcap * DV;
  auto issue_tile = [&](int tile, int stage) {
    const uint32_t ks = sbase + stage * stage_bytes, vs = ks + K_BYTES;
    const int key0 = tile * ST_KT;
#pragma unroll
    for (int i = 0; i < ST_KT * KCH / NT; ++i) {
      const int idx = i * NT + threadIdx.x;
      const int key = idx / KCH, ch = idx % KCH;
      const bool ok = key0 + key < kend;
      cp_async16(ks + (uint32_t)(key * KROW + ((ch ^ (key & 7)) << 4)), kbase + (int64_t)(key0 + (ok ? key : 0)) * DK + ch * 8, ok);
    }
    if (same_kv) return;
#pragma unroll
    for (int i = 0; i < ST_KT * VCH / NT; ++i) {
      const int idx = i * NT + threadIdx.x;
      const int key = idx / VCH, ch = idx % VCH;
      const bool ok = key0 + key < kend;
      cp_async16(vs + (uint32_t)(key * VROW + ((ch ^ (key & 7)) << 4)), vbase + (int64_t)(key0 + (ok ? key : 0)) * DV + ch * 8, ok);
    }
  };

  float o[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  // the sink opens the softmax: it is the running maximum, and its own term (one) sits in the sum of one thread of the quad
  // (the partial sums of a decode step leave the sink to the merge)
  const bool open_with_sink = !DECODE && sink;
  float m0 = open_with_sink ? sink[h0] * LOG2E : -INFINITY, m1 = m0;
  float s0 = (open_with_sink && qc == 0) ? 1.f : 0.f, s1 = s0;

  if (tile_lo < tile_hi) issue_tile(tile_lo, 0);
  cp_async_commit();
  for (int it = tile_lo; it < tile_hi; ++it) {
    const int stage = (it - tile_lo) & 1;
    if (it + 1 < tile_hi) issue_tile(it + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t ks = sbase + stage * stage_bytes, vs = same_kv ? ks : ks + K_BYTES;
    const int key0 = it * ST_KT;
    const int mat = lane >> 3, r = lane & 7;
    float sc[ST_KT / 8][4];
#pragma unroll
    for (int nt = 0; nt < ST_KT / 8; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
    for (int np = 0; np < ST_KT / 16; ++np) {
      const int key = 16 * np + r + 8 * (mat >> 1);
#pragma unroll
      for (int kstep = 0; kstep < DK / 16; ++kstep) {
        const int ch = 2 * kstep + (mat & 1);
        uint32_t bf[4];
        ldsm_x4(ks + (uint32_t)(key * KROW + ((ch ^ (key & 7)) << 4)), bf);
        mma16816<T>(sc[2 * np], qf[kstep], bf[0], bf[1]);
        mma16816<T>(sc[2 * np + 1], qf[kstep], bf[2], bf[3]);
      }
    }
    float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < ST_KT / 8; ++nt) {
      const int kcol = key0 + 8 * nt + 2 * qc;
      if constexpr (RULED) {
        const int d00 = pos0 - kcol, d01 = d00 - 1, d10 = pos1 - kcol, d11 = d10 - 1;
        const int wnd = rule.window > 0 ? rule.window : 0x7fffffff;
        sc[nt][0] = (d00 >= 0 && d00 < wnd) ? ruled_score_fast(sc[nt][0], rule, k_exp, cap2, r1_0, r2_0, d00, ptab) : -INFINITY;
        sc[nt][1] = (d01 >= 0 && d01 < wnd) ? ruled_score_fast(sc[nt][1], rule, k_exp, cap2, r1_0, r2_0, d01, ptab) : -INFINITY;
        sc[nt][2] = (d10 >= 0 && d10 < wnd) ? ruled_score_fast(sc[nt][2], rule, k_exp, cap2, r1_1, r2_1, d10, ptab) : -INFINITY;
        sc[nt][3] = (d11 >= 0 && d11 < wnd) ? ruled_score_fast(sc[nt][3], rule, k_exp, cap2, r1_1, r2_1, d11, ptab) : -INFINITY;
      }
      if (RULED && slope_log2 == 0.f) {                            // masked above; no linear bias: the scores just move to base 2
        sc[nt][0] *= LOG2E; sc[nt][1] *= LOG2E; sc[nt][2] *= LOG2E; sc[nt][3] *= LOG2E;
      } else {
        sc[nt][0] = kcol <= pos0 ? fmaf(sc[nt][0], LOG2E, -slope2_0 * (float)(pos0 - kcol)) : -INFINITY;
        sc[nt][1] = kcol + 1 <= pos0 ? fmaf(sc[nt][1], LOG2E, -slope2_0 * (float)(pos0 - kcol - 1)) : -INFINITY;
        sc[nt][2] = kcol <= pos1 ? fmaf(sc[nt][2], LOG2E, -slope2_1 * (float)(pos1 - kcol)) : -INFINITY;
        sc[nt][3] = kcol + 1 <= pos1 ? fmaf(sc[nt][3], LOG2E, -slope2_1 * (float)(pos1 - kcol - 1)) : -INFINITY;
      }
      t0 = fmaxf(t0, fmaxf(sc[nt][0], sc[nt][1]));
      t1 = fmaxf(t1, fmaxf(sc[nt][2], sc[nt][3]));
    }
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1)); t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    // finite from a CTA's first tile on: its first key is inside every row's bound (prompts: key 0; decode: one position)
    float mn0 = fmaxf(m0, t0), mn1 = fmaxf(m1, t1);
    const float keep0 = mn0, keep1 = mn1;
    if constexpr (RULED) {                           // nothing seen yet (the row's window begins later): exponentials against 0
      if (mn0 == -INFINITY) mn0 = 0.f;
      if (mn1 == -INFINITY) mn1 = 0.f;
    }
    const float corr0 = exp2f(m0 - mn0), corr1 = exp2f(m1 - mn1);
    m0 = keep0; m1 = keep1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < ST_KT / 8; ++nt) {
      sc[nt][0] = exp2f(sc[nt][0] - mn0); sc[nt][1] = exp2f(sc[nt][1] - mn0);
      sc[nt][2] = exp2f(sc[nt][2] - mn1); sc[nt][3] = exp2f(sc[nt][3] - mn1);
      ps0 += sc[nt][0] + sc[nt][1];
      ps1 += sc[nt][2] + sc[nt][3];
    }
    s0 = s0 * corr0 + ps0;
    s1 = s1 * corr1 + ps1;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) { o[j][0] *= corr0; o[j][1] *= corr0; o[j][2] *= corr1; o[j][3] *= corr1; }
#pragma unroll
    for (int kk = 0; kk < ST_KT / 16; ++kk) {
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
        ldsm_x4_trans(vs + (uint32_t)(key * VROW + ((ch ^ (key & 7)) << 4)), bf);
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
    const int64_t b0 = ((int64_t)e * H + h0) * gridDim.x + blockIdx.x, b1 = ((int64_t)e * H + h1) * gridDim.x + blockIdx.x;
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
  }
  const float inv0 = out_scale / s0, inv1 = out_scale / s1;
  T* o0 = out + (int64_t)tk0 * ld_out + (int64_t)h0 * DV;
  T* o1 = out + (int64_t)tk1 * ld_out + (int64_t)h1 * DV;
  const float* g0 = (RULED && rule.gate) ? rule.gate + (int64_t)tk0 * rule.ldg + (int64_t)h0 * DV : nullptr;
  const float* g1 = (RULED && rule.gate) ? rule.gate + (int64_t)tk1 * rule.ldg + (int64_t)h1 * DV : nullptr;
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) {
    const int c = 8 * j + 2 * qc;
    float a0 = o[j][0] * inv0, a1 = o[j][1] * inv0, b0 = o[j][2] * inv1, b1 = o[j][3] * inv1;
    if (RULED && g0) {
      if (l0 < n_e) { a0 *= sigmoid_fast(g0[c]); a1 *= sigmoid_fast(g0[c + 1]); }
      if (l1 < n_e) { b0 *= sigmoid_fast(g1[c]); b1 *= sigmoid_fast(g1[c + 1]); }
    }
    if (l0 < n_e) *reinterpret_cast<uint32_t*>(o0 + c) = pack2<T>(a0, a1);
    if (l1 < n_e) *reinterpret_cast<uint32_t*>(o1 + c) = pack2<T>(b0, b1);
  }
}

// out[e's token, h, :] = out_scale * (sum_s o_s 2^(m_s - m)) / (2^(sink log2e - m) + sum_s l_s 2^(m_s - m)), m the largest of them
template <typename T>
__global__ void sink_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ms,
                                       const int32_t* __restrict__ cu, const float* __restrict__ sink, T* __restrict__ out,
                                       int64_t ld_out, float out_scale, int H, int dv, int splits, const float* __restrict__ gate,
                                       int64_t ldg) {
  const int e = blockIdx.x, h = blockIdx.y;
  if (cu[e + 1] - cu[e] <= 0) return;
  const int64_t base = ((int64_t)e * H + h) * splits;
  float m = sink ? sink[h] * LOG2E : -INFINITY;
  for (int sidx = 0; sidx < splits; ++sidx) m = fmaxf(m, part_ms[(base + sidx) * 2]);
  float den = sink ? exp2f(sink[h] * LOG2E - m) : 0.f;
  for (int sidx = 0; sidx < splits; ++sidx) {
    const float ms = part_ms[(base + sidx) * 2];
    if (ms != -INFINITY) den += part_ms[(base + sidx) * 2 + 1] * exp2f(ms - m);
  }
  const float inv = out_scale / den;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float a = 0.f;
    for (int sidx = 0; sidx < splits; ++sidx) {
      const float ms = part_ms[(base + sidx) * 2];
      if (ms != -INFINITY) a = fmaf(part_o[(base + sidx) * dv + c], exp2f(ms - m), a);
    }
    const float gz = gate ? sigmoid_f(gate[(int64_t)cu[e] * ldg + (int64_t)h * dv + c]) : 1.f;
    out[(int64_t)cu[e] * ld_out + (int64_t)h * dv + c] = Tr<T>::from_f(a * inv * gz);
  }
}

constexpr int SINK_ATTN_MAX_SPLITS = 16;
constexpr int SINK_ATTN_MAX_TABLE = 16384;      // longest window whose penalties sit in shared memory (64 KB)

template <typename T, int DK, int DV, bool RULED>
static int sink_attn_tiles_launch(const float* q, const void* kc, const void* vc, int64_t Tcap, const int32_t* cu, const int32_t* rows,
                                  const int32_t* t_pos, const float* sink, float slope_log2, void* out, int64_t ld_out,
                                  float out_scale, int nb, int max_n, int H, int G, float* ws, size_t ws_bytes, cudaStream_t st,
                                  const ScoreRule& rule_in) {
  const int stage_smem = ST_STAGES * ST_KT * ((RULED && DK == DV && kc == vc) ? DK : DK + DV) * 2;
  // prompts with a window and a penalty: a table of the penalties of the distances 0 .. window - 1 behind the tile buffers
  ScoreRule rule = rule_in;
  rule.table = (RULED && max_n > 1 && rule.r1 && rule.window > 0 && rule.window <= SINK_ATTN_MAX_TABLE) ? rule.window : 0;
  const int smem = stage_smem + rule.table * (int)sizeof(float);
  if (max_n == 1) {
    // decode: shares of the key tiles per (entry, key/value head), as many as keep several CTAs per SM busy and the workspace holds
    auto kern = sink_attn_tile_kernel<T, DK, DV, true, RULED>;
    static int attr_smem = 48 * 1024;
    if (smem > attr_smem) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(sink_attn_tile_kernel)");
      attr_smem = smem;
    }
    const size_t per_split = (size_t)nb * H * (DV + 2) * sizeof(float);
    int splits = (int)((8 * 148 + (int64_t)nb * G - 1) / ((int64_t)nb * G));
    splits = splits < 1 ? 1 : splits > SINK_ATTN_MAX_SPLITS ? SINK_ATTN_MAX_SPLITS : splits;
    if ((size_t)splits * per_split > ws_bytes) splits = (int)(ws_bytes / per_split);
    if (splits < 1) return 1;                                     // no room for partial sums: the caller takes the per-token kernel
    float* part_o = ws;
    float* part_ms = ws + (size_t)nb * H * splits * DV;
    dim3 grid((unsigned)splits, (unsigned)G, (unsigned)nb);
    kern<<<grid, 32, smem, st>>>(q, (const T*)kc, (const T*)vc, Tcap, cu, rows, t_pos, sink, slope_log2, (T*)out, ld_out, out_scale,
                                 H, G, part_o, part_ms, rule);
    B200P_LAUNCH_CHECK("sink_attn_tile_kernel");
    sink_attn_merge_kernel<T><<<dim3((unsigned)nb, (unsigned)H), DV >= 128 ? 128 : 64, 0, st>>>(part_o, part_ms, cu, sink, (T*)out, ld_out,
                                                                                                   out_scale, H, DV, splits, rule.gate, rule.ldg);
    B200P_LAUNCH_CHECK("sink_attn_merge_kernel");
    return B200P_OK;
  }
  auto kern = sink_attn_tile_kernel<T, DK, DV, false, RULED>;
  static int attr_smem = 48 * 1024;                             // the table's size varies with the window: keep the largest asked for
  if (smem > attr_smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(sink_attn_tile_kernel)");
    attr_smem = smem;
  }
  dim3 grid((unsigned)((max_n + ST_QT - 1) / ST_QT), (unsigned)H, (unsigned)nb);
  kern<<<grid, ST_THREADS, smem, st>>>(q, (const T*)kc, (const T*)vc, Tcap, cu, rows, t_pos, sink, slope_log2, (T*)out, ld_out,
                                       out_scale, H, G, nullptr, nullptr, rule);
  B200P_LAUNCH_CHECK("sink_attn_tile_kernel");
  return B200P_OK;
}

// 1 when the tile kernel takes these sizes (16-bit caches, key and value sizes of 64 or 128)
static bool sink_attn_tiles_ok(int dk, int dv, int dtype) {
  return (dtype == B200P_F16 || dtype == B200P_BF16) && (dk == 64 || dk == 128) && (dv == 64 || dv == 128);
}

template <typename T>
static int sink_attn_tiles(const float* q, const void* kc, const void* vc, int64_t Tcap, const int32_t* cu, const int32_t* rows,
                           const int32_t* t_pos, const float* sink, float slope_log2, void* out, int64_t ld_out, float out_scale,
                           int nb, int max_n, int H, int G, int dk, int dv, float* ws, size_t ws_bytes, cudaStream_t st,
                           const ScoreRule* rule) {
  static const ScoreRule none = {0.f, nullptr, nullptr, 0, nullptr, 0, 0};
#define ST_CASE(DK_, DV_) \
  if (dk == DK_ && dv == DV_ && !rule) \
    return sink_attn_tiles_launch<T, DK_, DV_, false>(q, kc, vc, Tcap, cu, rows, t_pos, sink, slope_log2, out, ld_out, out_scale, nb, max_n, H, G, ws, ws_bytes, st, none)
#define ST_RULED(DK_, DV_) \
  if (dk == DK_ && dv == DV_ && rule) \
    return sink_attn_tiles_launch<T, DK_, DV_, true>(q, kc, vc, Tcap, cu, rows, t_pos, sink, slope_log2, out, ld_out, out_scale, nb, max_n, H, G, ws, ws_bytes, st, *rule)
  ST_CASE(64, 64);
  ST_CASE(64, 128);
  ST_CASE(128, 64);
  ST_CASE(128, 128);
  ST_RULED(64, 64);
  ST_RULED(128, 128);
  if (rule) return 1;                                            // other sizes with a rule: the caller takes the per-token kernel
#undef ST_CASE
#undef ST_RULED
  set_error("tile attention: unsupported sizes");
  return B200P_ERR_ARG;
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_sink_attn_prep(const float* proj, int64_t ldp, int64_t col_q, int64_t col_k, int64_t col_v, const float* wq,
                                    const float* wk, float eps, float scale, float temp_coef, float temp_every, float* q_out,
                                    void* kcache, void* vcache, int64_t Tcap, const int32_t* t_row, const int32_t* t_pos, int64_t M,
                                    int H, int G, int dk, int dv, int dtype, void* stream) {
  B200P_REQUIRE(proj && q_out && kcache && vcache && t_row && t_pos, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0, B200P_ERR_ARG, "bad head geometry");
  B200P_REQUIRE(temp_coef == 0.f || temp_every > 0.f, B200P_ERR_ARG, "the query temperature needs a positive block length");
  if (M == 0) return B200P_OK;
  const unsigned threads = (H + G) >= 8 ? 256 : 128;
  B200P_DISPATCH_DTYPE(dtype, T, (sink_attn_prep_kernel<T><<<(unsigned)M, threads, 0, (cudaStream_t)stream>>>(
      proj, ldp, col_q, col_k, col_v, wq, wk, eps, scale, temp_coef, temp_every, q_out, (T*)kcache, (T*)vcache, Tcap, t_row, t_pos,
      H, G, dk, dv)));
  B200P_LAUNCH_CHECK("sink_attn_prep_kernel");
  return B200P_OK;
}

template <typename T>
static int sink_attn_generic(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                             const int32_t* t_pos, const float* sink, float slope_log2, void* out, int64_t ld_out, float out_scale,
                             int64_t M, int H, int G, int dk, int dv, cudaStream_t st, const ScoreRule* rule = nullptr) {
  static const ScoreRule none = {0.f, nullptr, nullptr, 0, nullptr, 0, 0};
  const int per = H / G, nw = per < SA_MAX_HEADS ? per : SA_MAX_HEADS;
  const size_t smem = ((size_t)SA_KEYS * (dk + 1) + (size_t)SA_KEYS * dv + (size_t)nw * dk) * sizeof(float);
  auto kern = sink_attn_kernel<T>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(sink_attn_kernel)");
  }
  dim3 grid((unsigned)M, (unsigned)G, (unsigned)((per + nw - 1) / nw));
  kern<<<grid, nw * 32, smem, st>>>(q, (const T*)kcache, (const T*)vcache, Tcap, t_row, t_pos, sink, slope_log2, (T*)out, ld_out,
                                    out_scale, H, G, dk, dv, rule ? *rule : none);
  B200P_LAUNCH_CHECK("sink_attn_kernel");
  return B200P_OK;
}

extern "C" int b200p_sink_attn_tiles_supported(int dk, int dv, int dtype) { return sink_attn_tiles_ok(dk, dv, dtype) ? 1 : 0; }

extern "C" size_t b200p_sink_attn_workspace_bytes(int64_t nb, int H, int dv) {
  return (size_t)nb * H * SINK_ATTN_MAX_SPLITS * (dv + 2) * sizeof(float);
}

// the shared body of b200p_sink_attn and b200p_window_attn
static int attn_dispatch(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                         const int32_t* t_pos, const int32_t* cu, const int32_t* rows, int nb, int max_n, const float* sink,
                         float slope_log2, void* out, int64_t ld_out, float out_scale, int64_t M, int H, int G, int dk, int dv,
                         int dtype, void* workspace, size_t workspace_bytes, void* stream, const ScoreRule* rule) {
  B200P_REQUIRE(q && kcache && vcache && t_row && t_pos && out, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && G > 0 && H % G == 0 && G < 65536 && dk > 0 && dv > 0, B200P_ERR_ARG, "bad head geometry");
  B200P_REQUIRE(dv <= 32 * SA_MAX_VL && dk <= 1024, B200P_ERR_ARG, "value size above %d or key size above 1024 is not built",
                32 * SA_MAX_VL);
  B200P_REQUIRE(ld_out >= (int64_t)H * dv, B200P_ERR_ARG, "output rows are shorter than the heads");
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // prompts (entries of several tokens, described by cu / rows) of 16-bit models run on the tensor-core tile kernel
  // and so do decode steps (one token per entry) whose heads per key/value head fit a 16-row tile, given room for partial sums
  const bool prompts = max_n >= SINK_ATTN_TILES_MIN_TOKENS;
  const bool decode = max_n == 1 && H / G <= 16 && workspace && aligned(workspace, 16);
  if (cu && rows && nb > 0 && (prompts || decode) && sink_attn_tiles_ok(dk, dv, dtype) && ld_out % 2 == 0 &&
      aligned(kcache, 16) && aligned(vcache, 16) && aligned(out, 4) && aligned(q, 8) && nb < 65536 && H < 65536) {
    const int rc = dtype == B200P_F16
        ? sink_attn_tiles<__half>(q, kcache, vcache, Tcap, cu, rows, t_pos, sink, slope_log2, out, ld_out, out_scale, nb, max_n, H, G, dk, dv,
                                  (float*)workspace, workspace_bytes, st, rule)
        : sink_attn_tiles<__nv_bfloat16>(q, kcache, vcache, Tcap, cu, rows, t_pos, sink, slope_log2, out, ld_out, out_scale, nb, max_n, H, G,
                                         dk, dv, (float*)workspace, workspace_bytes, st, rule);
    if (rc != 1) return rc;
  }
  switch (dtype) {
    case B200P_F32: return sink_attn_generic<float>(q, kcache, vcache, Tcap, t_row, t_pos, sink, slope_log2, out, ld_out, out_scale, M, H, G, dk, dv, st, rule);
    case B200P_F16: return sink_attn_generic<__half>(q, kcache, vcache, Tcap, t_row, t_pos, sink, slope_log2, out, ld_out, out_scale, M, H, G, dk, dv, st, rule);
    case B200P_BF16: return sink_attn_generic<__nv_bfloat16>(q, kcache, vcache, Tcap, t_row, t_pos, sink, slope_log2, out, ld_out, out_scale, M, H, G, dk, dv, st, rule);
    default: set_error("bad dtype %d", dtype); return B200P_ERR_ARG;
  }
}

extern "C" int b200p_sink_attn(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                               const int32_t* t_pos, const int32_t* cu, const int32_t* rows, int nb, int max_n, const float* sink,
                               float slope_log2, void* out, int64_t ld_out, float out_scale, int64_t M, int H, int G, int dk,
                               int dv, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  return attn_dispatch(q, kcache, vcache, Tcap, t_row, t_pos, cu, rows, nb, max_n, sink, slope_log2, out, ld_out, out_scale, M, H, G, dk,
                       dv, dtype, workspace, workspace_bytes, stream, nullptr);
}

extern "C" int b200p_window_attn_prep(const float* proj, int64_t ldp, int64_t col_q, const float* conv_w, const float* conv_state,
                                      int taps, float scale, float* q_out, void* kcache, int64_t Tcap, const int32_t* t_row,
                                      const int32_t* t_pos, const int32_t* t_off, int64_t M, int H, int G, int dk, int dtype,
                                      void* stream) {
  B200P_REQUIRE(proj && conv_w && q_out && kcache && t_row && t_pos && t_off, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && G > 0 && H % G == 0 && dk > 0 && taps >= 1 && (taps == 1 || conv_state), B200P_ERR_ARG,
                "bad head geometry, or a convolution without its carried inputs");
  if (M == 0) return B200P_OK;
  const int C = (H + G) * dk;
  const bool vec = dk % 4 == 0 && ldp % 4 == 0 && col_q % 4 == 0 && aligned(proj, 16) && aligned(conv_w, 16) && aligned(q_out, 16) &&
                   (taps == 1 || aligned(conv_state, 16));
  const int per = vec ? C / 4 : C;
  const dim3 grid((unsigned)M, M >= 512 ? 1u : (unsigned)((per + 255) / 256 > 8 ? 8 : (per + 255) / 256));
  if (vec) {
    B200P_DISPATCH_DTYPE(dtype, T, (window_attn_prep_kernel<T, 4><<<grid, 256, 0, (cudaStream_t)stream>>>(
        proj, ldp, col_q, conv_w, conv_state, taps, scale, q_out, (T*)kcache, Tcap, t_row, t_pos, t_off, H, G, dk)));
  } else {
    B200P_DISPATCH_DTYPE(dtype, T, (window_attn_prep_kernel<T, 1><<<grid, 256, 0, (cudaStream_t)stream>>>(
        proj, ldp, col_q, conv_w, conv_state, taps, scale, q_out, (T*)kcache, Tcap, t_row, t_pos, t_off, H, G, dk)));
  }
  B200P_LAUNCH_CHECK("window_attn_prep_kernel");
  return B200P_OK;
}

extern "C" int b200p_window_attn(const float* q, const void* kcache, const void* vcache, int64_t Tcap, const int32_t* t_row,
                                 const int32_t* t_pos, const int32_t* cu, const int32_t* rows, int nb, int max_n, float softcap,
                                 const float* r1, const float* r2, int64_t window, const float* gate, int64_t ldg, void* out,
                                 int64_t ld_out, int64_t M, int H, int G, int dk, int dv, int dtype, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  B200P_REQUIRE((r1 == nullptr) == (r2 == nullptr), B200P_ERR_ARG, "the distance penalty needs both of its vectors");
  B200P_REQUIRE(window >= 0 && window < 0x7fffffff && softcap >= 0.f, B200P_ERR_ARG, "bad window or cap");
  B200P_REQUIRE(gate == nullptr || ldg >= (int64_t)H * dv, B200P_ERR_ARG, "gate rows are shorter than the heads");
  const ScoreRule rule = {softcap, r1, r2, (int)window, gate, ldg, 0};
  return attn_dispatch(q, kcache, vcache, Tcap, t_row, t_pos, cu, rows, nb, max_n, nullptr, 0.f, out, ld_out, 1.f, M, H, G, dk, dv, dtype,
                       workspace, workspace_bytes, stream, &rule);
}

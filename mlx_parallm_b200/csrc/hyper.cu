// Row-wise kernels of designs that keep several copies of the residual stream ("hyper-connections"), norm with a tanh instead of
// statistics, and add a short causal convolution over time to what every sublayer reads.
//   hyper_step_kernel   closes a sublayer and opens the next one in one pass over a token's copies:
//                         x'_r = sum_s mix[s, r] x_s + out[r] y          (every copy from the old ones; mix NULL: x' = x)
//                         u = sum_r in[r] x'_r;  n = tanh(alpha u) w + b (w NULL: n = u)
//                       and, when every entry brings ONE token (a decode step), also the convolution over n and the carried
//                       inputs, the storage-type result and the shift of the carried inputs -- the thread that reads a channel's
//                       history is the one that replaces it, so nothing else has to wait
//   canon_conv_kernel   prompts: x = n + sum_j w[j, :] n_(t - taps + 1 + j) over the portion's rows or, before its start, the
//                       carried inputs (zeros before the sequence's start); the carried inputs are committed afterwards by
//                       b200p_delta_conv_commit on n.  The taps are stored tap by tap, [taps, W], so that a thread's channels
//                       are neighbours in memory
//   tanh_norm_kernel    tanh(alpha h) w + b of given rows, into the storage type (the model's last norm)
// Everything is fp32 except the value handed to the next matrix product.
#include "common.cuh"

namespace b200p {

constexpr int HYPER_MAX_STREAMS = 8;
constexpr int CANON_MAX_TAPS = 16;

// V consecutive channels of a row, as one 16-byte access where V == 4
template <int V> struct Vec { float v[V]; };
template <int V> __device__ __forceinline__ Vec<V> ldv(const float* p) {
  Vec<V> r;
  if constexpr (V == 4) { const float4 q = *reinterpret_cast<const float4*>(p); r.v[0] = q.x; r.v[1] = q.y; r.v[2] = q.z; r.v[3] = q.w; }
  else r.v[0] = *p;
  return r;
}
template <int V> __device__ __forceinline__ void stv(float* p, const Vec<V>& r) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  else *p = r.v[0];
}
template <typename T, int V> __device__ __forceinline__ void stv_t(T* p, const Vec<V>& r) {
  if constexpr (V == 4 && sizeof(T) == 2) {
    T h[4] = {Tr<T>::from_f(r.v[0]), Tr<T>::from_f(r.v[1]), Tr<T>::from_f(r.v[2]), Tr<T>::from_f(r.v[3])};
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(h);
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) p[i] = Tr<T>::from_f(r.v[i]);
  }
}

// S copies (a template parameter: the S x S mixing sits in registers), V channels per thread.  One CTA row per token.
template <typename T, int S, int V>
__global__ void __launch_bounds__(256)
hyper_step_kernel(float* __restrict__ xs, const float* __restrict__ y, const float* __restrict__ src,
                  const float* __restrict__ mix, const float* __restrict__ outv, const float* __restrict__ inv,
                  const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
                  float* __restrict__ n_out, float* __restrict__ sum_out, int64_t W,
                  // fused convolution of a decode step (x_out != NULL)
                  const float* __restrict__ conv_w, float* __restrict__ conv_state, const int32_t* __restrict__ t_row,
                  const int32_t* __restrict__ t_pos, int taps, T* __restrict__ x_out) {
  float m[S * S], ov[S], iv[S];
#pragma unroll
  for (int i = 0; i < S * S; ++i) m[i] = mix ? mix[i] : ((i / S) == (i % S) ? 1.f : 0.f);
#pragma unroll
  for (int i = 0; i < S; ++i) {
    ov[i] = outv ? outv[i] : 0.f;
    iv[i] = inv ? inv[i] : 0.f;
  }
  const int64_t t = blockIdx.x;
  const float al = alpha ? alpha[0] : 1.f;
  float* xt = xs + t * S * W;
  int row = 0, pos = 0;
  if (x_out) { row = t_row[t]; pos = t_pos[t]; }
  for (int64_t c = ((int64_t)blockIdx.y * blockDim.x + threadIdx.x) * V; c < W; c += (int64_t)gridDim.y * blockDim.x * V) {
    Vec<V> old[S];
    if (src) {
      const Vec<V> e = ldv<V>(src + t * W + c);
#pragma unroll
      for (int s = 0; s < S; ++s) old[s] = e;
    } else {
#pragma unroll
      for (int s = 0; s < S; ++s) old[s] = ldv<V>(xt + s * W + c);
    }
    Vec<V> yv, u, total;
    if (y) yv = ldv<V>(y + t * W + c);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      if (!y) yv.v[i] = 0.f;
      u.v[i] = 0.f;
      total.v[i] = 0.f;
    }
#pragma unroll
    for (int r = 0; r < S; ++r) {
      Vec<V> nv;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) v = fmaf(m[s * S + r], old[s].v[i], v);
        v = fmaf(ov[r], yv.v[i], v);
        nv.v[i] = v;
        u.v[i] = fmaf(iv[r], v, u.v[i]);
        total.v[i] += v;
      }
      stv<V>(xt + r * W + c, nv);
    }
    if (sum_out) stv<V>(sum_out + t * W + c, total);
    if (!n_out && !x_out) continue;
    Vec<V> n = u;
    if (w) {
      const Vec<V> wv = ldv<V>(w + c);
#pragma unroll
      for (int i = 0; i < V; ++i) n.v[i] = fmaf(tanhf(al * u.v[i]), wv.v[i], b ? b[c + i] : 0.f);
    }
    if (n_out) stv<V>(n_out + t * W + c, n);
    if (x_out) {
      // one token per entry: the history is the carried inputs only; read them, add, then shift them by one
      float* st = conv_state + (int64_t)row * (taps - 1) * W + c;
      Vec<V> acc = n, cur;                                          // taps in the order of the prompt kernel
      for (int i = 0; i < taps - 1; ++i) {
        cur = ldv<V>(st + (int64_t)i * W);
        const bool seen = taps - 1 - i <= pos;                       // carried input i lies taps - 1 - i tokens back
#pragma unroll
        const Vec<V> wt = ldv<V>(conv_w + (int64_t)i * W + c);
#pragma unroll
        for (int k = 0; k < V; ++k) acc.v[k] = fmaf(wt.v[k], seen ? cur.v[k] : 0.f, acc.v[k]);
        if (i > 0) stv<V>(st + (int64_t)(i - 1) * W, cur);
      }
const Vec<V> wl = ldv<V>(conv_w + (int64_t)(taps - 1) * W + c);
#pragma unroll
      for (int k = 0; k < V; ++k) acc.v[k] = fmaf(wl.v[k], n.v[k], acc.v[k]);
      stv_t<T, V>(x_out + t * W + c, acc);
      if (taps > 1) stv<V>(st + (int64_t)(taps - 2) * W, n);
    }
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256)
canon_conv_kernel(const float* __restrict__ n, const float* __restrict__ conv_w, const float* __restrict__ conv_state,
                  const int32_t* __restrict__ t_row, const int32_t* __restrict__ t_pos, const int32_t* __restrict__ t_off,
                  T* __restrict__ x_out, int64_t W, int taps) {
  const int64_t t = blockIdx.x;
  const int row = t_row[t], pos = t_pos[t], off = t_off[t];
  const float* nt = n + t * W;
  for (int64_t c = ((int64_t)blockIdx.y * blockDim.x + threadIdx.x) * V; c < W; c += (int64_t)gridDim.y * blockDim.x * V) {
    Vec<V> acc = ldv<V>(nt + c);
    for (int j = 0; j < taps; ++j) {
      const int d = taps - 1 - j;                                   // tap j multiplies the input d tokens back
      if (d > pos) continue;                                        // before the sequence
      const Vec<V> in = d <= off ? ldv<V>(nt + c - (int64_t)d * W)
                                 : ldv<V>(conv_state + ((int64_t)row * (taps - 1) + (taps - 1 + off - d)) * W + c);
const Vec<V> wt = ldv<V>(conv_w + (int64_t)j * W + c);
#pragma unroll
      for (int k = 0; k < V; ++k) acc.v[k] = fmaf(wt.v[k], in.v[k], acc.v[k]);
    }
    stv_t<T, V>(x_out + t * W + c, acc);
  }
}

template <typename T>
__global__ void tanh_norm_kernel(const float* __restrict__ h, const float* __restrict__ alpha, const float* __restrict__ w,
                                 const float* __restrict__ b, T* __restrict__ x_out, int64_t W) {
  const int64_t t = blockIdx.x;
  const float al = alpha[0];
  for (int64_t c = threadIdx.x; c < W; c += blockDim.x)
    x_out[t * W + c] = Tr<T>::from_f(fmaf(tanhf(al * h[t * W + c]), w[c], b ? b[c] : 0.f));
}

}  // namespace b200p

using namespace b200p;

static inline dim3 row_grid(int64_t M, int64_t W, unsigned threads) {
  // one CTA row per token; wide models with few tokens spread a row over several CTAs
  unsigned per = (unsigned)((W + threads - 1) / threads);
  unsigned y = M >= 512 ? 1u : per > 8u ? 8u : per;
  return dim3((unsigned)M, y < 1u ? 1u : y);
}

template <typename T, int V>
static int hyper_step_launch(float* xs, const float* y, const float* src, const float* mix, const float* out, const float* in,
                             const float* alpha, const float* w, const float* b, float* n_out, float* sum_out, int64_t M, int streams,
                             int64_t W, const float* conv_w, float* conv_state, const int32_t* t_row, const int32_t* t_pos, int taps,
                             void* x_out, cudaStream_t st) {
  const unsigned threads = W / V >= 512 ? 256 : 128;
  const dim3 grid = row_grid(M, W / V, threads);
#define HS_CASE(S_)                                                                                                             \
  case S_:                                                                                                                      \
    hyper_step_kernel<T, S_, V><<<grid, threads, 0, st>>>(xs, y, src, mix, out, in, alpha, w, b, n_out, sum_out, W, conv_w,      \
                                                          conv_state, t_row, t_pos, taps, (T*)x_out);                           \
    break;
  switch (streams) {
    HS_CASE(1) HS_CASE(2) HS_CASE(3) HS_CASE(4) HS_CASE(5) HS_CASE(6) HS_CASE(7) HS_CASE(8)
  }
#undef HS_CASE
  B200P_LAUNCH_CHECK("hyper_step_kernel");
  return B200P_OK;
}

extern "C" int b200p_hyper_step(float* xs, const float* y, const float* src, const float* mix, const float* out, const float* in,
                                const float* alpha, const float* w, const float* b, float* n_out, float* sum_out, int64_t M,
                                int streams, int64_t W, const float* conv_w, float* conv_state, const int32_t* t_row,
                                const int32_t* t_pos, int taps, void* x_out, int dtype, void* stream) {
  B200P_REQUIRE(xs && W > 0, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(streams >= 1 && streams <= HYPER_MAX_STREAMS, B200P_ERR_ARG, "copies of the stream in [1, %d]", HYPER_MAX_STREAMS);
  B200P_REQUIRE((n_out == nullptr && x_out == nullptr) || in, B200P_ERR_ARG, "a norm output needs the reading weights");
  B200P_REQUIRE(w == nullptr || alpha, B200P_ERR_ARG, "the tanh norm needs its alpha");
  B200P_REQUIRE(x_out == nullptr || (conv_w && conv_state && t_row && t_pos && taps >= 1 && taps <= CANON_MAX_TAPS), B200P_ERR_ARG,
                "the fused convolution needs its taps (1..%d), carried inputs and the token plan", CANON_MAX_TAPS);
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // 16-byte accesses where every row of every buffer starts on a 16-byte boundary
  const bool vec = W % 4 == 0 && aligned(xs, 16) && aligned(y, 16) && aligned(src, 16) && aligned(w, 16) && aligned(n_out, 16) &&
                   aligned(sum_out, 16) && aligned(conv_state, 16) && aligned(conv_w, 16) && aligned(x_out, 8);
#define HS_DTYPE(T)                                                                                                              \
  return vec ? hyper_step_launch<T, 4>(xs, y, src, mix, out, in, alpha, w, b, n_out, sum_out, M, streams, W, conv_w, conv_state, \
                                       t_row, t_pos, taps, x_out, st)                                                            \
             : hyper_step_launch<T, 1>(xs, y, src, mix, out, in, alpha, w, b, n_out, sum_out, M, streams, W, conv_w, conv_state, \
                                       t_row, t_pos, taps, x_out, st)
  switch (x_out ? dtype : B200P_F32) {
    case B200P_F32: HS_DTYPE(float);
    case B200P_F16: HS_DTYPE(__half);
    case B200P_BF16: HS_DTYPE(__nv_bfloat16);
    default: set_error("bad dtype %d", dtype); return B200P_ERR_ARG;
  }
#undef HS_DTYPE
}

extern "C" int b200p_canon_conv(const float* n, const float* conv_w, const float* conv_state, const int32_t* t_row,
                                const int32_t* t_pos, const int32_t* t_off, void* x_out, int64_t M, int64_t W, int taps, int dtype,
                                void* stream) {
  B200P_REQUIRE(n && conv_w && conv_state && t_row && t_pos && t_off && x_out && W > 0, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(taps >= 1 && taps <= CANON_MAX_TAPS, B200P_ERR_ARG, "taps in [1, %d]", CANON_MAX_TAPS);
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = W % 4 == 0 && aligned(n, 16) && aligned(conv_state, 16) && aligned(conv_w, 16) && aligned(x_out, 8);
  const int64_t per = vec ? W / 4 : W;
  const unsigned threads = per >= 512 ? 256 : 128;
  const dim3 grid = row_grid(M, per, threads);
  if (vec) {
    B200P_DISPATCH_DTYPE(dtype, T, (canon_conv_kernel<T, 4><<<grid, threads, 0, st>>>(n, conv_w, conv_state, t_row, t_pos, t_off, (T*)x_out, W, taps)));
  } else {
    B200P_DISPATCH_DTYPE(dtype, T, (canon_conv_kernel<T, 1><<<grid, threads, 0, st>>>(n, conv_w, conv_state, t_row, t_pos, t_off, (T*)x_out, W, taps)));
  }
  B200P_LAUNCH_CHECK("canon_conv_kernel");
  return B200P_OK;
}

extern "C" int b200p_tanh_norm(const float* h, const float* alpha, const float* w, const float* b, void* x_out, int64_t M, int64_t W,
                               int dtype, void* stream) {
  B200P_REQUIRE(h && alpha && w && x_out && W > 0, B200P_ERR_ARG, "null pointer");
  if (M == 0) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (tanh_norm_kernel<T><<<(unsigned)M, W >= 1024 ? 256 : 128, 0, (cudaStream_t)stream>>>(
      h, alpha, w, b, (T*)x_out, W)));
  B200P_LAUNCH_CHECK("tanh_norm_kernel");
  return B200P_OK;
}

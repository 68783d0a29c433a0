// Row-wise kernels of designs that keep several copies of the residual stream ("hyper-connections"), norm with a tanh instead of
// statistics, and add a short causal convolution over time to what every sublayer reads.
//   hyper_step_kernel   closes a sublayer and opens the next one in one pass over a token's copies:
//                         x'_r = sum_s mix[s, r] x_s + out[r] y          (every copy from the old ones; mix NULL: x' = x)
//                         u = sum_r in[r] x'_r;  n = tanh(alpha u) w + b (w NULL: n = u)
//                       and, when every entry brings ONE token (a decode step), also the convolution over n and the carried
//                       inputs, the storage-type result and the shift of the carried inputs -- the thread that reads a channel's
//                       history is the one that replaces it, so nothing else has to wait
//   canon_conv_kernel   prompts: x = n + sum_j w[:, j] n_(t - taps + 1 + j) over the portion's rows or, before its start, the
//                       carried inputs (zeros before the sequence's start); the carried inputs are committed afterwards by
//                       b200p_delta_conv_commit on n
//   tanh_norm_kernel    tanh(alpha h) w + b of given rows, into the storage type (the model's last norm)
// Everything is fp32 except the value handed to the next matrix product.
#include "common.cuh"

namespace b200p {

constexpr int HYPER_MAX_STREAMS = 8;
constexpr int CANON_MAX_TAPS = 16;

struct HyperArgs {
  float mix[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS];     // [from, to]
  float out[HYPER_MAX_STREAMS];
  float in[HYPER_MAX_STREAMS];
};

// value of the convolution's input d tokens before token (row, pos, off) for channel c; cur = the portion's rows of n
__device__ __forceinline__ float canon_input(const float* __restrict__ n_t, int64_t ld, const float* __restrict__ state, int row,
                                             int pos, int off, int d, int taps, int64_t W, int64_t c) {
  if (d > pos) return 0.f;                                          // before the sequence
  if (d <= off) return n_t[c - (int64_t)d * ld];                    // inside this step's portion
  return state[((int64_t)row * (taps - 1) + (taps - 1 + off - d)) * W + c];
}

template <typename T>
__global__ void hyper_step_kernel(float* __restrict__ xs, const float* __restrict__ y, const float* __restrict__ src,
                                  const float* __restrict__ mix, const float* __restrict__ outv, const float* __restrict__ inv,
                                  const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
                                  float* __restrict__ n_out, float* __restrict__ sum_out, int S, int64_t W,
                                  // fused convolution of a decode step (x_out != NULL)
                                  const float* __restrict__ conv_w, float* __restrict__ conv_state, const int32_t* __restrict__ t_row,
                                  const int32_t* __restrict__ t_pos, int taps, T* __restrict__ x_out) {
  __shared__ HyperArgs a;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) a.mix[i] = mix ? mix[i] : ((i / S) == (i % S) ? 1.f : 0.f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    a.out[i] = outv ? outv[i] : 0.f;
    a.in[i] = inv ? inv[i] : 0.f;
  }
  __syncthreads();
  const int64_t t = blockIdx.x;
  const float al = alpha ? alpha[0] : 1.f;
  float* xt = xs + t * S * W;
  int row = 0, pos = 0;
  if (x_out) { row = t_row[t]; pos = t_pos[t]; }
  for (int64_t c = (int64_t)blockIdx.y * blockDim.x + threadIdx.x; c < W; c += (int64_t)gridDim.y * blockDim.x) {
    float old[HYPER_MAX_STREAMS], nw[HYPER_MAX_STREAMS];
    if (src) {
      const float e = src[t * W + c];
#pragma unroll
      for (int s = 0; s < HYPER_MAX_STREAMS; ++s) old[s] = e;
    } else {
#pragma unroll
      for (int s = 0; s < HYPER_MAX_STREAMS; ++s) old[s] = s < S ? xt[s * W + c] : 0.f;
    }
    const float yv = y ? y[t * W + c] : 0.f;
    float u = 0.f, total = 0.f;
#pragma unroll
    for (int r = 0; r < HYPER_MAX_STREAMS; ++r) {
      if (r < S) {
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
          if (s < S) v = fmaf(a.mix[s * S + r], old[s], v);
        v = fmaf(a.out[r], yv, v);
        nw[r] = v;
        xt[r * W + c] = v;
        u = fmaf(a.in[r], v, u);
        total += v;
      }
    }
    if (sum_out) sum_out[t * W + c] = total;
    if (!n_out && !x_out) continue;
    const float n = w ? fmaf(tanhf(al * u), w[c], b ? b[c] : 0.f) : u;
    if (n_out) n_out[t * W + c] = n;
    if (x_out) {
      // one token per entry: the history is the carried inputs only; read them, add, then shift them by one
      float* st = conv_state + (int64_t)row * (taps - 1) * W + c;
      float acc = n;                                                // taps in the order of the prompt kernel
      float hist[CANON_MAX_TAPS];
#pragma unroll
      for (int i = 0; i < CANON_MAX_TAPS; ++i) hist[i] = i < taps - 1 ? st[(int64_t)i * W] : 0.f;
#pragma unroll
      for (int i = 0; i < CANON_MAX_TAPS; ++i) {
        if (i < taps - 1) {
          const int d = taps - 1 - i;                               // carried input i lies d tokens back
          acc = fmaf(conv_w[c * taps + i], d <= pos ? hist[i] : 0.f, acc);
        }
      }
      acc = fmaf(conv_w[c * taps + taps - 1], n, acc);
      x_out[t * W + c] = Tr<T>::from_f(acc);
#pragma unroll
      for (int i = 0; i < CANON_MAX_TAPS; ++i)
        if (i < taps - 1) st[(int64_t)i * W] = i + 1 < taps - 1 ? hist[i + 1] : n;
    }
  }
}

template <typename T>
__global__ void canon_conv_kernel(const float* __restrict__ n, const float* __restrict__ conv_w, const float* __restrict__ conv_state,
                                  const int32_t* __restrict__ t_row, const int32_t* __restrict__ t_pos,
                                  const int32_t* __restrict__ t_off, T* __restrict__ x_out, int64_t W, int taps) {
  const int64_t t = blockIdx.x;
  const int row = t_row[t], pos = t_pos[t], off = t_off[t];
  const float* nt = n + t * W;
  for (int64_t c = (int64_t)blockIdx.y * blockDim.x + threadIdx.x; c < W; c += (int64_t)gridDim.y * blockDim.x) {
    float acc = nt[c];
    for (int j = 0; j < taps; ++j)
      acc = fmaf(conv_w[c * taps + j], canon_input(nt, W, conv_state, row, pos, off, taps - 1 - j, taps, W, c), acc);
    x_out[t * W + c] = Tr<T>::from_f(acc);
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
  const unsigned threads = W >= 1024 ? 256 : 128;
  B200P_DISPATCH_DTYPE(dtype, T, (hyper_step_kernel<T><<<row_grid(M, W, threads), threads, 0, (cudaStream_t)stream>>>(
      xs, y, src, mix, out, in, alpha, w, b, n_out, sum_out, streams, W, conv_w, conv_state, t_row, t_pos, taps, (T*)x_out)));
  B200P_LAUNCH_CHECK("hyper_step_kernel");
  return B200P_OK;
}

extern "C" int b200p_canon_conv(const float* n, const float* conv_w, const float* conv_state, const int32_t* t_row,
                                const int32_t* t_pos, const int32_t* t_off, void* x_out, int64_t M, int64_t W, int taps, int dtype,
                                void* stream) {
  B200P_REQUIRE(n && conv_w && conv_state && t_row && t_pos && t_off && x_out && W > 0, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(taps >= 1 && taps <= CANON_MAX_TAPS, B200P_ERR_ARG, "taps in [1, %d]", CANON_MAX_TAPS);
  if (M == 0) return B200P_OK;
  const unsigned threads = W >= 1024 ? 256 : 128;
  B200P_DISPATCH_DTYPE(dtype, T, (canon_conv_kernel<T><<<row_grid(M, W, threads), threads, 0, (cudaStream_t)stream>>>(
      n, conv_w, conv_state, t_row, t_pos, t_off, (T*)x_out, W, taps)));
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

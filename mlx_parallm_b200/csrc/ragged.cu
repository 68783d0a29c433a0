// Ragged-batch bookkeeping and the row-wise kernels of designs with a norm on both sides of every sublayer:
// per-token plan, end-of-step advance, hashed-bigram embedding, post-norm + residual + pre-norm, token-indexed gate.
#include "common.cuh"

namespace b200p {

__global__ void ragged_plan_kernel(const int32_t* __restrict__ cu, const int32_t* __restrict__ rows,
                                   const int32_t* __restrict__ lengths, int32_t* __restrict__ t_row, int32_t* __restrict__ t_pos,
                                   int32_t* __restrict__ t_off, int nb, int64_t M) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= M) return;
  int lo = 0, hi = nb - 1;                    // last entry e with cu[e] <= t (entries without tokens have cu[e] == cu[e+1])
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int r = rows[lo];
  const int off = (int)(t - cu[lo]);
  t_row[t] = r;
  t_off[t] = off;
  t_pos[t] = lengths[r] + off;
}

__global__ void ragged_advance_kernel(int32_t* __restrict__ lengths, int32_t* __restrict__ last_token,
                                      const int32_t* __restrict__ ids, const int32_t* __restrict__ cu,
                                      const int32_t* __restrict__ rows, int nb) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= nb) return;
  const int n = cu[e + 1] - cu[e];
  if (n <= 0) return;
  const int r = rows[e];
  lengths[r] += n;
  if (last_token) last_token[r] = ids[cu[e + 1] - 1];
}

template <typename T>
__global__ void embed_hashed_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ t_row,
                                    const int32_t* __restrict__ t_pos, const int32_t* __restrict__ t_off,
                                    const int32_t* __restrict__ last_token, const T* __restrict__ embed,
                                    const T* __restrict__ bigram, float* __restrict__ h, int64_t W, int64_t V, float scale,
                                    int64_t buckets, int64_t mul_prev, int64_t mul_cur) {
  const int64_t t = blockIdx.x;
  int64_t id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const T* e = embed + id * W;
  const T* b = nullptr;
  if (bigram) {
    int64_t bucket = buckets;                                     // the first token of a sequence
    if (t_pos[t] > 0) {
      const int64_t prev = t_off[t] > 0 ? ids[t - 1] : last_token[t_row[t]];
      bucket = ((prev % buckets) * (mul_prev % buckets) + (id % buckets) * (mul_cur % buckets)) % buckets;
      if (bucket < 0) bucket += buckets;
    }
    b = bigram + bucket * W;
  }
  float* o = h + t * W;
  for (int64_t c = threadIdx.x; c < W; c += blockDim.x) {
    float v = Tr<T>::to_f(e[c]) * scale;
    if (b) v += Tr<T>::to_f(b[c]);
    o[c] = v;
  }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();                 // red may still be read from an earlier call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < nw; ++i) s += red[i];      // same order in every thread
  return s;
}

template <typename T>
__global__ void norm_add_norm_kernel(const float* __restrict__ y, const float* __restrict__ w_post, float* __restrict__ h,
                                     const float* __restrict__ w_next, T* __restrict__ x_out, T* __restrict__ raw_out, int64_t W,
                                     float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  float* hr = h + row * W;
  if (y) {
    const float* yr = y + row * W;
    float ss = 0.f;
    for (int64_t c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(yr[c], yr[c], ss);
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)W + eps);
    float hs = 0.f;
    for (int64_t c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = hr[c] + yr[c] * inv * w_post[c];
      hr[c] = v;
      hs = fmaf(v, v, hs);
      if (raw_out) raw_out[row * W + c] = Tr<T>::from_f(v);
    }
    if (x_out) {
      hs = block_sum(hs, red);
      const float invh = 1.f / sqrtf(hs / (float)W + eps);
      for (int64_t c = threadIdx.x; c < W; c += blockDim.x) x_out[row * W + c] = Tr<T>::from_f(hr[c] * invh * w_next[c]);
    }
  } else {
    float hs = 0.f;
    for (int64_t c = threadIdx.x; c < W; c += blockDim.x) {
      const float v = hr[c];
      hs = fmaf(v, v, hs);
      if (raw_out) raw_out[row * W + c] = Tr<T>::from_f(v);
    }
    if (x_out) {
      hs = block_sum(hs, red);
      const float invh = 1.f / sqrtf(hs / (float)W + eps);
      for (int64_t c = threadIdx.x; c < W; c += blockDim.x) x_out[row * W + c] = Tr<T>::from_f(hr[c] * invh * w_next[c]);
    }
  }
}

// Residual stream of designs whose sublayers are added without a norm of their own (several branches may read one normed
// input and are summed into the stream together): h += c1 y1 + c2 y2, then the copies the next step needs.
template <typename T>
__global__ void residual_add_norm_kernel(float* __restrict__ h, const float* __restrict__ y1, float c1, const float* __restrict__ y2,
                                         float c2, const float* __restrict__ w_next, T* __restrict__ x_out, T* __restrict__ raw_out,
                                         int64_t ld_raw, int64_t W, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  float* hr = h + row * W;
  float hs = 0.f;
  for (int64_t c = threadIdx.x; c < W; c += blockDim.x) {
    float v = hr[c];
    if (y1 || y2) {
      float add = 0.f;
      if (y1) add = c1 * y1[row * W + c];
      if (y2) add += c2 * y2[row * W + c];
      v += add;
      hr[c] = v;
    }
    hs = fmaf(v, v, hs);
    if (raw_out) raw_out[row * ld_raw + c] = Tr<T>::from_f(v);
  }
  if (x_out) {
    hs = block_sum(hs, red);
    const float invh = 1.f / sqrtf(hs / (float)W + eps);
    for (int64_t c = threadIdx.x; c < W; c += blockDim.x) x_out[row * W + c] = Tr<T>::from_f(hr[c] * invh * w_next[c]);
  }
}

template <typename T>
__global__ void cast_columns_kernel(const float* __restrict__ src, int64_t ld_src, T* __restrict__ dst, int64_t ld_dst, int64_t M,
                                    int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * n) return;
  const int64_t t = i / n, c = i % n;
  dst[t * ld_dst + c] = Tr<T>::from_f(src[t * ld_src + c]);
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void token_gate_kernel(const float* __restrict__ gate, const T* __restrict__ table, const int32_t* __restrict__ ids,
                                  T* __restrict__ out, int64_t M, int d, int64_t ld_table, int64_t col0) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * d) return;
  const int64_t t = i / d;
  const int c = (int)(i % d);
  const float e = Tr<T>::to_f(table[(int64_t)ids[t] * ld_table + col0 + c]);
  out[i] = Tr<T>::from_f(gelu_tanh_f(gate[i]) * e);
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_ragged_plan(const int32_t* cu, const int32_t* rows, const int32_t* lengths, int32_t* t_row, int32_t* t_pos,
                                 int32_t* t_off, int nb, int64_t M, void* stream) {
  B200P_REQUIRE(cu && rows && lengths && t_row && t_pos && t_off && nb > 0, B200P_ERR_ARG, "null pointer or empty batch");
  if (M == 0) return B200P_OK;
  ragged_plan_kernel<<<(unsigned)((M + 255) / 256), 256, 0, (cudaStream_t)stream>>>(cu, rows, lengths, t_row, t_pos, t_off, nb, M);
  B200P_LAUNCH_CHECK("ragged_plan_kernel");
  return B200P_OK;
}

extern "C" int b200p_ragged_advance(int32_t* lengths, int32_t* last_token, const int32_t* ids, const int32_t* cu,
                                    const int32_t* rows, int nb, void* stream) {
  B200P_REQUIRE(lengths && ids && cu && rows && nb > 0, B200P_ERR_ARG, "null pointer or empty batch");
  ragged_advance_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, (cudaStream_t)stream>>>(lengths, last_token, ids, cu, rows, nb);
  B200P_LAUNCH_CHECK("ragged_advance_kernel");
  return B200P_OK;
}

extern "C" int b200p_embed_hashed(const int32_t* ids, const int32_t* t_row, const int32_t* t_pos, const int32_t* t_off,
                                  const int32_t* last_token, const void* embed, const void* bigram, float* h, int64_t M, int64_t W,
                                  int64_t V, float scale, int64_t buckets, int64_t mul_prev, int64_t mul_cur, int dtype,
                                  void* stream) {
  B200P_REQUIRE(ids && t_row && t_pos && t_off && embed && h, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(!bigram || (last_token && buckets > 0), B200P_ERR_ARG, "a bigram table needs last_token and buckets > 0");
  if (M == 0) return B200P_OK;
  const unsigned threads = W >= 1024 ? 256 : 128;
  B200P_DISPATCH_DTYPE(dtype, T, (embed_hashed_kernel<T><<<(unsigned)M, threads, 0, (cudaStream_t)stream>>>(
      ids, t_row, t_pos, t_off, last_token, (const T*)embed, (const T*)bigram, h, W, V, scale, buckets, mul_prev, mul_cur)));
  B200P_LAUNCH_CHECK("embed_hashed_kernel");
  return B200P_OK;
}

extern "C" int b200p_norm_add_norm(const float* y, const float* w_post, float* h, const float* w_next, void* x_out, void* raw_out,
                                   int64_t M, int64_t W, float eps, int dtype, void* stream) {
  B200P_REQUIRE(h && W > 0, B200P_ERR_ARG, "null residual stream");
  B200P_REQUIRE(!y || w_post, B200P_ERR_ARG, "y needs its norm weight");
  B200P_REQUIRE(!x_out || w_next, B200P_ERR_ARG, "x_out needs its norm weight");
  if (M == 0) return B200P_OK;
  const unsigned threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
  B200P_DISPATCH_DTYPE(dtype, T, (norm_add_norm_kernel<T><<<(unsigned)M, threads, 0, (cudaStream_t)stream>>>(
      y, w_post, h, w_next, (T*)x_out, (T*)raw_out, W, eps)));
  B200P_LAUNCH_CHECK("norm_add_norm_kernel");
  return B200P_OK;
}

extern "C" int b200p_residual_add_norm(float* h, const float* y1, float c1, const float* y2, float c2, const float* w_next,
                                       void* x_out, void* raw_out, int64_t ld_raw, int64_t M, int64_t W, float eps, int dtype,
                                       void* stream) {
  B200P_REQUIRE(h && W > 0, B200P_ERR_ARG, "null residual stream");
  B200P_REQUIRE(!x_out || w_next, B200P_ERR_ARG, "x_out needs its norm weight");
  B200P_REQUIRE(!raw_out || ld_raw >= W, B200P_ERR_ARG, "raw_out rows are shorter than the stream");
  if (M == 0) return B200P_OK;
  const unsigned threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
  B200P_DISPATCH_DTYPE(dtype, T, (residual_add_norm_kernel<T><<<(unsigned)M, threads, 0, (cudaStream_t)stream>>>(
      h, y1, c1, y2, c2, w_next, (T*)x_out, (T*)raw_out, ld_raw, W, eps)));
  B200P_LAUNCH_CHECK("residual_add_norm_kernel");
  return B200P_OK;
}

extern "C" int b200p_cast_columns(const float* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t M, int64_t n, int dtype,
                                  void* stream) {
  B200P_REQUIRE(src && dst && n > 0 && ld_src >= n && ld_dst >= n, B200P_ERR_ARG, "null pointer or bad shape");
  if (M == 0) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (cast_columns_kernel<T><<<(unsigned)((M * n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      src, ld_src, (T*)dst, ld_dst, M, n)));
  B200P_LAUNCH_CHECK("cast_columns_kernel");
  return B200P_OK;
}

extern "C" int b200p_token_gate(const float* gate, const void* table, const int32_t* ids, void* out, int64_t M, int d,
                                int64_t ld_table, int64_t col0, int dtype, void* stream) {
  B200P_REQUIRE(gate && table && ids && out && d > 0, B200P_ERR_ARG, "null pointer");
  if (M == 0) return B200P_OK;
  const int64_t n = M * d;
  B200P_DISPATCH_DTYPE(dtype, T, (token_gate_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      gate, (const T*)table, ids, (T*)out, M, d, ld_table, col0)));
  B200P_LAUNCH_CHECK("token_gate_kernel");
  return B200P_OK;
}

namespace b200p {
__global__ void scale_kernel(float* __restrict__ y, int64_t n, float s) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] *= s;
}
}  // namespace b200p

extern "C" int b200p_scale(float* y, int64_t n, float s, void* stream) {
  B200P_REQUIRE(y || n == 0, B200P_ERR_ARG, "null pointer");
  if (n == 0) return B200P_OK;
  b200p::scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(y, n, s);
  B200P_LAUNCH_CHECK("scale_kernel");
  return B200P_OK;
}

// Selective state-space layer (state-space duality form: a scalar decay per head and token), over a ragged batch.  The
// recurrence itself is the plain decayed accumulation of the delta-rule unit (b200p_delta_scan, B200P_SCAN_ACCUMULATE) with
// k = B, q = C (shared by the heads of a group), v = dt x and decay = exp(-exp(A_log) dt); this unit holds what surrounds it:
//   ssm_prep_kernel   short causal convolution (with bias) + silu of the x, B, C channels; dt = softplus(dt + dt_bias); the
//                     scan's inputs and the convolved x for the skip term                                               (per token)
//   ssm_out_kernel    y = o + D x; y * silu(z); rms norm in equal parts of the channels; weight                          (per token)
// The convolution's carried inputs are kept by b200p_delta_conv_commit.  Everything here is fp32 except the output row.
#include "common.cuh"

namespace b200p {

__device__ __forceinline__ float ssm_silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float ssm_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int SSM_MAX_TAPS = 16;

// proj row: [z (inner) | x (inner) | B (G N) | C (G N) | dt (H)], inner = H dv; the convolution runs over the channels x, B, C
// (column col_x + c, c < inner + 2 G N); tap j multiplies the input taps-1-j tokens back (the last tap is the current token's).
__global__ void ssm_prep_kernel(const float* __restrict__ proj, int64_t ldp, int64_t col_x, int64_t col_dt,
                                const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                                const float* __restrict__ conv_state, const float* __restrict__ A_log,
                                const float* __restrict__ dt_bias, const int32_t* __restrict__ t_row,
                                const int32_t* __restrict__ t_pos, const int32_t* __restrict__ t_off, float* __restrict__ xs,
                                float* __restrict__ v, float* __restrict__ kn, float* __restrict__ qn, float* __restrict__ decay,
                                int H, int dv, int GN, int taps) {
  extern __shared__ float dts[];                     // dt of every head of this token
  const int64_t t = blockIdx.x;
  const int inner = H * dv, C = inner + 2 * GN;
  const int row = t_row[t], pos = t_pos[t], off = t_off[t];
  const float* pt = proj + t * ldp;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float dt = ssm_softplus(pt[col_dt + h] + dt_bias[h]);
    dts[h] = dt;
    decay[t * H + h] = expf(-expf(A_log[h]) * dt);
  }
  __syncthreads();
  const float* px = pt + col_x;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = conv_b ? conv_b[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int d = taps - 1 - j;
      float in;
      if (d > pos) in = 0.f;                         // before the sequence
      else if (d <= off) in = px[c - (int64_t)d * ldp];
      else in = conv_state[((int64_t)row * (taps - 1) + (taps - 1 + off - d)) * C + c];
      acc = fmaf(conv_w[(int64_t)c * taps + j], in, acc);
    }
    const float a = ssm_silu(acc);
    if (c < inner) {
      xs[t * inner + c] = a;
      v[t * inner + c] = dts[c / dv] * a;
    } else if (c < inner + GN) {
      kn[t * GN + (c - inner)] = a;
    } else {
      qn[t * GN + (c - inner - GN)] = a;
    }
  }
}

// y = (o + D_h xs) * silu(z); the `parts` equal runs of the inner channels are each divided by their own root mean square;
// out (dtype, row stride ld_out) = that * norm_w[c].  A part is summed by `slices` warps in a fixed order.
template <typename T>
__global__ void ssm_out_kernel(const float* __restrict__ o, const float* __restrict__ xs, const float* __restrict__ z, int64_t ldz,
                               const float* __restrict__ D, const float* __restrict__ norm_w, T* __restrict__ out, int64_t ld_out,
                               int H, int dv, int parts, int slices, float eps) {
  extern __shared__ float ssm_sm[];                  // y [inner], then the partial sums [parts * slices]
  const int64_t t = blockIdx.x;
  const int inner = H * dv, len = inner / parts;
  float* y = ssm_sm;
  float* red = ssm_sm + inner;
  const float* zt = z + t * ldz;
  for (int c = threadIdx.x; c < inner; c += blockDim.x)
    y[c] = fmaf(D ? D[c / dv] : 0.f, xs[t * inner + c], o[t * inner + c]) * ssm_silu(zt[c]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int idx = warp; idx < parts * slices; idx += nw) {
    const int g = idx / slices, s = idx % slices;
    const int c0 = g * len + (int)((int64_t)len * s / slices), c1 = g * len + (int)((int64_t)len * (s + 1) / slices);
    float ss = 0.f;
    for (int c = c0 + lane; c < c1; c += 32) ss = fmaf(y[c], y[c], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[idx] = ss;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < inner; c += blockDim.x) {
    const int g = c / len;
    float tot = 0.f;
    for (int s = 0; s < slices; ++s) tot += red[g * slices + s];
    out[t * ld_out + c] = Tr<T>::from_f(y[c] / sqrtf(tot / (float)len + eps) * norm_w[c]);
  }
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_ssm_prep(const float* proj, int64_t ldp, int64_t col_x, int64_t col_dt, const float* conv_w, const float* conv_b,
                              const float* conv_state, const float* A_log, const float* dt_bias, const int32_t* t_row,
                              const int32_t* t_pos, const int32_t* t_off, float* xs, float* v, float* kn, float* qn, float* decay,
                              int64_t M, int H, int dv, int groups, int state, int taps, void* stream) {
  B200P_REQUIRE(proj && conv_w && conv_state && A_log && dt_bias && t_row && t_pos && t_off && xs && v && kn && qn && decay,
                B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(H > 0 && dv > 0 && groups > 0 && state > 0 && H % groups == 0, B200P_ERR_ARG, "bad head geometry");
  B200P_REQUIRE(taps >= 1 && taps <= SSM_MAX_TAPS, B200P_ERR_ARG, "convolution taps must be in [1, %d]", SSM_MAX_TAPS);
  B200P_REQUIRE((size_t)H * sizeof(float) <= 48 * 1024, B200P_ERR_ARG, "too many heads");
  if (M == 0) return B200P_OK;
  const unsigned threads = M <= 256 ? 1024 : 256;        // a decode batch has few tokens and thousands of channels each
  ssm_prep_kernel<<<(unsigned)M, threads, (size_t)H * sizeof(float), (cudaStream_t)stream>>>(
      proj, ldp, col_x, col_dt, conv_w, conv_b, conv_state, A_log, dt_bias, t_row, t_pos, t_off, xs, v, kn, qn, decay, H, dv,
      groups * state, taps);
  B200P_LAUNCH_CHECK("ssm_prep_kernel");
  return B200P_OK;
}

extern "C" int b200p_ssm_out(const float* o, const float* xs, const float* z, int64_t ldz, const float* D, const float* norm_w,
                             void* out, int64_t ld_out, int64_t M, int H, int dv, int parts, float eps, int dtype, void* stream) {
  B200P_REQUIRE(o && xs && z && norm_w && out && H > 0 && dv > 0, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(parts > 0 && (H * dv) % parts == 0, B200P_ERR_ARG, "the channels do not split into %d equal parts", parts);
  B200P_REQUIRE(ld_out >= (int64_t)H * dv, B200P_ERR_ARG, "output rows are shorter than the channels");
  if (M == 0) return B200P_OK;
  const int inner = H * dv;
  const unsigned threads = inner >= 2048 ? 512 : inner >= 512 ? 256 : 128;
  const int nw = threads / 32;
  const int slices = parts >= nw ? 1 : nw / parts;
  const size_t smem = ((size_t)inner + (size_t)parts * slices) * sizeof(float);
  B200P_REQUIRE(smem <= 200 * 1024, B200P_ERR_ARG, "%d channels do not fit the shared memory of one block", inner);
#define SSM_OUT(T)                                                                                                       \
  do {                                                                                                                   \
    auto kern = ssm_out_kernel<T>;                                                                                       \
    if (smem > 48 * 1024) {                                                                                              \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(ssm_out_kernel)");                                 \
    }                                                                                                                    \
    kern<<<(unsigned)M, threads, smem, (cudaStream_t)stream>>>(o, xs, z, ldz, D, norm_w, (T*)out, ld_out, H, dv, parts, \
                                                               slices, eps);                                             \
  } while (0)
  switch (dtype) {
    case B200P_F32: SSM_OUT(float); break;
    case B200P_F16: SSM_OUT(__half); break;
    case B200P_BF16: SSM_OUT(__nv_bfloat16); break;
    default: set_error("bad dtype %d", dtype); return B200P_ERR_ARG;
  }
#undef SSM_OUT
  B200P_LAUNCH_CHECK("ssm_out_kernel");
  return B200P_OK;
}

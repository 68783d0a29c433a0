// Routed mixture of experts over a packed token batch:
//   moe_route_kernel    fp32 router logits (+ bias) -> the `top` largest per token and the softmax over those alone   (per token)
//   moe_route_sigmoid_kernel  scores = sigmoid(logits); experts picked by score + correction inside the best expert groups;
//                       weights = the picked experts' scores over their sum, times a scale                              (per token)
//   moe_plan_kernel     tokens counted per expert, segment offsets, a slot for every (token, choice)                 (one CTA)
//   moe_gather_kernel   activation rows copied into slot order, so that an expert's rows are contiguous              (per slot)
//   moe_combine_kernel  y[t] = gate[t] shared[t] + sum_k weight[t, k] * expert_out[slot(t, k)], in the order of the choices   (per token)
// The experts themselves are two grouped GEMMs (b200p_gemm_grouped) over the segments.  Every launch has the same shape whatever
// the routing, so a decode step with experts sits in a captured graph.
#include "common.cuh"

namespace b200p {

constexpr int MOE_MAX_PER_LANE = 32;    // experts <= 1024
constexpr int MOE_MAX_TOP = 32;

__global__ void moe_route_kernel(const float* __restrict__ logits, int64_t ldl, const float* __restrict__ bias,
                                 int32_t* __restrict__ ids, float* __restrict__ wts, int64_t M, int E, int top) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= M) return;
  float z[MOE_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
    const int e = i * 32 + lane;
    z[i] = e < E ? logits[t * ldl + e] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  float first = 0.f, den = 0.f, mine = 0.f;
  int my_id = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int be = E;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i)
      if (z[i] > best) { best = z[i]; be = i * 32 + lane; }          // ascending e within a lane: ties keep the smallest index
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if (k == 0) first = best;
    const float p = expf(best - first);                              // the first pick is the largest: exponents <= 0
    den += p;
    if (lane == k) { mine = p; my_id = be; }
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i)
      if (i * 32 + lane == be) z[i] = -INFINITY;
  }
  if (lane < top) {
    ids[t * top + lane] = my_id;
    wts[t * top + lane] = mine / den;
  }
}

// One warp per token.  s_e = sigmoid(z_e); picking score c_e = s_e + correction_e.  The experts form `count` groups of
// neighbours; a group's score is the sum of its two largest picking scores (its only one for groups of one expert); only the
// experts of the `keep` best groups can be picked (the others count as -inf, since picking scores may be negative).  The `top`
// largest picking scores win, ties to the smaller index; weights w_k = s_k / (sum of the picked s + 1e-20) * scale.
__global__ void moe_route_sigmoid_kernel(const float* __restrict__ logits, int64_t ldl, const float* __restrict__ correction,
                                         int32_t* __restrict__ ids, float* __restrict__ wts, int64_t M, int E, int top, int count,
                                         int keep, float scale, int renorm) {
  extern __shared__ float mr_sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= M) return;
  float* sc = mr_sm + (size_t)warp * (2 * E + count);     // scores
  float* pick = sc + E;                                    // picking scores, -inf once masked or taken
  float* gs = pick + E;                                    // group scores
  for (int e = lane; e < E; e += 32) {
    const float s = 1.f / (1.f + expf(-logits[t * ldl + e]));
    sc[e] = s;
    pick[e] = s + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (count > 1 && keep < count) {
    const int per = E / count;
    for (int g = lane; g < count; g += 32) {
      float a = -INFINITY, b = -INFINITY;                  // the two largest of the group
      for (int i = 0; i < per; ++i) {
        const float v = pick[g * per + i];
        if (v > a) { b = a; a = v; }
        else if (v > b) b = v;
      }
      gs[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // drop the count - keep worst groups: repeatedly the smallest score, ties dropping the larger index first
    for (int r = 0; r < count - keep; ++r) {
      float worst = INFINITY;
      int wg = -1;
      for (int g = lane; g < count; g += 32) {
        const float v = gs[g];
        if (v == v && (v < worst || (v == worst && g > wg))) { worst = v; wg = g; }      // NaN marks a dropped group
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ow = __shfl_xor_sync(0xffffffffu, worst, o);
        const int og = __shfl_xor_sync(0xffffffffu, wg, o);
        if (og >= 0 && (wg < 0 || ow < worst || (ow == worst && og > wg))) { worst = ow; wg = og; }
      }
      if (lane == 0) gs[wg] = __int_as_float(0x7fc00000);
      for (int i = lane; i < per; i += 32) pick[wg * per + i] = -INFINITY;
      __syncwarp();
    }
  }
  float den = 0.f, mine = 0.f;
  int my_id = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int be = E;
    for (int e = lane; e < E; e += 32)
      if (pick[e] > best) { best = pick[e]; be = e; }                  // ascending e within a lane: ties keep the smallest index
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if (be >= E) be = 0;                                               // fewer candidates than picks: cannot happen with keep * per >= top
    const float s = sc[be];
    den += s;
    if (lane == k) { mine = s; my_id = be; }
    __syncwarp();
    if (lane == 0) pick[be] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    ids[t * top + lane] = my_id;
    wts[t * top + lane] = renorm ? mine / (den + 1e-20f) * scale : mine * scale;       // renorm 0: the scores as they are
  }
}

__global__ void moe_plan_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ seg, int32_t* __restrict__ slot_of,
                                int32_t* __restrict__ token_of, int64_t n, int E, int top) {
  extern __shared__ int32_t cnt[];               // [E] counts, then [E] cursors
  int32_t* cur = cnt + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t run = 0;
    for (int e = 0; e < E; ++e) {
      seg[e] = run;
      cur[e] = run;
      run += cnt[e];
    }
    seg[E] = run;
  }
  __syncthreads();
  // the order of an expert's rows is whatever the atomics give: every row is computed on its own, so the values do not depend on it
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const int32_t s = atomicAdd(&cur[ids[i]], 1);
    slot_of[i] = s;
    token_of[s] = (int32_t)(i / top);
  }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int32_t* __restrict__ token_of, T* __restrict__ xs, int64_t W) {
  const int64_t s = blockIdx.x;
  const T* src = x + (int64_t)token_of[s] * W;
  T* dst = xs + s * W;
  if (W % 8 == 0 && sizeof(T) == 2) {
    for (int64_t c = threadIdx.x * 8; c < W; c += blockDim.x * 8) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
  } else {
    for (int64_t c = threadIdx.x; c < W; c += blockDim.x) dst[c] = src[c];
  }
}

// xs[slot_of[t, k], :] = wts[t, k] * x[t, :]: designs whose routing weight multiplies the expert's INPUT (the product is
// formed in fp32 and rounded once to the storage type)
template <typename T>
__global__ void moe_scatter_scaled_kernel(const T* __restrict__ x, const int32_t* __restrict__ slot_of, const float* __restrict__ wts,
                                          T* __restrict__ xs, int64_t W) {
  const int64_t i = blockIdx.x;                        // (token, choice)
  const int top = gridDim.y;
  const int64_t tk = i * top + blockIdx.y;
  const float w = wts[tk];
  const T* src = x + i * W;
  T* dst = xs + (int64_t)slot_of[tk] * W;
  if (sizeof(T) == 2 && W % 8 == 0) {                  // 16-byte pieces of eight 16-bit values (rows start on 16-byte boundaries)
    for (int64_t c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
      uint4 raw = *reinterpret_cast<const uint4*>(src + c);
      T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = Tr<T>::from_f(w * Tr<T>::to_f(v[i]));
      *reinterpret_cast<uint4*>(dst + c) = raw;
    }
    return;
  }
  for (int64_t c = threadIdx.x; c < W; c += blockDim.x) dst[c] = Tr<T>::from_f(w * Tr<T>::to_f(src[c]));
}

__global__ void moe_combine_kernel(const float* __restrict__ ye, const int32_t* __restrict__ slot_of, const float* __restrict__ wts,
                                   const float* __restrict__ shared_y, const float* __restrict__ shared_gate, int64_t ldg,
                                   float* __restrict__ y, int64_t W, int top) {
  const int64_t t = blockIdx.x;
  const float sg = shared_gate ? 1.f / (1.f + expf(-shared_gate[t * ldg])) : 1.f;
  __shared__ int32_t sl[MOE_MAX_TOP];
  __shared__ float wt[MOE_MAX_TOP];
  if (threadIdx.x < top) {
    sl[threadIdx.x] = slot_of[t * top + threadIdx.x];
    wt[threadIdx.x] = wts ? wts[t * top + threadIdx.x] : 1.f;
  }
  __syncthreads();
  for (int64_t c = threadIdx.x; c < W; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) a = fmaf(wt[k], ye[(int64_t)sl[k] * W + c], a);
    if (shared_y) a = fmaf(sg, shared_y[t * W + c], a);
    y[t * W + c] = a;
  }
}

}  // namespace b200p

using namespace b200p;

extern "C" int b200p_moe_route(const float* logits, int64_t ldl, const float* bias, int32_t* ids, float* wts, int32_t* seg,
                               int32_t* slot_of, int32_t* token_of, int64_t M, int E, int top, void* stream) {
  B200P_REQUIRE(logits && ids && wts && seg && slot_of && token_of, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(E > 0 && E <= 32 * MOE_MAX_PER_LANE && top > 0 && top <= E && top <= MOE_MAX_TOP, B200P_ERR_ARG,
                "experts in [1, %d] and top in [1, min(experts, %d)]", 32 * MOE_MAX_PER_LANE, MOE_MAX_TOP);
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  moe_route_kernel<<<(unsigned)((M + 3) / 4), 128, 0, st>>>(logits, ldl, bias, ids, wts, M, E, top);
  B200P_LAUNCH_CHECK("moe_route_kernel");
  moe_plan_kernel<<<1, 1024, 2 * E * sizeof(int32_t), st>>>(ids, seg, slot_of, token_of, M * top, E, top);
  B200P_LAUNCH_CHECK("moe_plan_kernel");
  return B200P_OK;
}

extern "C" int b200p_moe_route_sigmoid(const float* logits, int64_t ldl, const float* correction, int32_t* ids, float* wts,
                                       int32_t* seg, int32_t* slot_of, int32_t* token_of, int64_t M, int E, int top, int count,
                                       int keep, float scale, void* stream) {
  B200P_REQUIRE(logits && ids && wts && seg && slot_of && token_of, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(E > 0 && E <= 32 * MOE_MAX_PER_LANE && top > 0 && top <= E && top <= MOE_MAX_TOP, B200P_ERR_ARG,
                "experts in [1, %d] and top in [1, min(experts, %d)]", 32 * MOE_MAX_PER_LANE, MOE_MAX_TOP);
  B200P_REQUIRE(count >= 1 && E % count == 0 && keep >= 1 && keep <= count && (int64_t)keep * (E / count) >= top, B200P_ERR_ARG,
                "expert groups: equal groups, 1 <= keep <= count, and the kept groups hold at least `top` experts");
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int warps = 4;
  const size_t smem = (size_t)warps * (2 * E + count) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_route_sigmoid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(moe_route_sigmoid_kernel)");
  }
  moe_route_sigmoid_kernel<<<(unsigned)((M + warps - 1) / warps), warps * 32, smem, st>>>(logits, ldl, correction, ids, wts, M, E, top,
                                                                                           count, keep, scale, 1);
  B200P_LAUNCH_CHECK("moe_route_sigmoid_kernel");
  moe_plan_kernel<<<1, 1024, 2 * E * sizeof(int32_t), st>>>(ids, seg, slot_of, token_of, M * top, E, top);
  B200P_LAUNCH_CHECK("moe_plan_kernel");
  return B200P_OK;
}

extern "C" int b200p_moe_route_scores(const float* logits, int64_t ldl, int32_t* ids, float* wts, int32_t* seg, int32_t* slot_of,
                                      int32_t* token_of, int64_t M, int E, int top, void* stream) {
  B200P_REQUIRE(logits && ids && wts && seg && slot_of && token_of, B200P_ERR_ARG, "null pointer");
  B200P_REQUIRE(E > 0 && E <= 32 * MOE_MAX_PER_LANE && top > 0 && top <= E && top <= MOE_MAX_TOP, B200P_ERR_ARG,
                "experts in [1, %d] and top in [1, min(experts, %d)]", 32 * MOE_MAX_PER_LANE, MOE_MAX_TOP);
  if (M == 0) return B200P_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int warps = 4;
  const size_t smem = (size_t)warps * (2 * E + 1) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_route_sigmoid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(moe_route_sigmoid_kernel)");
  }
  moe_route_sigmoid_kernel<<<(unsigned)((M + warps - 1) / warps), warps * 32, smem, st>>>(logits, ldl, nullptr, ids, wts, M, E, top, 1, 1,
                                                                                           1.f, 0);
  B200P_LAUNCH_CHECK("moe_route_sigmoid_kernel");
  moe_plan_kernel<<<1, 1024, 2 * E * sizeof(int32_t), st>>>(ids, seg, slot_of, token_of, M * top, E, top);
  B200P_LAUNCH_CHECK("moe_plan_kernel");
  return B200P_OK;
}

extern "C" int b200p_moe_scatter_scaled(const void* x, const int32_t* slot_of, const float* wts, void* xs, int64_t M, int64_t W, int top,
                                        int dtype, void* stream) {
  B200P_REQUIRE(x && slot_of && wts && xs && W > 0 && top > 0 && top <= MOE_MAX_TOP, B200P_ERR_ARG, "null pointer or bad top");
  B200P_REQUIRE(dtype == B200P_F32 || W % 8 != 0 || (aligned(x, 16) && aligned(xs, 16)), B200P_ERR_ALIGN, "x and xs must be 16-byte aligned");
  if (M == 0) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (moe_scatter_scaled_kernel<T><<<dim3((unsigned)M, (unsigned)top), 128, 0, (cudaStream_t)stream>>>(
      (const T*)x, slot_of, wts, (T*)xs, W)));
  B200P_LAUNCH_CHECK("moe_scatter_scaled_kernel");
  return B200P_OK;
}

extern "C" int b200p_moe_gather(const void* x, const int32_t* token_of, void* xs, int64_t slots, int64_t W, int dtype, void* stream) {
  B200P_REQUIRE(x && token_of && xs && W > 0, B200P_ERR_ARG, "null pointer");
  if (slots == 0) return B200P_OK;
  B200P_DISPATCH_DTYPE(dtype, T, (moe_gather_kernel<T><<<(unsigned)slots, 128, 0, (cudaStream_t)stream>>>(
      (const T*)x, token_of, (T*)xs, W)));
  B200P_LAUNCH_CHECK("moe_gather_kernel");
  return B200P_OK;
}

extern "C" int b200p_moe_combine(const float* ye, const int32_t* slot_of, const float* wts, const float* shared_y,
                                 const float* shared_gate, int64_t ldg, float* y, int64_t M, int64_t W, int top, void* stream) {
  B200P_REQUIRE(ye && slot_of && y && W > 0 && top > 0 && top <= MOE_MAX_TOP, B200P_ERR_ARG, "null pointer or bad top");
  if (M == 0) return B200P_OK;
  moe_combine_kernel<<<(unsigned)M, W >= 1024 ? 256 : 128, 0, (cudaStream_t)stream>>>(ye, slot_of, wts, shared_y, shared_gate, ldg, y, W, top);
  B200P_LAUNCH_CHECK("moe_combine_kernel");
  return B200P_OK;
}

// A mixture of gated feed-forward experts, token by token: every token goes to the `top` experts with the largest router
// logits, weighted by the softmax over those logits only.
//
//   moe_route:  a block per token: logits = W_r x + b in float32 from the float32 stream, `top` rounds of arg-max (the
//               lower expert on ties), then the weights.
//   moe_up:     per (token, choice): the chosen expert's gate and up rows times the token's activations, then the
//               clamped gated unit g sigmoid(alpha g) (u + shift), g = min(gate, limit), u = clamp(up, -limit, limit).
//               Gate and up rows interleave in the stacked weight [experts, 2 ff, width].
//   moe_down:   per token: sum over its choices of weight * W_down[expert] act, stored (or added) in float32.
//
// A warp owns an output value: its lanes split the reduction in 16-byte pieces, sums in float32. These kernels read an
// expert's weights once per token that chose it, which is what a step of few tokens needs.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;
constexpr int MAX_EXPERTS = 256;
constexpr int MAX_TOP = 16;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ float piece(const float* a, const float* b) {
  float4 x = *(const float4*)a, y = *(const float4*)b;
  return fmaf(x.w, y.w, fmaf(x.z, y.z, fmaf(x.y, y.y, x.x * y.x)));
}
__device__ __forceinline__ float piece(const __nv_bfloat16* a, const __nv_bfloat16* b) {
  uint4 ra = *(const uint4*)a, rb = *(const uint4*)b;
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
    s = fmaf(x.x, y.x, s);
    s = fmaf(x.y, y.y, s);
  }
  return s;
}

// This lane's share of a . b over n values (the warp's shares add up to the dot product).
template <typename T>
__device__ __forceinline__ float lane_dot(const T* a, const T* b, int n, int lane) {
  float s = 0.f;
  if (n % Vec<T>::N == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
    for (int d = lane * Vec<T>::N; d < n; d += 32 * Vec<T>::N) s += piece(a + d, b + d);
  } else {
    for (int d = lane; d < n; d += 32) s = fmaf(to_float(a[d]), to_float(b[d]), s);
  }
  return s;
}

// The router's weights are float32 whatever the activations are.
template <typename X>
__device__ __forceinline__ float lane_dot_router(const float* w, const X* x, int n, int lane) {
  float s = 0.f;
  for (int d = lane; d < n; d += 32) s = fmaf(w[d], to_float(x[d]), s);
  return s;
}
template <>
__device__ __forceinline__ float lane_dot_router<float>(const float* w, const float* x, int n, int lane) {
  return lane_dot(w, x, n, lane);
}

template <typename X>
__global__ void __launch_bounds__(WARPS * 32) moe_route_kernel(
    const X* __restrict__ x, int width, const float* __restrict__ w, const float* __restrict__ bias, int experts,
    int top, int tokens, int* __restrict__ chosen, float* __restrict__ weights) {
  // a block per token: its warps share the experts' logits out, warp 0 then chooses
  __shared__ float logits[MAX_EXPERTS];
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int t = blockIdx.x;
  const X* row = x + (size_t)t * width;
  for (int e = warp; e < experts; e += WARPS) {
    float s = warp_sum(lane_dot_router(w + (size_t)e * width, row, width, lane));
    if (lane == 0) logits[e] = s + (bias != nullptr ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  float kept[MAX_TOP];
  float largest = 0.f, total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int where = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      float v = logits[e];
      if (v > best) { best = v; where = e; }  // (ascending e: the first of equals stays)
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int ow = __shfl_xor_sync(0xffffffffu, where, o);
      if (ov > best || (ov == best && ow < where)) { best = ov; where = ow; }
    }
    if (where == 0x7fffffff) where = k;  // (only rows without a finite logit)
    if (k == 0) largest = best;
    kept[k] = expf(best - largest);
    total += kept[k];
    if (lane == 0) {
      chosen[(size_t)t * top + k] = where;
      logits[where] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0)
    for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] = kept[k] / total;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) moe_up_kernel(
    T* __restrict__ act, const T* __restrict__ h, int width, const T* __restrict__ w_gate_up, int ff, int top,
    const int* __restrict__ chosen, float limit, float alpha, float shift) {
  pdl_launch_dependents();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int f = blockIdx.y * WARPS + warp;
  if (f >= ff) return;
  pdl_wait();
  int a = blockIdx.x;
  int e = chosen[a];
  const T* row = h + (size_t)(a / top) * width;
  const T* wg = w_gate_up + ((size_t)e * 2 * ff + 2 * f) * width;
  float g = warp_sum(lane_dot(wg, row, width, lane));
  float u = warp_sum(lane_dot(wg + width, row, width, lane));
  if (lane == 0) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    act[(size_t)a * ff + f] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + shift));
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) moe_down_kernel(
    float* __restrict__ out, const T* __restrict__ act, int ff, const T* __restrict__ w_down, int width, int top,
    const int* __restrict__ chosen, const float* __restrict__ weights, int accumulate) {
  pdl_launch_dependents();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int n = blockIdx.y * WARPS + warp;
  if (n >= width) return;
  pdl_wait();
  int t = blockIdx.x;
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    int a = t * top + k;
    int e = chosen[a];
    float s = warp_sum(lane_dot(w_down + ((size_t)e * width + n) * ff, act + (size_t)a * ff, ff, lane));
    sum = fmaf(weights[a], s, sum);
  }
  if (lane == 0) {
    size_t at = (size_t)t * width + n;
    out[at] = accumulate ? out[at] + sum : sum;
  }
}
}  // namespace

DLLM_EXPORT int dllm_moe_route(const void* x, int width, const float* w, const float* bias, int experts, int top,
                               int tokens, int* chosen, float* weights, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (experts <= 0 || experts > MAX_EXPERTS || top <= 0 || top > MAX_TOP || top > experts || width <= 0)
    return DLLM_UNSUPPORTED_SIZE;
  if (x == nullptr || w == nullptr || chosen == nullptr || weights == nullptr) return DLLM_BAD_ARGUMENT;
  dim3 grid(tokens), block(WARPS * 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(moe_route_kernel<float>, grid, block, 0, stream, (const float*)x, width, w, bias, experts,
                           top, tokens, chosen, weights);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(moe_route_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, width, w,
                           bias, experts, top, tokens, chosen, weights);
  return DLLM_BAD_ARGUMENT;
}

DLLM_EXPORT int dllm_moe_up(void* act, const void* h, int width, const void* w_gate_up, int ff, int top, int tokens,
                            const int* chosen, float limit, float alpha, float shift, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || ff <= 0 || top <= 0 || ff > 65535 * WARPS) return DLLM_UNSUPPORTED_SIZE;
  dim3 grid(tokens * top, (ff + WARPS - 1) / WARPS), block(WARPS * 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(moe_up_kernel<float>, grid, block, 0, stream, (float*)act, (const float*)h, width,
                           (const float*)w_gate_up, ff, top, chosen, limit, alpha, shift);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(moe_up_kernel<__nv_bfloat16>, grid, block, 0, stream, (__nv_bfloat16*)act,
                           (const __nv_bfloat16*)h, width, (const __nv_bfloat16*)w_gate_up, ff, top, chosen, limit, alpha,
                           shift);
  return DLLM_BAD_ARGUMENT;
}

DLLM_EXPORT int dllm_moe_down(float* out, const void* act, int ff, const void* w_down, int width, int top, int tokens,
                              const int* chosen, const float* weights, int accumulate, int dtype,
                              cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || ff <= 0 || top <= 0 || width > 65535 * WARPS) return DLLM_UNSUPPORTED_SIZE;
  dim3 grid(tokens, (width + WARPS - 1) / WARPS), block(WARPS * 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(moe_down_kernel<float>, grid, block, 0, stream, out, (const float*)act, ff,
                           (const float*)w_down, width, top, chosen, weights, accumulate);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(moe_down_kernel<__nv_bfloat16>, grid, block, 0, stream, out, (const __nv_bfloat16*)act, ff,
                           (const __nv_bfloat16*)w_down, width, top, chosen, weights, accumulate);
  return DLLM_BAD_ARGUMENT;
}

// CUDA-core attention over the cache: one warp per (row, query token, head), fp32 math, online
// softmax, 8 keys per step.  Serves fp32 caches and checks the tensor-core kernel on the device.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "sdv2_internal.h"

namespace sdv2 {

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);

template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xFFFF0000u));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y);
  __nv_bfloat162 b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

constexpr int kKeysPerStep = 8;

template <typename T>
__global__ void __launch_bounds__(128) attn_simt_kernel(const __grid_constant__ SimtAttnParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t total = static_cast<int64_t>(p.rows) * p.q_tokens * p.heads;
  if (warp_global >= total) return;  // whole warp leaves together
  const int h = static_cast<int>(warp_global % p.heads);
  const int64_t r = warp_global / p.heads;
  const int t = static_cast<int>(r % p.q_tokens);
  const int b = static_cast<int>(r / p.q_tokens);
  const int len = p.seq_lens[b];

  const T* qp = static_cast<const T*>(p.q.ptr) + b * p.q.stride_row + t * p.q.stride_tok + h * p.q.stride_head + lane * 4;
  const T* kbase = static_cast<const T*>(p.k.ptr) + b * p.k.stride_row + h * p.k.stride_head + lane * 4;
  const T* vbase = static_cast<const T*>(p.v.ptr) + b * p.v.stride_row + h * p.v.stride_head + lane * 4;
  float4 q = load4<T>(qp);
  q.x *= p.scale; q.y *= p.scale; q.z *= p.scale; q.w *= p.scale;

  float m = -INFINITY, l = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < len; s0 += kKeysPerStep) {
    float sc[kKeysPerStep];
#pragma unroll
    for (int i = 0; i < kKeysPerStep; ++i) {
      const int s = s0 + i;
      float d = 0.f;
      if (s < len) {
        const float4 k = load4<T>(kbase + static_cast<int64_t>(s) * p.k.stride_tok);
        d = q.x * k.x + q.y * k.y + q.z * k.z + q.w * k.w;
      }
      sc[i] = d;
    }
#pragma unroll
    for (int i = 0; i < kKeysPerStep; ++i) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], o);
      if (s0 + i >= len) sc[i] = -INFINITY;
    }
    float mx = m;
#pragma unroll
    for (int i = 0; i < kKeysPerStep; ++i) mx = fmaxf(mx, sc[i]);
    const float alpha = __expf(m - mx);  // m = -inf on the first step gives 0
    l *= alpha;
    acc.x *= alpha; acc.y *= alpha; acc.z *= alpha; acc.w *= alpha;
    m = mx;
#pragma unroll
    for (int i = 0; i < kKeysPerStep; ++i) {
      const int s = s0 + i;
      if (s < len) {
        const float pr = __expf(sc[i] - m);
        l += pr;
        const float4 v = load4<T>(vbase + static_cast<int64_t>(s) * p.v.stride_tok);
        acc.x += pr * v.x; acc.y += pr * v.y; acc.z += pr * v.z; acc.w += pr * v.w;
      }
    }
  }
  const float inv = 1.f / l;
  T* op = static_cast<T*>(p.out.ptr) + b * p.out.stride_row + t * p.out.stride_tok + h * p.out.stride_head + lane * 4;
  store4(op, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
}

cudaError_t launch_attn_simt(const SimtAttnParams& p, int dtype, cudaStream_t stream) {
  const int64_t warps = static_cast<int64_t>(p.rows) * p.q_tokens * p.heads;
  const int threads = 128;
  const int64_t blocks = (warps * 32 + threads - 1) / threads;
  if (blocks <= 0 || blocks > 0x7FFFFFFFLL) return cudaErrorInvalidValue;
  if (dtype == SDV2_DTYPE_BF16)
    attn_simt_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p);
  else
    attn_simt_kernel<float><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace sdv2

// Fused 3D rotary embedding + K/V slot write for the sink + ring-buffer cache.
//
// One thread owns one 16-byte vector position (b, t, c) and walks a few heads with it, so the
// rope table entries (4 complex doubles for bf16, 2 for fp32) are fetched once and reused.
// All global accesses are 16-byte vectors; a warp touches whole 256/512-byte head rows.
// Pure streaming: 3 reads + 3 writes of [rows, tokens, heads, head_dim]; bound by HBM bandwidth.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sdv2_internal.h"

namespace sdv2 {

// bf16 bit pattern -> double, exactly.  Normal numbers are rebuilt with integer ops (the
// conversion unit is far narrower than the integer pipe); zero/subnormal/inf/nan take the
// hardware conversion.
__device__ __forceinline__ double bf16_bits_to_f64(uint32_t b) {
  const uint32_t em = b & 0x7FFFu;
  const uint32_t e = em >> 7;
  if (e != 0u && e != 0xFFu) {
    const uint32_t hi = ((b & 0x8000u) << 16) | ((em << 13) + 0x38000000u);
    return __hiloint2double(static_cast<int>(hi), 0);
  }
  return static_cast<double>(__uint_as_float(b << 16));
}

// (a + ib) * (c + id) with every product and sum rounded separately, as the reference's CPU
// complex128 multiply does; then fp64 -> fp32 (RN).  bf16 storage adds a second RNE step.
__device__ __forceinline__ void rope_pair(double a, double b, double2 cs, float& re, float& im) {
  re = __double2float_rn(__dsub_rn(__dmul_rn(a, cs.x), __dmul_rn(b, cs.y)));
  im = __double2float_rn(__dadd_rn(__dmul_rn(a, cs.y), __dmul_rn(b, cs.x)));
}

template <typename T>
struct Vec;  // 16-byte vector of T

template <>
struct Vec<__nv_bfloat16> {
  static constexpr int kPairs = 4;
  __device__ static uint4 rope(uint4 x, const double2 (&cs)[4]) {
    uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float re, im;
      rope_pair(bf16_bits_to_f64(w[i] & 0xFFFFu), bf16_bits_to_f64(w[i] >> 16), cs[i], re, im);
      const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(re));
      const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(im));
      w[i] = lo | (hi << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <>
struct Vec<float> {
  static constexpr int kPairs = 2;
  __device__ static uint4 rope(uint4 x, const double2 (&cs)[2]) {
    float re0, im0, re1, im1;
    rope_pair(static_cast<double>(__uint_as_float(x.x)), static_cast<double>(__uint_as_float(x.y)), cs[0],
              re0, im0);
    rope_pair(static_cast<double>(__uint_as_float(x.z)), static_cast<double>(__uint_as_float(x.w)), cs[1],
              re1, im1);
    return make_uint4(__float_as_uint(re0), __float_as_uint(im0), __float_as_uint(re1), __float_as_uint(im1));
  }
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ void st_vec(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

constexpr int kHeadsPerThread = 4;

template <typename T>
__global__ void __launch_bounds__(256) rope_kv_append_kernel(const __grid_constant__ AppendParams p) {
  constexpr int kPairs = Vec<T>::kPairs;
  constexpr int kElems = 2 * kPairs;
  const int vph = p.head_dim / kElems;  // vectors per head row
  const int hgroups = (p.heads + kHeadsPerThread - 1) / kHeadsPerThread;
  const int64_t total = static_cast<int64_t>(p.rows) * p.tokens * hgroups * vph;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;

  if (idx == 0 && p.global_end_dev != nullptr) {
    for (int b = 0; b < p.rows; ++b) {
      p.global_end_dev[b] = p.global_end_val[b];
      p.local_end_dev[b] = p.local_end_val[b];
    }
  }
  if (idx >= total) return;

  const int c = static_cast<int>(idx % vph);
  int64_t r = idx / vph;
  const int hg = static_cast<int>(r % hgroups);
  r /= hgroups;
  const int t = static_cast<int>(r % p.tokens);
  const int b = static_cast<int>(r / p.tokens);

  // token -> (frame, grid row, grid column); tokens are ordered frame-major
  const int plane = p.grid_h * p.grid_w;
  const int f = t / plane;
  const int rem = t - f * plane;
  const int y = rem / p.grid_w;
  const int x = rem - y * p.grid_w;
  const int64_t trow = p.start_frame[b] + f;

  double2 cs[kPairs];
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int j = c * kPairs + i;  // complex column inside the head
    const int64_t row = j < p.cols_t ? trow : (j < p.cols_t + p.cols_h ? y : x);
    cs[i] = __ldg(p.table + row * p.half + j);
  }

  const int64_t slot = p.dst_begin[b] + t;
  const int e0 = c * kElems;
#pragma unroll
  for (int i = 0; i < kHeadsPerThread; ++i) {
    const int h = i * hgroups + hg;
    if (h < p.heads) {
      const T* qp = static_cast<const T*>(p.q.ptr) + b * p.q.stride_row + t * p.q.stride_tok + h * p.q.stride_head + e0;
      const T* kp = static_cast<const T*>(p.k.ptr) + b * p.k.stride_row + t * p.k.stride_tok + h * p.k.stride_head + e0;
      const T* vp = static_cast<const T*>(p.v.ptr) + b * p.v.stride_row + t * p.v.stride_tok + h * p.v.stride_head + e0;
      const uint4 qv = ld_stream(qp);
      const uint4 kv = ld_stream(kp);
      const uint4 vv = ld_stream(vp);
      T* qo = static_cast<T*>(p.q_out.ptr) + b * p.q_out.stride_row + t * p.q_out.stride_tok + h * p.q_out.stride_head + e0;
      T* kc = static_cast<T*>(p.k_cache.ptr) + b * p.k_cache.stride_row + slot * p.k_cache.stride_tok + h * p.k_cache.stride_head + e0;
      T* vc = static_cast<T*>(p.v_cache.ptr) + b * p.v_cache.stride_row + slot * p.v_cache.stride_tok + h * p.v_cache.stride_head + e0;
      st_vec(qo, Vec<T>::rope(qv, cs));
      st_vec(kc, Vec<T>::rope(kv, cs));
      st_vec(vc, vv);
    }
  }
}

cudaError_t launch_rope_kv_append(const AppendParams& p, int dtype, cudaStream_t stream) {
  const int elems = dtype == SDV2_DTYPE_BF16 ? 8 : 4;
  const int vph = p.head_dim / elems;
  const int hgroups = (p.heads + kHeadsPerThread - 1) / kHeadsPerThread;
  const int64_t total = static_cast<int64_t>(p.rows) * p.tokens * hgroups * vph;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks <= 0 || blocks > 0x7FFFFFFFLL) return cudaErrorInvalidValue;
  if (dtype == SDV2_DTYPE_BF16)
    rope_kv_append_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p);
  else
    rope_kv_append_kernel<float><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace sdv2

// Fused element-wise kernels for the operations directly around the attention path of a DiT block
// (bf16 tensors, fp32 statistics).  Each replaces a chain of PyTorch element-wise launches and
// reproduces that chain's intermediate bf16 roundings, so the values handed to the projections and
// to the cache kernels are the ones the unfused chain would produce.
//
//   rmsnorm        : bf16( bf16(x * rsqrt(mean(x^2) + eps)) * w )                     per token row
//   ln_modulate    : bf16( bf16( bf16(LN(x)) * bf16(1 + scale[b, frame]) ) + shift[b, frame] )  per token row
//   gate_residual  : bf16( x + bf16(y * gate[b, frame]) )                              per element
//   layernorm_affine: bf16( w * ((x - mean) * rstd) + b )                             per token row
//   gelu_tanh      : bf16( x / (1 + exp(-2 sqrt(2/pi) (x + 0.044715 x^3))) )                per element
//   residual_layernorm: x_new = gate_residual(x, y, gate) or bf16(x + y), then either LayerNorm form of x_new
//
// All of them are pure streaming kernels (one read and one write of [tokens, dim], plus y for the
// last), bound by HBM bandwidth; 16-byte vector accesses, one token row per block for the two
// normalisations.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "sdv2_internal.h"

namespace sdv2 {

constexpr int kRowThreads = 256;
constexpr int kMaxVecPerThread = 4;  // dim <= 256 * 4 * 8 = 8192

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float lo_f(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (kRowThreads / 32) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

struct RowParams {
  const __nv_bfloat16* x;
  __nv_bfloat16* out;
  int64_t x_stride, out_stride;  // elements between token rows
  int64_t n_rows;
  int dim;
  float eps;
  const __nv_bfloat16* w;        // rmsnorm weight [dim]
  const __nv_bfloat16* scale1p;  // ln_modulate: scale, row (b * frames + f) at mod_stride elements
  const __nv_bfloat16* shift;    // ln_modulate: shift, same addressing
  int64_t mod_stride;
  int tokens_per_batch, tokens_per_frame, frames;
  // ln_rows_kernel with a residual in front: x_new = bf16(x + y) or bf16(x + bf16(y * gate[b, frame]))
  const __nv_bfloat16* res_y;
  const __nv_bfloat16* res_gate;  // row (b * frames + f) at gate_stride elements; null = plain addition
  __nv_bfloat16* res_out;         // x_new, rows of dim elements
  int64_t gate_stride;
};

template <bool kLayerNorm>
__global__ void __launch_bounds__(kRowThreads) row_norm_kernel(const __grid_constant__ RowParams p) {
  __shared__ float red[kRowThreads / 32];
  const int64_t row = blockIdx.x;
  const int n_vec = p.dim >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(p.x + row * p.x_stride);
  uint4 v[kMaxVecPerThread];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int c = threadIdx.x + i * kRowThreads;
    if (c < n_vec) {
      v[i] = xr[c];
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      if (kLayerNorm) {
#pragma unroll
        for (int j = 0; j < 4; ++j) s += lo_f(w[j]) + hi_f(w[j]);
      } else {
        ss = rms_accumulate(ss, v[i]);     // shared with the append kernel's fused q/k norm
      }
    }
  }
  float mean = 0.f, rstd;
  if (kLayerNorm) {
    mean = block_sum(s, red) / p.dim;
    // second pass over the registers for the variance: sum (x - mean)^2
    float d2 = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVecPerThread; ++i) {
      const int c = threadIdx.x + i * kRowThreads;
      if (c < n_vec) {
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = lo_f(w[j]) - mean, b = hi_f(w[j]) - mean;
          d2 += a * a + b * b;
        }
      }
    }
    rstd = rsqrtf(block_sum(d2, red) / p.dim + p.eps);
  } else {
    rstd = rms_rstd(block_sum(ss, red), p.dim, p.eps);
  }
  const uint4* mul = nullptr;
  const uint4* add = nullptr;
  if (kLayerNorm) {
    const int64_t b = row / p.tokens_per_batch;
    const int f = static_cast<int>((row - b * p.tokens_per_batch) / p.tokens_per_frame);
    const int64_t off = (b * p.frames + f) * p.mod_stride;
    mul = reinterpret_cast<const uint4*>(p.scale1p + off);
    add = reinterpret_cast<const uint4*>(p.shift + off);
  } else {
    mul = reinterpret_cast<const uint4*>(p.w);
  }
  uint4* orow = reinterpret_cast<uint4*>(p.out + row * p.out_stride);
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int c = threadIdx.x + i * kRowThreads;
    if (c < n_vec) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      const uint4 m4 = __ldg(mul + c);
      const uint32_t m[4] = {m4.x, m4.y, m4.z, m4.w};
      uint32_t a4[4] = {0, 0, 0, 0};
      if (kLayerNorm) {
        const uint4 t = __ldg(add + c);
        a4[0] = t.x; a4[1] = t.y; a4[2] = t.z; a4[3] = t.w;
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (!kLayerNorm) {
          o[j] = rms_scale_pair(w[j], rstd, m[j]);
          continue;
        }
        float lo = bf16_round((lo_f(w[j]) - mean) * rstd);
        float hi = bf16_round((hi_f(w[j]) - mean) * rstd);
        const float ml = kLayerNorm ? bf16_round(1.f + lo_f(m[j])) : lo_f(m[j]);   // (1 + scale) is a bf16 op upstream
        const float mh = kLayerNorm ? bf16_round(1.f + hi_f(m[j])) : hi_f(m[j]);
        lo = lo * ml;
        hi = hi * mh;
        if (kLayerNorm) {
          lo = bf16_round(lo) + lo_f(a4[j]);
          hi = bf16_round(hi) + hi_f(a4[j]);
        }
        o[j] = pack_bf16x2(lo, hi);
      }
      orow[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// LayerNorm with one warp per token row: the row stays in registers between the two statistics passes and
// the output pass, the reductions are shuffles only (no block barrier), and each lane has kVecPerLane
// independent 16-byte loads in flight.  kAffine = false: the adaLN modulation of ln_modulate;
// kAffine = true: out = bf16(weight * ((x - mean) * rstd) + bias) with fp32 arithmetic, the formula of
// torch.nn.LayerNorm on bf16 tensors (norm3 of the block, models/wan/causal_model.py:473-476).
constexpr int kLnWarps = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// kResidual: the row normalised is x_new = x + y (optionally y * gate first, rounded as the separate
// gate_residual kernel rounds it), and x_new is written out as well: the block's residual additions in
// front of norm3 and norm2 cost no launch and no second pass over the row.
template <int kVecPerLane, bool kAffine, bool kResidual>
__global__ void __launch_bounds__(kLnWarps * 32) ln_rows_kernel(const __grid_constant__ RowParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + (threadIdx.x >> 5);
  if (row >= p.n_rows) return;
  const int n_vec = p.dim >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(p.x + row * p.x_stride);
  uint4 v[kVecPerLane];
#pragma unroll
  for (int i = 0; i < kVecPerLane; ++i) {
    const int c = lane + i * 32;
    v[i] = c < n_vec ? xr[c] : make_uint4(0u, 0u, 0u, 0u);
  }
  const int64_t batch = row / p.tokens_per_batch;   // (unused by the affine form without a residual)
  const int frame = static_cast<int>((row - batch * p.tokens_per_batch) / p.tokens_per_frame);
  if (kResidual) {
    const uint4* yr = reinterpret_cast<const uint4*>(p.res_y + row * static_cast<int64_t>(p.dim));
    const uint4* gr = p.res_gate == nullptr ? nullptr
        : reinterpret_cast<const uint4*>(p.res_gate + (batch * p.frames + frame) * p.gate_stride);
    uint4* xo = reinterpret_cast<uint4*>(p.res_out + row * static_cast<int64_t>(p.dim));
#pragma unroll
    for (int i = 0; i < kVecPerLane; ++i) {
      const int c = lane + i * 32;
      if (c < n_vec) {
        const uint4 yv = yr[c];
        const uint32_t xw[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, yw[4] = {yv.x, yv.y, yv.z, yv.w};
        uint32_t gw[4] = {0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u};
        if (gr != nullptr) {
          const uint4 gv = __ldg(gr + c);
          gw[0] = gv.x; gw[1] = gv.y; gw[2] = gv.z; gw[3] = gv.w;
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // without a gate y is added as it is (bf16(y * 1) == y)
          const float lo = lo_f(xw[j]) + (gr != nullptr ? bf16_round(lo_f(yw[j]) * lo_f(gw[j])) : lo_f(yw[j]));
          const float hi = hi_f(xw[j]) + (gr != nullptr ? bf16_round(hi_f(yw[j]) * hi_f(gw[j])) : hi_f(yw[j]));
          o[j] = pack_bf16x2(lo, hi);
        }
        v[i] = make_uint4(o[0], o[1], o[2], o[3]);
        xo[c] = v[i];
      }
    }
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kVecPerLane; ++i) {
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) s += lo_f(w[j]) + hi_f(w[j]);
  }
  const float mean = warp_sum(s) / p.dim;
  float d2 = 0.f;
#pragma unroll
  for (int i = 0; i < kVecPerLane; ++i) {
    if (lane + i * 32 < n_vec) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = lo_f(w[j]) - mean, b = hi_f(w[j]) - mean;
        d2 += a * a + b * b;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(d2) / p.dim + p.eps);
  const uint4* mul;
  const uint4* add;
  if (kAffine) {
    mul = reinterpret_cast<const uint4*>(p.w);
    add = reinterpret_cast<const uint4*>(p.shift);
  } else {
    const int64_t off = (batch * p.frames + frame) * p.mod_stride;
    mul = reinterpret_cast<const uint4*>(p.scale1p + off);
    add = reinterpret_cast<const uint4*>(p.shift + off);
  }
  uint4* orow = reinterpret_cast<uint4*>(p.out + row * p.out_stride);
#pragma unroll
  for (int i = 0; i < kVecPerLane; ++i) {
    const int c = lane + i * 32;
    if (c < n_vec) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      const uint4 m4 = __ldg(mul + c), a4 = __ldg(add + c);
      const uint32_t m[4] = {m4.x, m4.y, m4.z, m4.w}, a[4] = {a4.x, a4.y, a4.z, a4.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float lo, hi;
        if (kAffine) {
          lo = lo_f(m[j]) * (rstd * (lo_f(w[j]) - mean)) + lo_f(a[j]);
          hi = hi_f(m[j]) * (rstd * (hi_f(w[j]) - mean)) + hi_f(a[j]);
        } else {
          lo = bf16_round(bf16_round((lo_f(w[j]) - mean) * rstd) * bf16_round(1.f + lo_f(m[j]))) + lo_f(a[j]);
          hi = bf16_round(bf16_round((hi_f(w[j]) - mean) * rstd) * bf16_round(1.f + hi_f(m[j]))) + hi_f(a[j]);
        }
        o[j] = pack_bf16x2(lo, hi);
      }
      orow[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// RMS norm with one warp per token row, for rows of at most 2048 elements.  The sum of squares is formed in
// exactly the order of row_norm_kernel (and therefore of the append kernel's fused norm): lane l holds the
// vectors l + 32 g, g = 0..7, i.e. the partial sums the 256 threads of that kernel hold one each; group g is
// reduced by the same butterfly as warp g there, and the eight group sums by the same tree.
__global__ void __launch_bounds__(kLnWarps * 32) rms_rows_kernel(const __grid_constant__ RowParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + (threadIdx.x >> 5);
  if (row >= p.n_rows) return;
  const int n_vec = p.dim >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(p.x + row * p.x_stride);
  uint4 v[8];
  float g[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + i * 32;
    v[i] = c < n_vec ? xr[c] : make_uint4(0u, 0u, 0u, 0u);
    g[i] = c < n_vec ? rms_accumulate(0.f, v[i]) : 0.f;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) g[i] = warp_sum(g[i]);
  const float rstd = rms_rstd(rms_fold_groups(g), p.dim, p.eps);
  const uint4* wv = reinterpret_cast<const uint4*>(p.w);
  uint4* orow = reinterpret_cast<uint4*>(p.out + row * p.out_stride);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + i * 32;
    if (c < n_vec) {
      const uint4 m = __ldg(wv + c);
      orow[c] = make_uint4(rms_scale_pair(v[i].x, rstd, m.x), rms_scale_pair(v[i].y, rstd, m.y),
                           rms_scale_pair(v[i].z, rstd, m.z), rms_scale_pair(v[i].w, rstd, m.w));
    }
  }
}

// Picks the instantiation whose lanes hold the whole row; false when the row is longer than any of them.
template <bool kAffine, bool kResidual>
bool launch_ln_rows(const RowParams& p, cudaStream_t stream) {
  const int per_lane = ((p.dim >> 3) + 31) / 32;
  const unsigned grid = static_cast<unsigned>((p.n_rows + kLnWarps - 1) / kLnWarps);
  if (per_lane <= 6)
    ln_rows_kernel<6, kAffine, kResidual><<<grid, kLnWarps * 32, 0, stream>>>(p);
  else if (per_lane <= 8)
    ln_rows_kernel<8, kAffine, kResidual><<<grid, kLnWarps * 32, 0, stream>>>(p);
  else if (per_lane <= 20)
    ln_rows_kernel<20, kAffine, kResidual><<<grid, kLnWarps * 32, 0, stream>>>(p);
  else
    return false;
  return true;
}

struct GateParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* y;
  const __nv_bfloat16* gate;  // row (b * frames + f) at mod_stride elements
  __nv_bfloat16* out;
  int64_t n_rows, mod_stride;
  int dim, tokens_per_batch, tokens_per_frame, frames;
};

__global__ void __launch_bounds__(256) gate_residual_kernel(const __grid_constant__ GateParams p) {
  const int n_vec = p.dim >> 3;
  const int64_t total = p.n_rows * n_vec;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / n_vec;
    const int c = static_cast<int>(i - row * n_vec);
    const int64_t b = row / p.tokens_per_batch;
    const int f = static_cast<int>((row - b * p.tokens_per_batch) / p.tokens_per_frame);
    const uint4 xv = reinterpret_cast<const uint4*>(p.x)[i];
    const uint4 yv = reinterpret_cast<const uint4*>(p.y)[i];
    const uint4 gv = __ldg(reinterpret_cast<const uint4*>(p.gate + (b * p.frames + f) * p.mod_stride) + c);
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, yw[4] = {yv.x, yv.y, yv.z, yv.w},
                   gw[4] = {gv.x, gv.y, gv.z, gv.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = lo_f(xw[j]) + bf16_round(lo_f(yw[j]) * lo_f(gw[j]));
      const float hi = hi_f(xw[j]) + bf16_round(hi_f(yw[j]) * hi_f(gw[j]));
      o[j] = pack_bf16x2(lo, hi);
    }
    reinterpret_cast<uint4*>(p.out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// tanh-approximated GELU, 0.5 x (1 + tanh(u)) with u = sqrt(2/pi) (x + 0.044715 x^3), evaluated as
// x / (1 + exp(-2u)): the same function without the cancellation in 1 + tanh(u), a handful of instructions
// per element, so the kernel streams at memory speed (the libm tanh of the op chain is compute-bound).
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * (x * x * x));
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(u * -2.8853900817779268f));  // exp(-2u)
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return x * r;
}

__global__ void __launch_bounds__(256) gelu_tanh_kernel(const uint4* __restrict__ x, uint4* __restrict__ out,
                                                        int64_t n_vec) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 v = x[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack_bf16x2(gelu_tanh(lo_f(w[j])), gelu_tanh(hi_f(w[j])));
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace sdv2

namespace {
bool a16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
}

extern "C" int sdv2_gelu_tanh(const void* x, void* out, int64_t n, void* stream) {
  if (!x || !out || n <= 0) return SDV2_ERR_INVALID_ARG;
  if (n % 8) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (!a16(x) || !a16(out)) return SDV2_ERR_MISALIGNED;
  const int64_t n_vec = n >> 3;
  int64_t blocks = (n_vec + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  sdv2::gelu_tanh_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<uint4*>(out), n_vec);
  return cudaGetLastError() == cudaSuccess ? SDV2_OK : SDV2_ERR_CUDA;
}

extern "C" int sdv2_rmsnorm(const void* x, int64_t x_row_stride, const void* weight, void* out,
                            int64_t out_row_stride, int64_t n_rows, int dim, float eps, void* stream) {
  if (!x || !weight || !out || n_rows <= 0 || dim <= 0) return SDV2_ERR_INVALID_ARG;
  if (dim % 8 || dim > sdv2::kRowThreads * sdv2::kMaxVecPerThread * 8) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (!a16(x) || !a16(weight) || !a16(out) || x_row_stride % 8 || out_row_stride % 8) return SDV2_ERR_MISALIGNED;
  if (n_rows > 0x7FFFFFFFLL) return SDV2_ERR_UNSUPPORTED_SHAPE;
  sdv2::RowParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.x_stride = x_row_stride;
  p.out_stride = out_row_stride;
  p.n_rows = n_rows;
  p.dim = dim;
  p.eps = eps;
  p.w = static_cast<const __nv_bfloat16*>(weight);
  if (dim <= 2048)
    sdv2::rms_rows_kernel<<<static_cast<unsigned>((n_rows + sdv2::kLnWarps - 1) / sdv2::kLnWarps), sdv2::kLnWarps * 32,
                            0, static_cast<cudaStream_t>(stream)>>>(p);
  else
    sdv2::row_norm_kernel<false><<<static_cast<unsigned>(n_rows), sdv2::kRowThreads, 0,
                                   static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? SDV2_OK : SDV2_ERR_CUDA;
}

extern "C" int sdv2_ln_modulate(const void* x, const void* scale1p, const void* shift, int64_t mod_row_stride,
                                void* out, int batch, int frames, int tokens_per_frame, int dim, float eps,
                                void* stream) {
  if (!x || !scale1p || !shift || !out || batch <= 0 || frames <= 0 || tokens_per_frame <= 0 || dim <= 0)
    return SDV2_ERR_INVALID_ARG;
  if (mod_row_stride < dim || mod_row_stride % 8) return SDV2_ERR_MISALIGNED;
  if (dim % 8 || dim > sdv2::kRowThreads * sdv2::kMaxVecPerThread * 8) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (!a16(x) || !a16(scale1p) || !a16(shift) || !a16(out)) return SDV2_ERR_MISALIGNED;
  const int64_t n_rows = static_cast<int64_t>(batch) * frames * tokens_per_frame;
  if (n_rows > 0x7FFFFFFFLL) return SDV2_ERR_UNSUPPORTED_SHAPE;
  sdv2::RowParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.x_stride = p.out_stride = dim;
  p.n_rows = n_rows;
  p.dim = dim;
  p.eps = eps;
  p.scale1p = static_cast<const __nv_bfloat16*>(scale1p);
  p.shift = static_cast<const __nv_bfloat16*>(shift);
  p.mod_stride = mod_row_stride;
  p.frames = frames;
  p.tokens_per_frame = tokens_per_frame;
  p.tokens_per_batch = frames * tokens_per_frame;
  if (!sdv2::launch_ln_rows<false, false>(p, static_cast<cudaStream_t>(stream)))  // rows of more than 5120 elements
    sdv2::row_norm_kernel<true><<<static_cast<unsigned>(n_rows), sdv2::kRowThreads, 0,
                                  static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? SDV2_OK : SDV2_ERR_CUDA;
}

extern "C" int sdv2_layernorm_affine(const void* x, const void* weight, const void* bias, void* out, int64_t n_rows,
                                     int dim, float eps, void* stream) {
  if (!x || !weight || !bias || !out || n_rows <= 0 || dim <= 0) return SDV2_ERR_INVALID_ARG;
  if (dim % 8 || dim > 5120 || n_rows > 0x7FFFFFFFLL) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (!a16(x) || !a16(weight) || !a16(bias) || !a16(out)) return SDV2_ERR_MISALIGNED;
  sdv2::RowParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.x_stride = p.out_stride = dim;
  p.n_rows = n_rows;
  p.dim = dim;
  p.eps = eps;
  p.w = static_cast<const __nv_bfloat16*>(weight);
  p.shift = static_cast<const __nv_bfloat16*>(bias);
  p.frames = 1;
  p.tokens_per_frame = p.tokens_per_batch = static_cast<int>(n_rows);
  if (!sdv2::launch_ln_rows<true, false>(p, static_cast<cudaStream_t>(stream))) return SDV2_ERR_UNSUPPORTED_SHAPE;
  return cudaGetLastError() == cudaSuccess ? SDV2_OK : SDV2_ERR_CUDA;
}

extern "C" int sdv2_residual_layernorm(const void* x, const void* y, const void* gate, int64_t gate_row_stride,
                                       void* x_out, int affine, const void* mul, const void* add,
                                       int64_t mod_row_stride, void* out, int batch, int frames,
                                       int tokens_per_frame, int dim, float eps, void* stream) {
  if (!x || !y || !x_out || !mul || !add || !out || batch <= 0 || frames <= 0 || tokens_per_frame <= 0 || dim <= 0)
    return SDV2_ERR_INVALID_ARG;
  if (dim % 8 || dim > 5120) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (!a16(x) || !a16(y) || !a16(x_out) || !a16(mul) || !a16(add) || !a16(out) || (gate && !a16(gate)))
    return SDV2_ERR_MISALIGNED;
  if (gate && (gate_row_stride < dim || gate_row_stride % 8)) return SDV2_ERR_MISALIGNED;
  if (!affine && (mod_row_stride < dim || mod_row_stride % 8)) return SDV2_ERR_MISALIGNED;
  const int64_t n_rows = static_cast<int64_t>(batch) * frames * tokens_per_frame;
  if (n_rows > 0x7FFFFFFFLL) return SDV2_ERR_UNSUPPORTED_SHAPE;
  sdv2::RowParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.x_stride = p.out_stride = dim;
  p.n_rows = n_rows;
  p.dim = dim;
  p.eps = eps;
  if (affine) {
    p.w = static_cast<const __nv_bfloat16*>(mul);
  } else {
    p.scale1p = static_cast<const __nv_bfloat16*>(mul);
    p.mod_stride = mod_row_stride;
  }
  p.shift = static_cast<const __nv_bfloat16*>(add);
  p.frames = frames;
  p.tokens_per_frame = tokens_per_frame;
  p.tokens_per_batch = frames * tokens_per_frame;
  p.res_y = static_cast<const __nv_bfloat16*>(y);
  p.res_gate = static_cast<const __nv_bfloat16*>(gate);
  p.res_out = static_cast<__nv_bfloat16*>(x_out);
  p.gate_stride = gate_row_stride;
  const bool ok = affine ? sdv2::launch_ln_rows<true, true>(p, static_cast<cudaStream_t>(stream))
                         : sdv2::launch_ln_rows<false, true>(p, static_cast<cudaStream_t>(stream));
  if (!ok) return SDV2_ERR_UNSUPPORTED_SHAPE;
  return cudaGetLastError() == cudaSuccess ? SDV2_OK : SDV2_ERR_CUDA;
}

extern "C" int sdv2_gate_residual(const void* x, const void* y, const void* gate, int64_t mod_row_stride, void* out,
                                  int batch, int frames, int tokens_per_frame, int dim, void* stream) {
  if (!x || !y || !gate || !out || batch <= 0 || frames <= 0 || tokens_per_frame <= 0 || dim <= 0)
    return SDV2_ERR_INVALID_ARG;
  if (mod_row_stride < dim || mod_row_stride % 8) return SDV2_ERR_MISALIGNED;
  if (dim % 8) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (!a16(x) || !a16(y) || !a16(gate) || !a16(out)) return SDV2_ERR_MISALIGNED;
  sdv2::GateParams p = {};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.y = static_cast<const __nv_bfloat16*>(y);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.n_rows = static_cast<int64_t>(batch) * frames * tokens_per_frame;
  p.mod_stride = mod_row_stride;
  p.dim = dim;
  p.frames = frames;
  p.tokens_per_frame = tokens_per_frame;
  p.tokens_per_batch = frames * tokens_per_frame;
  const int64_t total = p.n_rows * (dim >> 3);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  sdv2::gate_residual_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? SDV2_OK : SDV2_ERR_CUDA;
}

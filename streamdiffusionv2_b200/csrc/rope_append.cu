// Fused 3D rotary embedding + K/V slot write for the sink + ring-buffer cache.
//
// Pure streaming work (3 reads + 3 writes of [rows, tokens, heads, head_dim]); bound by HBM.
//
// Staged kernel (the default): persistent CTAs, one per SM.  A producer warp streams whole token
// rows of q, k and v into a ring of shared-memory stages with bulk asynchronous copies
// (cp.async.bulk, completion counted on an mbarrier), so memory latency is hidden by the copy
// engine instead of by registers; 16 consumer warps rope q and k out of shared memory in fp64
// and write q_out / K slot / V slot with 16-byte coalesced stores.  Tokens are split evenly
// over the CTAs (to within one token).
//
// Direct kernel: one thread per 16-byte vector straight from global memory; used when a token
// row is not one contiguous run of heads or is too large for a stage.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "sdv2_internal.h"

namespace sdv2 {

// ------------------------------------------------------------------------------------------
// arithmetic shared by both kernels
// ------------------------------------------------------------------------------------------

// True when one of the two bf16 in `w` has an all-zero or all-one exponent (zero, subnormal,
// inf, nan): those take the hardware conversion instead of the integer rebuild below.
__device__ __forceinline__ uint32_t bf16x2_special(uint32_t w) {
  // (exp + 1) & 0xFE == 0  <=>  exp in {0, 255}; then the classic zero-halfword test
  const uint32_t v = ((w & 0x7F807F80u) + 0x00800080u) & 0x7F007F00u;
  return (v - 0x00010001u) & ~v & 0x80008000u;
}
// bf16 (normal) in the low / high half of w -> double, exactly, with integer ops only.
__device__ __forceinline__ double bf16lo_to_f64_normal(uint32_t w) {
  const uint32_t hi = ((((w << 13) & 0x0FFFE000u) + 0x38000000u)) | ((w << 16) & 0x80000000u);
  return __hiloint2double(static_cast<int>(hi), 0);
}
__device__ __forceinline__ double bf16hi_to_f64_normal(uint32_t w) {
  const uint32_t hi = ((((w >> 3) & 0x0FFFE000u) + 0x38000000u)) | (w & 0x80000000u);
  return __hiloint2double(static_cast<int>(hi), 0);
}

// (a + ib) * (c + id) with every product and sum rounded separately, as the reference's CPU
// complex128 multiply does; then fp64 -> fp32 (RN).  bf16 storage adds a second RNE step.
__device__ __forceinline__ void rope_pair(double a, double b, double2 cs, float& re, float& im) {
  re = __double2float_rn(__dsub_rn(__dmul_rn(a, cs.x), __dmul_rn(b, cs.y)));
  im = __double2float_rn(__dadd_rn(__dmul_rn(a, cs.y), __dmul_rn(b, cs.x)));
}

template <typename T>
struct Vec;  // one 16-byte vector of T

template <>
struct Vec<__nv_bfloat16> {
  static constexpr int kPairs = 4;
  __device__ __forceinline__ static uint4 rope(uint4 x, const double2 (&cs)[4]) {
    uint32_t w[4] = {x.x, x.y, x.z, x.w};
    const uint32_t special = bf16x2_special(w[0]) | bf16x2_special(w[1]) | bf16x2_special(w[2]) | bf16x2_special(w[3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      double a, b;
      if (special == 0) {
        a = bf16lo_to_f64_normal(w[i]);
        b = bf16hi_to_f64_normal(w[i]);
      } else {
        a = static_cast<double>(__uint_as_float(w[i] << 16));
        b = static_cast<double>(__uint_as_float(w[i] & 0xFFFF0000u));
      }
      float re, im;
      rope_pair(a, b, cs[i], re, im);
      w[i] = pack_bf16x2(re, im);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <>
struct Vec<float> {
  static constexpr int kPairs = 2;
  __device__ __forceinline__ static uint4 rope(uint4 x, const double2 (&cs)[2]) {
    float re0, im0, re1, im1;
    rope_pair(static_cast<double>(__uint_as_float(x.x)), static_cast<double>(__uint_as_float(x.y)), cs[0],
              re0, im0);
    rope_pair(static_cast<double>(__uint_as_float(x.z)), static_cast<double>(__uint_as_float(x.w)), cs[1],
              re1, im1);
    return make_uint4(__float_as_uint(re0), __float_as_uint(im0), __float_as_uint(re1), __float_as_uint(im1));
  }
};

// n / d for n * d < 2^32 with m = ceil(2^32 / d)
__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint32_t m) { return __umulhi(n, m); }

// rope multipliers of vector column c of a token at (table row for time, grid row, grid column)
template <int kPairs>
__device__ __forceinline__ void load_cs(const AppendParams& p, int c, int64_t trow, int y, int x,
                                        double2 (&cs)[kPairs]) {
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int j = c * kPairs + i;  // complex column inside the head
    const int64_t row = j < p.cols_t ? trow : (j < p.cols_t + p.cols_h ? y : x);
    cs[i] = __ldg(p.table + row * p.half + j);
  }
}

__device__ __forceinline__ void write_index(const AppendParams& p) {
  if (p.global_end_dev != nullptr) {
    for (int b = 0; b < p.rows; ++b) {
      p.global_end_dev[b] = p.global_end_val[b];
      p.local_end_dev[b] = p.local_end_val[b];
    }
  }
}

// ------------------------------------------------------------------------------------------
// direct kernel: grid (token blocks, heads, rows), 256 threads = (256 / vph) tokens x vph vectors
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) rope_kv_append_direct_kernel(const __grid_constant__ AppendParams p) {
  constexpr int kPairs = Vec<T>::kPairs;
  constexpr int kElems = 2 * kPairs;
  const int vph = p.head_dim / kElems;
  const int tok_per_block = 256 / vph;
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) write_index(p);
  const int tl = fast_div(threadIdx.x, p.magic_vph);
  const int c = threadIdx.x - tl * vph;
  const int t = blockIdx.x * tok_per_block + tl;
  if (tl >= tok_per_block || t >= p.tokens) return;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int f = fast_div(t, p.magic_plane);
  const int rem = t - f * p.plane;
  const int y = fast_div(rem, p.magic_w);
  const int x = rem - y * p.grid_w;
  double2 cs[kPairs];
  load_cs<kPairs>(p, c, p.start_frame[b] + f, y, x, cs);
  const int64_t slot = p.dst_begin[b] + t;
  const int e0 = c * kElems;
  const T* qp = static_cast<const T*>(p.q.ptr) + b * p.q.stride_row + t * p.q.stride_tok + h * p.q.stride_head + e0;
  const T* kp = static_cast<const T*>(p.k.ptr) + b * p.k.stride_row + t * p.k.stride_tok + h * p.k.stride_head + e0;
  const T* vp = static_cast<const T*>(p.v.ptr) + b * p.v.stride_row + t * p.v.stride_tok + h * p.v.stride_head + e0;
  const uint4 qv = *reinterpret_cast<const uint4*>(qp);
  const uint4 kv = *reinterpret_cast<const uint4*>(kp);
  const uint4 vv = *reinterpret_cast<const uint4*>(vp);
  T* qo = static_cast<T*>(p.q_out.ptr) + b * p.q_out.stride_row + t * p.q_out.stride_tok + h * p.q_out.stride_head + e0;
  T* kc = static_cast<T*>(p.k_cache.ptr) + b * p.k_cache.stride_row + slot * p.k_cache.stride_tok + h * p.k_cache.stride_head + e0;
  T* vc = static_cast<T*>(p.v_cache.ptr) + b * p.v_cache.stride_row + slot * p.v_cache.stride_tok + h * p.v_cache.stride_head + e0;
  *reinterpret_cast<uint4*>(qo) = Vec<T>::rope(qv, cs);
  *reinterpret_cast<uint4*>(kc) = Vec<T>::rope(kv, cs);
  *reinterpret_cast<uint4*>(vc) = vv;
}

// ------------------------------------------------------------------------------------------
// staged kernel
// ------------------------------------------------------------------------------------------
namespace staged {
constexpr int kStages = 3;
constexpr int kConsumerWarps = 16;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;            // + producer warp
constexpr uint32_t kStageBytes = 72 * 1024;          // q | k | v token rows of one tile
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 128 + 128;  // + barriers + alignment slack
constexpr int kMaxTileTokens = 8;
}  // namespace staged

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

template <typename T>
__global__ void __launch_bounds__(staged::kThreads, 1)
rope_kv_append_staged_kernel(const __grid_constant__ AppendParams p) {
  using namespace staged;
  constexpr int kPairs = Vec<T>::kPairs;
  constexpr int kElems = 2 * kPairs;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + kStages * kStageBytes;  // full[kStages], empty[kStages]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + kStages * kStageBytes + 64);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar0 + 8 * s, 1);
      mbar_init(bar0 + 8 * (kStages + s), kConsumerWarps);
    }
    fence_mbar_init();
    if (blockIdx.x == 0) write_index(p);
  }
  __syncthreads();

  // this CTA's contiguous range of (row, token) pairs
  const int64_t total = static_cast<int64_t>(p.rows) * p.tokens;
  const int lo = static_cast<int>(total * blockIdx.x / gridDim.x);
  const int hi = static_cast<int>(total * (blockIdx.x + 1) / gridDim.x);
  const uint32_t row_bytes = static_cast<uint32_t>(p.heads) * p.head_dim * sizeof(T);
  const int tile_tokens = p.tile_tokens;
  const uint32_t tensor_stride = tile_tokens * row_bytes;  // q | k | v blocks inside a stage

  if (warp == kConsumerWarps) {
    // ---------------------------------------------------------------- producer
    int cur = lo, i = 0;
    bool ok = true;
    while (cur < hi && ok) {
      const int b = cur / p.tokens;
      const int t0 = cur - b * p.tokens;
      const int n = min(min(tile_tokens, hi - cur), p.tokens - t0);
      const int s = i % kStages;
      if (i >= kStages) {
        ok = mbar_wait(bar0 + 8 * (kStages + s), ((i / kStages) - 1) & 1, abort_flag, p.status, WAIT_TILE_FREE);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (lane == 0) mbar_expect_tx(bar0 + 8 * s, 3u * n * row_bytes);
      __syncwarp();
      const uint32_t sbase = base + s * kStageBytes;
      for (int c = lane; c < 3 * n; c += 32) {
        const int which = c / n;  // 0 q, 1 k, 2 v
        const int j = c - which * n;
        const sdv2_view& vw = which == 0 ? p.q : (which == 1 ? p.k : p.v);
        const T* src = static_cast<const T*>(vw.ptr) + b * vw.stride_row + static_cast<int64_t>(t0 + j) * vw.stride_tok;
        bulk_load(sbase + which * tensor_stride + j * row_bytes, src, row_bytes, bar0 + 8 * s);
      }
      cur += n;
      ++i;
    }
    if (!ok && lane == 0) {
      // leave no copy in flight: bounded wait for the stages already requested
      for (int k = (i > kStages ? i - kStages : 0); k < i; ++k) {
        const long long t0c = clock64();
        while (!mbar_try_wait(bar0 + 8 * (k % kStages), (k / kStages) & 1) && clock64() - t0c < kWaitBudgetCycles) {
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers
    const int vph = p.head_dim / kElems;
    const int row_vecs = p.heads * vph;
    int cur = lo, i = 0;
    while (cur < hi) {
      const int b = cur / p.tokens;
      const int t0 = cur - b * p.tokens;
      const int n = min(min(tile_tokens, hi - cur), p.tokens - t0);
      const int s = i % kStages;
      bool ok = mbar_wait(bar0 + 8 * s, (i / kStages) & 1, abort_flag, p.status, WAIT_KV_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint8_t* sq = gbase + s * kStageBytes;
      const int n_vec = n * row_vecs;
      for (int v = threadIdx.x; v < n_vec; v += kConsumers) {
        const int j = fast_div(v, p.magic_row_vecs);  // token inside the tile
        const int rv = v - j * row_vecs;               // vector inside the token row
        const int h = fast_div(rv, p.magic_vph);
        const int c = rv - h * vph;
        const int t = t0 + j;
        const int f = fast_div(t, p.magic_plane);
        const int rem = t - f * p.plane;
        const int y = fast_div(rem, p.magic_w);
        const int x = rem - y * p.grid_w;
        double2 cs[kPairs];
        load_cs<kPairs>(p, c, p.start_frame[b] + f, y, x, cs);
        const uint32_t off = static_cast<uint32_t>(j) * row_bytes + static_cast<uint32_t>(rv) * 16u;
        const uint4 qv = *reinterpret_cast<const uint4*>(sq + off);
        const uint4 kv = *reinterpret_cast<const uint4*>(sq + tensor_stride + off);
        const uint4 vv = *reinterpret_cast<const uint4*>(sq + 2 * tensor_stride + off);
        const int64_t slot = p.dst_begin[b] + t;
        const int e0 = c * kElems;
        T* qo = static_cast<T*>(p.q_out.ptr) + b * p.q_out.stride_row + t * p.q_out.stride_tok + h * p.q_out.stride_head + e0;
        T* kc = static_cast<T*>(p.k_cache.ptr) + b * p.k_cache.stride_row + slot * p.k_cache.stride_tok + h * p.k_cache.stride_head + e0;
        T* vc = static_cast<T*>(p.v_cache.ptr) + b * p.v_cache.stride_row + slot * p.v_cache.stride_tok + h * p.v_cache.stride_head + e0;
        *reinterpret_cast<uint4*>(vc) = vv;
        *reinterpret_cast<uint4*>(qo) = Vec<T>::rope(qv, cs);
        *reinterpret_cast<uint4*>(kc) = Vec<T>::rope(kv, cs);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar0 + 8 * (kStages + s));
      cur += n;
      ++i;
    }
  }
}

static uint32_t magic_of(uint32_t d) { return static_cast<uint32_t>(((1ull << 32) + d - 1) / d); }

cudaError_t launch_rope_kv_append(const AppendParams& p_in, int dtype, cudaStream_t stream) {
  AppendParams p = p_in;
  const int esize = dtype == SDV2_DTYPE_BF16 ? 2 : 4;
  const int elems = 16 / esize;
  const int vph = p.head_dim / elems;
  p.plane = p.grid_h * p.grid_w;
  p.magic_plane = magic_of(p.plane);
  p.magic_w = magic_of(p.grid_w);
  const int row_vecs = p.heads * vph;
  p.magic_row_vecs = magic_of(row_vecs);
  p.magic_vph = magic_of(vph);
  const uint32_t row_bytes = static_cast<uint32_t>(p.heads) * p.head_dim * esize;
  // fast_div is exact while numerator * divisor < 2^32
  const bool div_ok = static_cast<uint64_t>(p.tokens) * p.plane < (1ull << 32) &&
                      static_cast<uint64_t>(staged::kMaxTileTokens) * row_vecs * row_vecs < (1ull << 32);
  if (!div_ok || vph > 256) return cudaErrorInvalidValue;
  const bool rows_contiguous = p.q.stride_head == p.head_dim && p.k.stride_head == p.head_dim &&
                               p.v.stride_head == p.head_dim;
  int tile_tokens = static_cast<int>(staged::kStageBytes / (3u * row_bytes));
  if (tile_tokens > staged::kMaxTileTokens) tile_tokens = staged::kMaxTileTokens;
  if (rows_contiguous && tile_tokens >= 1) {
    p.tile_tokens = tile_tokens;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    const int64_t total = static_cast<int64_t>(p.rows) * p.tokens;
    const int grid = static_cast<int>(total < sms ? total : sms);
    if (dtype == SDV2_DTYPE_BF16) {
      e = cudaFuncSetAttribute(rope_kv_append_staged_kernel<__nv_bfloat16>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(staged::kSmemBytes));
      if (e != cudaSuccess) return e;
      rope_kv_append_staged_kernel<__nv_bfloat16><<<grid, staged::kThreads, staged::kSmemBytes, stream>>>(p);
    } else {
      e = cudaFuncSetAttribute(rope_kv_append_staged_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(staged::kSmemBytes));
      if (e != cudaSuccess) return e;
      rope_kv_append_staged_kernel<float><<<grid, staged::kThreads, staged::kSmemBytes, stream>>>(p);
    }
    return cudaGetLastError();
  }
  const int tok_per_block = 256 / vph;
  dim3 grid((p.tokens + tok_per_block - 1) / tok_per_block, p.heads, p.rows);
  if (dtype == SDV2_DTYPE_BF16)
    rope_kv_append_direct_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else
    rope_kv_append_direct_kernel<float><<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace sdv2

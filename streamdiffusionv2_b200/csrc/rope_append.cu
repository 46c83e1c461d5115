// Fused 3D rotary embedding + K/V slot write for the sink + ring-buffer cache.
//
// Pure streaming work (3 reads + 3 writes of [rows, tokens, heads, head_dim]); bound by HBM.
//
// Staged kernel (the default): persistent CTAs, one per SM.  A producer warp streams whole token
// rows of q, k and v into a ring of shared-memory stages with bulk asynchronous copies
// (cp.async.bulk, completion counted on an mbarrier), so memory latency is hidden by the copy
// engine instead of by registers, and builds each tile's per-token rope multiplier rows next to
// them.  The consumer warps rope q and k out of shared memory in fp64 and write q_out / K slot /
// V slot with 16-byte coalesced stores.  Tokens are split evenly over the CTAs (to within one).
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

// (a + ib) * (c + id) with every product and sum rounded separately, as the reference's CPU
// complex128 multiply does; then fp64 -> fp32 (RN).  bf16 storage adds a second RNE step.
__device__ __forceinline__ void rope_pair(double a, double b, double2 cs, float& re, float& im) {
  re = __double2float_rn(__dsub_rn(__dmul_rn(a, cs.x), __dmul_rn(b, cs.y)));
  im = __double2float_rn(__dadd_rn(__dmul_rn(a, cs.y), __dmul_rn(b, cs.x)));
}

template <typename T>
struct Vec;  // one 16-byte vector of T

// bf16 -> fp32 is a 16-bit shift; fp32 -> fp64 uses the hardware conversion, which is exact for
// every input class (zeros, subnormals, infinities, NaNs).  Rebuilding the double with integer
// ops was measured slower: it costs ~3x the issue slots and needs a special-value test.
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int kPairs = 4;
  __device__ __forceinline__ static uint4 rope(uint4 x, const double2 (&cs)[4]) {
    uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float re, im;
      rope_pair(static_cast<double>(__uint_as_float(w[i] << 16)),
                static_cast<double>(__uint_as_float(w[i] & 0xFFFF0000u)), cs[i], re, im);
      w[i] = pack_bf16x2(re, im);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  // RMS-normalise first (bf16(bf16(x * rstd) * weight), the roundings of the unfused norm), then rope
  __device__ __forceinline__ static uint4 rope_normed(uint4 x, const double2 (&cs)[4], float rstd, uint4 wv) {
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    return rope(make_uint4(rms_scale_pair(x.x, rstd, ww[0]), rms_scale_pair(x.y, rstd, ww[1]),
                           rms_scale_pair(x.z, rstd, ww[2]), rms_scale_pair(x.w, rstd, ww[3])), cs);
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
  __device__ __forceinline__ static uint4 rope_normed(uint4 x, const double2 (&cs)[2], float, uint4) {
    return rope(x, cs);  // the fused norm exists for bf16 only; the launcher never asks for it here
  }
};

// n / d for n * d < 2^32 with m = ceil(2^32 / d)
__device__ __forceinline__ int fast_div(uint32_t n, uint32_t m) { return static_cast<int>(__umulhi(n, m)); }

// table entry for complex column `col` of a token at (time row, grid row y, grid column x)
__device__ __forceinline__ double2 table_entry(const AppendParams& p, int col, int64_t trow, int y, int x) {
  const int64_t row = col < p.cols_t ? trow : (col < p.cols_t + p.cols_h ? y : x);
  return __ldg(p.table + row * p.half + col);
}

// Per-row slot parameters come from the launch parameters or, for launches that must not carry
// per-step values (a captured graph), from a device array the host refreshes between steps.
__device__ __forceinline__ int64_t row_start_frame(const AppendParams& p, int b) {
  return p.step_dev != nullptr ? p.step_dev[b] : p.start_frame[b];
}
__device__ __forceinline__ int64_t row_dst_begin(const AppendParams& p, int b) {
  return p.step_dev != nullptr ? p.step_dev[p.rows + b] : p.dst_begin[b];
}

// Device-resident parameters cannot be validated by the host: every thread checks them (the same
// few cached loads) and the whole launch writes nothing when a slot would leave the cache or a
// frame the rope table.  Block 0 records that in the status word.
__device__ __forceinline__ bool step_params_ok(const AppendParams& p) {
  if (p.step_dev == nullptr) return true;
  bool ok = true;
  for (int b = 0; b < p.rows; ++b) {
    const int64_t f = p.step_dev[b], d = p.step_dev[p.rows + b];
    ok = ok && f >= 0 && f + p.grid_f <= p.table_rows && d >= 0 && d + p.tokens <= p.cache_tokens;
  }
  return ok;
}

__device__ __forceinline__ void write_index(const AppendParams& p) {
  if (p.global_end_dev != nullptr) {
    for (int b = 0; b < p.rows; ++b) {
      p.global_end_dev[b] = p.step_dev != nullptr ? p.step_dev[2 * p.rows + b] : p.global_end_val[b];
      p.local_end_dev[b] = p.step_dev != nullptr ? p.step_dev[3 * p.rows + b] : p.local_end_val[b];
    }
  }
}

__device__ __forceinline__ void report_bad_step_params(const AppendParams& p) {
  if (p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(BAD_STEP_PARAMS));
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
  const bool first = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0;
  if (!step_params_ok(p)) {
    if (first) report_bad_step_params(p);
    return;
  }
  if (first) write_index(p);
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
#pragma unroll
  for (int i = 0; i < kPairs; ++i) cs[i] = table_entry(p, c * kPairs + i, row_start_frame(p, b) + f, y, x);
  const int64_t slot = row_dst_begin(p, b) + t;
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
constexpr int kMaxStages = 8;
constexpr int kStagesWanted = 3;             // larger tiles beat more stages: per-tile handshakes cost
constexpr int kMaxConsumerWarps = 20;
constexpr int kProducerWarps = 3;            // warp 0 of the group also issues the bulk copies
constexpr int kMinConsumerWarps = 12;
constexpr int kMaxTileTokens = 8;
constexpr int kMultBatch = 4;                // table loads in flight per producer lane
constexpr uint32_t kSmemLimit = 220 * 1024;  // stages + barriers; the rest stays L1
constexpr uint32_t kTailBytes = 512;         // barriers, abort flag, alignment slack
}  // namespace staged

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Stage layout: q rows | k rows | v rows (tile_tokens x row_bytes each) | multiplier rows
// (tile_tokens x half complex doubles) | with kNorm: 1 / rms of every q row, then of every k row, then the
// 8 group sums of every row from which they are folded.  The producer group (the last warps) issues the bulk copies
// of a tile and builds the tile's multiplier rows from the rope table; each of its warps then
// arrives on the stage's "full" barrier, which completes once the copied bytes are in as well.
// Barrier over `threads` threads (a multiple of 32) that also ANDs a flag over them.
__device__ __forceinline__ bool named_barrier_and(int id, int threads, bool flag) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %3, 0;\n\t"
      "bar.red.and.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(threads), "r"(static_cast<uint32_t>(flag))
      : "memory");
  return r != 0;
}

template <typename T, bool kNorm>
__global__ void __launch_bounds__((staged::kMaxConsumerWarps + staged::kProducerWarps) * 32, 1)
rope_kv_append_staged_kernel(const __grid_constant__ AppendParams p) {
  using namespace staged;
  constexpr int kPairs = Vec<T>::kPairs;
  constexpr int kElems = 2 * kPairs;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  uint8_t* gbase = smem_raw + (base - raw);
  const int consumer_warps = (blockDim.x >> 5) - kProducerWarps;
  const int consumers = consumer_warps * 32;
  const uint32_t row_bytes = static_cast<uint32_t>(p.heads) * p.head_dim * sizeof(T);
  const int tile_tokens = p.tile_tokens;
  const uint32_t tensor_stride = tile_tokens * row_bytes;
  const uint32_t mult_off = 3 * tensor_stride;
  const uint32_t mult_row_bytes = static_cast<uint32_t>(p.half) * 16u;
  const uint32_t stage_bytes = p.stage_bytes;
  const int kStages = p.stages;
  const uint32_t bar0 = base + kStages * stage_bytes;  // full[stages], empty[stages]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + kStages * stage_bytes + 16 * kMaxStages);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (!step_params_ok(p)) {  // uniform over the grid: no barrier was touched, no copy issued
    if (blockIdx.x == 0 && threadIdx.x == 0) report_bad_step_params(p);
    return;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar0 + 8 * s, kProducerWarps);
      mbar_init(bar0 + 8 * (kStages + s), consumer_warps);
    }
    fence_mbar_init();
    if (blockIdx.x == 0) write_index(p);
  }
  __syncthreads();

  // this CTA's contiguous range of (row, token) pairs
  const int64_t total = static_cast<int64_t>(p.rows) * p.tokens;
  const int lo = static_cast<int>(total * blockIdx.x / gridDim.x);
  const int hi = static_cast<int>(total * (blockIdx.x + 1) / gridDim.x);

  if (warp >= consumer_warps) {
    // ---------------------------------------------------------------- producer group
    const int pw = warp - consumer_warps;                 // 0 issues the copies
    const int plane_id = pw * 32 + lane;                  // lane inside the group
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
      const uint32_t sbase = base + s * stage_bytes;
      for (int c = lane; pw == 0 && c < 3 * n; c += 32) {
        const int which = c / n;  // 0 q, 1 k, 2 v
        const int j = c - which * n;
        const sdv2_view& vw = which == 0 ? p.q : (which == 1 ? p.k : p.v);
        const T* src = static_cast<const T*>(vw.ptr) + b * vw.stride_row + static_cast<int64_t>(t0 + j) * vw.stride_tok;
        bulk_load(sbase + which * tensor_stride + j * row_bytes, src, row_bytes, bar0 + 8 * s);
      }
      double2* mult = reinterpret_cast<double2*>(gbase + s * stage_bytes + mult_off);
      const int64_t frame0 = row_start_frame(p, b);
      const int n_ent = n * p.half;
      for (int e0 = plane_id; e0 < n_ent; e0 += kProducerWarps * 32 * kMultBatch) {
        double2 val[kMultBatch];  // all loads of a batch in flight before the first store
#pragma unroll
        for (int u = 0; u < kMultBatch; ++u) {
          const int e = e0 + kProducerWarps * 32 * u;
          if (e < n_ent) {
            const int j = fast_div(e, p.magic_half);
            const int col = e - j * p.half;
            const int t = t0 + j;
            const int f = fast_div(t, p.magic_plane);
            const int rem = t - f * p.plane;
            const int y = fast_div(rem, p.magic_w);
            val[u] = table_entry(p, col, frame0 + f, y, rem - y * p.grid_w);
          }
        }
#pragma unroll
        for (int u = 0; u < kMultBatch; ++u)
          if (e0 + kProducerWarps * 32 * u < n_ent) mult[e0 + kProducerWarps * 32 * u] = val[u];
      }
      __syncwarp();
      // one arrival per producer warp; the phase completes when the copied bytes are in as well
      if (lane == 0) {
        if (pw == 0) mbar_expect_tx(bar0 + 8 * s, 3u * n * row_bytes);
        else mbar_arrive(bar0 + 8 * s);
      }
      cur += n;
      ++i;
    }
    if (!ok && lane == 0 && pw == 0) {
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
      if (!kNorm && !ok) break;
      const uint8_t* sq = gbase + s * stage_bytes;
      const float* rstd_s = reinterpret_cast<const float*>(sq + mult_off + tile_tokens * mult_row_bytes);
      if (kNorm) {
        // 1 / rms of every staged q and k row, summed in the order sdv2_rmsnorm uses.  Pass 1, all consumer
        // threads: a task is one of the norm kernel's 256 "thread slots" of one row (vectors slot, slot + 256,
        // ... chained); 32 consecutive slots sit in one warp and are folded with the xor butterfly into one
        // group sum.  Pass 2, one thread per row: the 8 group sums through the fixed tree, then 1 / rms.
        float* rstd_w = const_cast<float*>(rstd_s);
        float* gsum = rstd_w + 2 * tile_tokens;                        // [2 * tile_tokens][8]
        const int slots = min(256, (row_vecs + 31) & ~31);             // slots that hold at least one vector, per warp
        if (ok) {
          for (int task = threadIdx.x; task < 2 * n * slots; task += consumers) {
            const int r = task / slots;                                // row: q rows first, then k rows
            const int t = task - r * slots;
            const int which = r >= n ? 1 : 0;
            const uint8_t* rowp = sq + which * tensor_stride + (r - which * n) * row_bytes;
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int c = t + i * 256;
              if (c < row_vecs) ss = rms_accumulate(ss, *reinterpret_cast<const uint4*>(rowp + c * 16));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) gsum[r * 8 + (t >> 5)] = ss;
          }
        }
        ok = named_barrier_and(1, consumers, ok);   // consumers only; the producer group never joins
        if (ok && threadIdx.x < 2 * n) {
          float g[8];
#pragma unroll
          for (int w = 0; w < 8; ++w) g[w] = w * 32 < slots ? gsum[threadIdx.x * 8 + w] : 0.f;
          rstd_w[threadIdx.x] = rms_rstd(rms_fold_groups(g), p.heads * p.head_dim, p.norm_eps);
        }
        // a warp whose wait was abandoned still arrives, and everybody leaves together
        ok = named_barrier_and(1, consumers, ok);
        if (!ok) break;
      }
      const int n_vec = n * row_vecs;
      const int64_t slot0 = row_dst_begin(p, b) + t0;
      T* qo_base = static_cast<T*>(p.q_out.ptr) + b * p.q_out.stride_row + t0 * p.q_out.stride_tok;
      T* kc_base = static_cast<T*>(p.k_cache.ptr) + b * p.k_cache.stride_row + slot0 * p.k_cache.stride_tok;
      T* vc_base = static_cast<T*>(p.v_cache.ptr) + b * p.v_cache.stride_row + slot0 * p.v_cache.stride_tok;
      for (int v = threadIdx.x; v < n_vec; v += consumers) {
        const int j = fast_div(v, p.magic_row_vecs);  // token inside the tile
        const int rv = v - j * row_vecs;               // vector inside the token row
        const int h = fast_div(rv, p.magic_vph);
        const int c = rv - h * vph;
        const double2* mrow = reinterpret_cast<const double2*>(sq + mult_off + j * mult_row_bytes) + c * kPairs;
        double2 cs[kPairs];
#pragma unroll
        for (int q = 0; q < kPairs; ++q) cs[q] = mrow[q];
        const uint32_t off = static_cast<uint32_t>(j) * row_bytes + static_cast<uint32_t>(rv) * 16u;
        const uint4 qv = *reinterpret_cast<const uint4*>(sq + off);
        const uint4 kv = *reinterpret_cast<const uint4*>(sq + tensor_stride + off);
        const uint4 vv = *reinterpret_cast<const uint4*>(sq + 2 * tensor_stride + off);
        const int e0 = c * kElems;
        *reinterpret_cast<uint4*>(vc_base + j * p.v_cache.stride_tok + h * p.v_cache.stride_head + e0) = vv;
        uint4 qr, kr;
        if (kNorm) {
          const uint4 wq = __ldg(reinterpret_cast<const uint4*>(p.norm_q_weight) + rv);
          const uint4 wk = __ldg(reinterpret_cast<const uint4*>(p.norm_k_weight) + rv);
          qr = Vec<T>::rope_normed(qv, cs, rstd_s[j], wq);
          kr = Vec<T>::rope_normed(kv, cs, rstd_s[n + j], wk);
        } else {
          qr = Vec<T>::rope(qv, cs);
          kr = Vec<T>::rope(kv, cs);
        }
        *reinterpret_cast<uint4*>(qo_base + j * p.q_out.stride_tok + h * p.q_out.stride_head + e0) = qr;
        *reinterpret_cast<uint4*>(kc_base + j * p.k_cache.stride_tok + h * p.k_cache.stride_head + e0) = kr;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar0 + 8 * (kStages + s));
      cur += n;
      ++i;
    }
  }
}

static uint32_t magic_of(uint32_t d) { return static_cast<uint32_t>(((1ull << 32) + d - 1) / d); }

template <typename T, bool kNorm>
static cudaError_t launch_staged(const AppendParams& p, int device, int grid, int threads, uint32_t smem,
                                 cudaStream_t stream) {
  static DynamicSmemGrant smem_grant;  // one per instantiation
  cudaError_t e = smem_grant.ensure(rope_kv_append_staged_kernel<T, kNorm>, static_cast<int>(smem), device);
  if (e != cudaSuccess) return e;
  rope_kv_append_staged_kernel<T, kNorm><<<grid, threads, smem, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_rope_kv_append(const AppendParams& p_in, int dtype, cudaStream_t stream) {
  AppendParams p = p_in;
  const int esize = dtype == SDV2_DTYPE_BF16 ? 2 : 4;
  const int elems = 16 / esize;
  const int vph = p.head_dim / elems;
  const int row_vecs = p.heads * vph;
  const uint32_t row_bytes = static_cast<uint32_t>(p.heads) * p.head_dim * esize;
  p.plane = p.grid_h * p.grid_w;
  p.magic_plane = magic_of(p.plane);
  p.magic_w = magic_of(p.grid_w);
  p.magic_row_vecs = magic_of(row_vecs);
  p.magic_vph = magic_of(vph);
  p.magic_half = magic_of(p.half);
  // fast_div is exact while numerator * divisor < 2^32
  const bool div_ok = static_cast<uint64_t>(p.tokens) * p.plane < (1ull << 32) &&
                      static_cast<uint64_t>(staged::kMaxTileTokens) * row_vecs * row_vecs < (1ull << 32);
  if (!div_ok || vph > 256 || vph < 1) return cudaErrorInvalidValue;
  if (p.norm_q_weight != nullptr && (dtype != SDV2_DTYPE_BF16 || row_vecs > 1024)) return cudaErrorNotSupported;

  const bool rows_contiguous = p.q.stride_head == p.head_dim && p.k.stride_head == p.head_dim &&
                               p.v.stride_head == p.head_dim;
  // tile size and consumer-warp count: the tile's vectors should split evenly over the consumer
  // threads and three stages must fit in shared memory; then more warps and larger tiles
  const uint32_t mult_row = static_cast<uint32_t>(p.half) * 16u;
  const bool norm = p.norm_q_weight != nullptr;
  const uint32_t norm_row = norm ? 8u + 64u : 0u;   // per token: 1 / rms of its q and k rows + 2 x 8 group sums
  int best_tt = 0, best_w = 0;
  double best_score = 0.0;
  for (int tt = 1; tt <= staged::kMaxTileTokens; ++tt) {
    const uint32_t stage = (3u * tt * row_bytes + tt * (mult_row + norm_row) + 127u) & ~127u;
    if (static_cast<uint64_t>(stage) * staged::kStagesWanted + staged::kTailBytes > staged::kSmemLimit) break;
    for (int w = staged::kMinConsumerWarps; w <= staged::kMaxConsumerWarps; ++w) {
      const int n_vec = tt * row_vecs, thr = 32 * w;
      const int iters = (n_vec + thr - 1) / thr;
      const double util = static_cast<double>(n_vec) / (static_cast<double>(iters) * thr);
      const double score = util + 1e-3 * w + 1e-4 * tt;
      if (score > best_score) {
        best_score = score;
        best_tt = tt;
        best_w = w;
      }
    }
  }
  if (rows_contiguous && best_tt >= 1) {
    p.tile_tokens = best_tt;
    p.stage_bytes = (3u * best_tt * row_bytes + best_tt * (mult_row + norm_row) + 127u) & ~127u;
    p.stages = staged::kStagesWanted;
    const uint32_t smem = p.stages * p.stage_bytes + staged::kTailBytes;
    DeviceInfo di;
    cudaError_t e = device_info(&di);
    if (e != cudaSuccess) return e;
    const int64_t total = static_cast<int64_t>(p.rows) * p.tokens;
    const int grid = static_cast<int>(total < di.sms ? total : di.sms);
    const int threads = (best_w + staged::kProducerWarps) * 32;
    if (norm) return launch_staged<__nv_bfloat16, true>(p, di.device, grid, threads, smem, stream);
    return dtype == SDV2_DTYPE_BF16 ? launch_staged<__nv_bfloat16, false>(p, di.device, grid, threads, smem, stream)
                                    : launch_staged<float, false>(p, di.device, grid, threads, smem, stream);
  }
  if (norm) return cudaErrorNotSupported;   // the per-vector kernel has no row statistics
  const int tok_per_block = 256 / vph;
  dim3 grid((p.tokens + tok_per_block - 1) / tok_per_block, p.heads, p.rows);
  if (dtype == SDV2_DTYPE_BF16)
    rope_kv_append_direct_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else
    rope_kv_append_direct_kernel<float><<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace sdv2

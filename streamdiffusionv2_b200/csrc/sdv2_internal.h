// Launch-parameter structs and launcher prototypes shared by the kernel files and the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/sdv2.h"

namespace sdv2 {

struct AppendParams {
  sdv2_view q, k, v, q_out, k_cache, v_cache;
  const double2* table;  // [table_rows][half] (re, im)
  int rows, tokens, heads, head_dim, half;
  int grid_h, grid_w;
  int cols_t, cols_h;  // complex columns in the temporal and height groups (width gets the rest)
  // filled in by the launcher
  int plane;                // grid_h * grid_w
  uint32_t magic_plane, magic_w, magic_row_vecs, magic_vph, magic_half;  // ceil(2^32 / d) for exact n / d
  int tile_tokens;          // tokens per shared-memory stage (staged kernel)
  uint32_t stage_bytes;     // bytes of one stage: q | k | v rows | multiplier rows
  int stages;               // stages in the shared-memory ring
  int* status;              // optional device word that records an abandoned wait
  int64_t* global_end_dev;
  int64_t* local_end_dev;
  // per-row slot parameters: either the four host-filled arrays below, or, when step_dev is set,
  // a device array [4][rows] (start_frame | dst_begin | global_end | local_end) read by the kernel
  const int64_t* step_dev;
  int64_t cache_tokens;     // bounds for the device-resident parameters
  int table_rows, grid_f;
  // optional RMS norm of q and k over the whole token row (heads * head_dim elements) in front of
  // the rope: bf16 weights [heads * head_dim], or null for no norm (bf16 tensors only)
  const void* norm_q_weight;
  const void* norm_k_weight;
  float norm_eps;
  uint32_t norm_bytes;      // per-stage bytes for the row statistics (staged kernel)
  int64_t start_frame[SDV2_MAX_ROWS];
  int64_t dst_begin[SDV2_MAX_ROWS];
  int64_t global_end_val[SDV2_MAX_ROWS];
  int64_t local_end_val[SDV2_MAX_ROWS];
};

// Returns cudaErrorNotSupported when a norm is requested for a layout the staged kernel cannot take.
cudaError_t launch_rope_kv_append(const AppendParams& p, int dtype, cudaStream_t stream);

struct AttnParams {
  void* out;
  int64_t out_stride_row, out_stride_tok, out_stride_head;  // elements
  int rows, q_tokens, heads;
  int kv_row_broadcast;  // 1: every row reads K/V row 0 (stride-0 expand)
  float scale_log2;      // softmax_scale * log2(e)
  int* status;           // first word of the workspace
  // tail split: tiles [0, n_full) run whole; each of the n_tail tiles after them is cut into `split`
  // key ranges whose partial results (unnormalised O, running max, running sum) go to scratch
  int pair_tiles;        // query tile pairs per (head, row)
  int n_full, n_tail, split;
  float* part_o;         // [n_tail * split][2][128][128] fp32
  float* part_ml;        // [n_tail * split][2][2][128] fp32: max (log2 units), sum
  long long* trace;      // measurement builds only: cycle stamps of CTA 0, 32 per key tile; null otherwise
  int trace_mode;        // with trace: bit 8 (256) runs the MMA rate measurement instead of the attention
  int seq_lens[SDV2_MAX_ROWS];
};

constexpr int kAttnMaxPartialSlots = 192;
constexpr size_t kAttnStatusBytes = 256;
constexpr size_t kAttnPartialBytesPerSlot = 2 * 128 * 128 * 4 + 2 * 2 * 128 * 4;
constexpr int kAttnMinKvTilesForSplit = 16;

// Tail split of the attention grid.  With one CTA per SM, n_tiles = w * sms + tail leaves only
// `tail` SMs busy in the last wave; each of those tiles is cut into `split` key ranges so that the
// last wave takes 1/split of a tile time.  Worth a second launch only when a tile is long
// (min_kv_tiles >= kAttnMinKvTilesForSplit).  The split is lowered until tail * split partial
// slots fit in kAttnMaxPartialSlots, so scratch of that many slots always suffices.
// Returns the split (1 = no split); *n_tail = tiles that are split.
inline int attn_tail_split(int64_t n_tiles, int sms, int min_kv_tiles, bool have_scratch, int* n_tail) {
  *n_tail = 0;
  if (sms <= 0 || !have_scratch) return 1;
  const int tail = static_cast<int>(n_tiles % sms);
  if (tail == 0 || min_kv_tiles < kAttnMinKvTilesForSplit) return 1;
  int split = sms / tail;
  if (split > min_kv_tiles) split = min_kv_tiles;
  if (split > 32) split = 32;
  while (split >= 2 && tail * split > kAttnMaxPartialSlots) --split;
  if (split < 2) return 1;
  *n_tail = tail;
  return split;
}

// Per-device facts that never change while the process lives, looked up once per device.
struct DeviceInfo {
  int device;
  int sms;
};
cudaError_t device_info(DeviceInfo* out);

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device, per-function setting: one instance
// of this class per kernel remembers what was already granted on each device, so that a launch
// makes the runtime call only the first time (or when it needs more than before).
class DynamicSmemGrant {
 public:
  template <typename Kernel>
  cudaError_t ensure(Kernel kernel, int bytes, int device) {
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu_);
    if (granted_[device] >= bytes) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) granted_[device] = bytes;
    return e;
  }

 private:
  static constexpr int kMaxDevices = 64;
  std::mutex mu_;
  int granted_[kMaxDevices] = {};
};

#ifdef __CUDACC__
// RMS statistics shared by sdv2_rmsnorm and the append kernel's fused q/k norm, so that the two
// produce the same bits: a row of n_vec 16-byte vectors is summed as 256 "thread" partials (vector
// c goes to thread c % 256, in ascending order, squares added with fused multiply-adds in element
// order), each group of 32 threads is folded with an xor butterfly (16, 8, 4, 2, 1), and the 8
// group sums with the tree ((g0+g4)+(g2+g6)) + ((g1+g5)+(g3+g7)).
__device__ __forceinline__ float rms_accumulate(float ss, uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a = __uint_as_float(w[j] << 16), b = __uint_as_float(w[j] & 0xFFFF0000u);
    ss = __fmaf_rn(a, a, ss);
    ss = __fmaf_rn(b, b, ss);
  }
  return ss;
}
__device__ __forceinline__ float rms_fold_groups(const float (&g)[8]) {
  return ((g[0] + g[4]) + (g[2] + g[6])) + ((g[1] + g[5]) + (g[3] + g[7]));
}
__device__ __forceinline__ float rms_rstd(float sum_sq, int dim, float eps) { return rsqrtf(sum_sq / dim + eps); }
// bf16(bf16(x * rstd) * weight) for the two halves of a packed bf16 pair
__device__ __forceinline__ uint32_t rms_scale_pair(uint32_t x, float rstd, uint32_t w) {
  uint32_t t, o;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(t) : "f"(__uint_as_float(x & 0xFFFF0000u) * rstd),
      "f"(__uint_as_float(x << 16) * rstd));
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o) : "f"(__uint_as_float(t & 0xFFFF0000u) * __uint_as_float(w & 0xFFFF0000u)),
      "f"(__uint_as_float(t << 16) * __uint_as_float(w << 16)));
  return o;
}
#endif

// Records a failing CUDA call for sdv2_last_cuda_error() and returns SDV2_ERR_CUDA.
int record_cuda_error(cudaError_t e);

cudaError_t launch_attn_tcgen05(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                                const AttnParams& p, cudaStream_t stream);

struct SimtAttnParams {
  sdv2_view q, k, v, out;
  int rows, q_tokens, heads;
  float scale;
  int seq_lens[SDV2_MAX_ROWS];
};
cudaError_t launch_attn_simt(const SimtAttnParams& p, int dtype, cudaStream_t stream);

cudaError_t launch_umma_selftest(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_v,
                                 const void* p_dev, float* s_out, float* o_out, int* status,
                                 cudaStream_t stream);

constexpr int kRingPlanInputs = 7;  // start frame | global end | local end | evict | pop | push value | append slot
struct RingPlanParams {
  const void* sim;       // [rows][sink_frames] similarities of the new frame to the sink frames, or null (no test)
  int dtype, rows, sink_frames;
  float threshold;
  int64_t* queue;        // [rows][1 + queue_cap]: length, entries
  int queue_cap;
  int64_t frame_tokens, sink_tokens, new_tokens;
  const int64_t* host_dev;                          // optional device copy of host_val, [kRingPlanInputs][rows]
  int64_t host_val[kRingPlanInputs][SDV2_MAX_ROWS];
  int64_t* step_params;  // out: [4][rows] for the append kernel
  int* status;
};
cudaError_t launch_ring_plan(const RingPlanParams& p, cudaStream_t stream);

constexpr int kFrameMeanChunks = 16;   // token chunks per frame in the first pass
struct FrameMeansParams {
  sdv2_view k_cache, v_cache, k_new, v_new;   // heads of a token back to back
  int rows, sink_frames, frame_tokens, row_elems, dtype, chunks;
  float* partial;   // [rows][sink + 1][2][chunks][row_elems]
  void* means;      // [rows][sink + 1][2][row_elems], in the tensors' type
};
cudaError_t launch_frame_means(const FrameMeansParams& p, cudaStream_t stream);

cudaError_t launch_wait_timeout_selftest(int* status, long long budget_cycles, cudaStream_t stream);

}  // namespace sdv2

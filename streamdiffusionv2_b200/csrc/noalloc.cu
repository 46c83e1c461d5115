// sdv2_attn_kvcache_static: cache attention for hosts that cannot hand the library a workspace.
//
// Some embedders of this library own no device allocator at all: a C or C++ serving loop that was
// given a fixed set of borrowed tensor pointers by its framework, a worker whose whole memory
// budget was carved up at start-up (K/V caches, weights, decoder engine) and that must not call
// cudaMalloc in the per-chunk path because an allocation serialises the device and can fail late,
// or a plug-in ABI that simply has no slot for "scratch pointer + size".  For them the scratch the
// split attention kernel needs (the status block and the partial results of the tail tiles) lives
// here, in a file-scope device array that every GPU loading the library holds until exit.
//
// Limits, stated once: the array holds the 256-byte status block plus kStaticSlots = 192 partial
// slots of 133,120 bytes, 25,559,296 bytes (24.4 MiB) per GPU in total.  A call whose tail split
// would need more slots than that is refused with SDV2_ERR_WORKSPACE before anything is launched.
//
// Sharing: all calls on a device use the same array.  It keeps whatever the previous call left;
// partial slots are always written by the attention kernel before the combine kernel reads them,
// and the status block is zeroed once at set-up and afterwards only by sdv2_read_status, so
// nothing stale is ever consumed.  Two calls that overlap on the GPU (different streams, or two
// host threads) would write the same slots and race: callers must order them.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "sdv2_internal.h"

namespace {

constexpr int kStaticSlots = sdv2::kAttnMaxPartialSlots;  // 192
constexpr size_t kStaticBytes = sdv2::kAttnStatusBytes + kStaticSlots * sdv2::kAttnPartialBytesPerSlot;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
struct DeviceScratch {
  bool ready = false;
  void* ptr = nullptr;
};
DeviceScratch g_devices[kMaxDevices];
std::mutex g_mutex;

// Device address of the array on the current device; resolved and zero-initialised (status block
// only) on the first call per device.  That first call synchronises and must therefore happen
// before any stream capture begins.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceScratch& d = g_devices[dev];
  if (!d.ready) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);  // per device: each GPU has its own copy
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemset(p, 0, sdv2::kAttnStatusBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    d.ptr = p;
    d.ready = true;
  }
  *out = d.ptr;
  return 0;
}

// Partial slots the launcher's tail split will use for this problem on this device (same
// arithmetic as the launcher, so the refusal below is exact).
int slots_needed(int rows, int q_tokens, int heads, const int32_t* seq_lens, int sms) {
  const int64_t pair_tiles = (q_tokens + 255) / 256;
  const int64_t n_tiles = pair_tiles * heads * rows;
  int min_kv = 0x7FFFFFFF;
  for (int b = 0; b < rows; ++b) {
    const int kv = (seq_lens[b] + 127) / 128;
    if (kv < min_kv) min_kv = kv;
  }
  const int tail = static_cast<int>(n_tiles % sms);
  if (tail == 0 || min_kv < 16) return 0;
  int split = sms / tail;
  if (split > min_kv) split = min_kv;
  if (split > 32) split = 32;
  return split >= 2 ? tail * split : 0;
}

}  // namespace

extern "C" int sdv2_attn_kvcache_static(const sdv2_view* q, const sdv2_view* k_cache, const sdv2_view* v_cache,
                                        const sdv2_view* out, int rows, int q_tokens, int heads, int head_dim,
                                        int64_t cache_tokens, const int32_t* seq_lens, float softmax_scale,
                                        void** status_dev_out, void* stream) {
  if (seq_lens == nullptr || rows <= 0 || q_tokens <= 0 || heads <= 0) return SDV2_ERR_INVALID_ARG;
  if (rows > SDV2_MAX_ROWS) return SDV2_ERR_UNSUPPORTED_SHAPE;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return SDV2_ERR_CUDA;
  for (int b = 0; b < rows; ++b)
    if (seq_lens[b] < 1 || seq_lens[b] > cache_tokens) return SDV2_ERR_INVALID_ARG;
  // refuse, before any launch, what the built-in array cannot hold
  if (slots_needed(rows, q_tokens, heads, seq_lens, sms) > kStaticSlots) return SDV2_ERR_WORKSPACE;
  void* scratch = nullptr;
  if (scratch_for_current_device(&scratch) != 0) return SDV2_ERR_CUDA;
  if (status_dev_out != nullptr) *status_dev_out = scratch;  // may be passed to sdv2_read_status
  return sdv2_attn_kvcache(q, k_cache, v_cache, out, rows, q_tokens, heads, head_dim, cache_tokens, seq_lens,
                           softmax_scale, scratch, kStaticBytes, stream);
}

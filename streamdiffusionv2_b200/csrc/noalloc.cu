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
// slots of 133,120 bytes, 25,559,296 bytes (24.4 MiB) per GPU in total.  That is always enough:
// the launcher lowers the tail split until it fits 192 slots (attn_tail_split), so no shape is
// refused for lack of scratch.  What is refused is what sdv2_attn_kvcache refuses too, plus more
// than SDV2_MAX_ROWS cache rows.
//
// Sharing: all calls on a device use the same array.  It keeps whatever the previous call left;
// partial slots are always written by the attention kernel before the combine kernel reads them,
// and the status block starts as zeros (static device storage is zero-initialised when the module
// is loaded) and is afterwards cleared only by sdv2_read_status, so nothing stale is ever
// consumed.  Two calls that overlap on the GPU (different streams, or two host threads) would
// write the same slots and race: callers must order them.
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

// Device address of the array on the current device, resolved on the first call per device (a
// host-side look-up: nothing is launched, copied or synchronised).
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return sdv2::record_cuda_error(e);
  if (dev < 0 || dev >= kMaxDevices) return sdv2::record_cuda_error(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceScratch& d = g_devices[dev];
  if (!d.ready) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);  // per device: each GPU has its own copy
    if (e != cudaSuccess) return sdv2::record_cuda_error(e);
    d.ptr = p;
    d.ready = true;
  }
  *out = d.ptr;
  return SDV2_OK;
}

}  // namespace

extern "C" int sdv2_attn_kvcache_static(const sdv2_view* q, const sdv2_view* k_cache, const sdv2_view* v_cache,
                                        const sdv2_view* out, int rows, int q_tokens, int heads, int head_dim,
                                        int64_t cache_tokens, const int32_t* seq_lens, float softmax_scale,
                                        void** status_dev_out, void* stream) {
  if (seq_lens == nullptr || rows <= 0 || q_tokens <= 0 || heads <= 0) return SDV2_ERR_INVALID_ARG;
  if (rows > SDV2_MAX_ROWS) return SDV2_ERR_UNSUPPORTED_SHAPE;
  sdv2::DeviceInfo di;
  cudaError_t e = sdv2::device_info(&di);
  if (e != cudaSuccess) return sdv2::record_cuda_error(e);
  int min_kv = 0x7FFFFFFF;
  for (int b = 0; b < rows; ++b) {
    if (seq_lens[b] < 1 || seq_lens[b] > cache_tokens) return SDV2_ERR_INVALID_ARG;
    const int kv = (seq_lens[b] + 127) / 128;
    if (kv < min_kv) min_kv = kv;
  }
  // cannot fail: the launcher's split (the same helper) never asks for more than the array holds
  int n_tail = 0;
  const int split = sdv2::attn_tail_split(static_cast<int64_t>((q_tokens + 255) / 256) * heads * rows, di.sms, min_kv,
                                          true, &n_tail);
  if (n_tail * split > kStaticSlots) return SDV2_ERR_WORKSPACE;
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != SDV2_OK) return rc;
  if (status_dev_out != nullptr) *status_dev_out = scratch;  // may be passed to sdv2_read_status
  return sdv2_attn_kvcache(q, k_cache, v_cache, out, rows, q_tokens, heads, head_dim, cache_tokens, seq_lens,
                           softmax_scale, scratch, kStaticBytes, stream);
}

// C ABI of libsdv2.so: argument validation, TMA descriptor construction, launches.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "sdv2_internal.h"

namespace {
thread_local int g_last_cuda_error = 0;
}

namespace sdv2 {

int record_cuda_error(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return SDV2_ERR_CUDA;
}

cudaError_t device_info(DeviceInfo* out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int sms[kMaxDevices];  // 0 = not looked up yet
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (sms[dev] == 0) {
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    if (n <= 0) return cudaErrorInvalidDevice;
    sms[dev] = n;
  }
  out->device = dev;
  out->sms = sms[dev];
  return cudaSuccess;
}

}  // namespace sdv2

namespace {

int cuda_fail(cudaError_t e) { return sdv2::record_cuda_error(e); }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// pointer, strides (in elements of `esize` bytes) all 16-byte aligned
int check_view(const sdv2_view* v, int esize, bool allow_row_broadcast) {
  if (v == nullptr || v->ptr == nullptr) return SDV2_ERR_INVALID_ARG;
  if (!aligned16(v->ptr)) return SDV2_ERR_MISALIGNED;
  const int64_t per16 = 16 / esize;
  if (v->stride_tok <= 0 || v->stride_head <= 0) return SDV2_ERR_INVALID_ARG;
  if (v->stride_row < 0 || (v->stride_row == 0 && !allow_row_broadcast)) return SDV2_ERR_INVALID_ARG;
  if (v->stride_row % per16 || v->stride_tok % per16 || v->stride_head % per16) return SDV2_ERR_MISALIGNED;
  return SDV2_OK;
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

// bf16 [rows, tokens, heads, 128] view -> 4-D map (d, head, token, row), box 64 x 1 x 128 x 1,
// 128-byte swizzle, out-of-range rows read as zero.
int make_tile_map(CUtensorMap* tm, const sdv2_view* v, int rows, int64_t tokens, int heads) {
  auto fn = encode_fn();
  if (fn == nullptr) return cuda_fail(cudaErrorSymbolNotFound);
  cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(tokens),
                        static_cast<cuuint64_t>(rows)};
  // a broadcast or single row still needs a legal (non-zero, 16-byte multiple) stride
  const int64_t row_stride = (v->stride_row > 0 ? v->stride_row : v->stride_tok * tokens);
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(v->stride_head) * 2, static_cast<cuuint64_t>(v->stride_tok) * 2,
                           static_cast<cuuint64_t>(row_stride) * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, v->ptr, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return SDV2_ERR_CUDA;
  }
  return SDV2_OK;
}

int make_square_map(CUtensorMap* tm, const void* ptr) {
  auto fn = encode_fn();
  if (fn == nullptr) return cuda_fail(cudaErrorSymbolNotFound);
  cuuint64_t dims[2] = {128, 128};
  cuuint64_t strides[1] = {256};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return SDV2_ERR_CUDA;
  }
  return SDV2_OK;
}

constexpr size_t kStatusBytes = sdv2::kAttnStatusBytes;

int attn_common(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v, const sdv2_view* out, int rows,
                int q_tokens, int heads, int head_dim, int64_t kv_extent, const int32_t* seq_lens,
                int uniform_len, float softmax_scale, void* workspace, size_t workspace_bytes,
                bool allow_kv_broadcast, void* stream) {
  if (rows <= 0 || q_tokens <= 0 || heads <= 0 || kv_extent <= 0) return SDV2_ERR_INVALID_ARG;
  if (head_dim != 128 || rows > SDV2_MAX_ROWS || heads > 65535) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (workspace == nullptr || workspace_bytes < kStatusBytes) return SDV2_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return SDV2_ERR_MISALIGNED;
  int rc;
  if ((rc = check_view(q, 2, false)) != SDV2_OK) return rc;
  if ((rc = check_view(out, 2, false)) != SDV2_OK) return rc;
  if ((rc = check_view(k, 2, allow_kv_broadcast)) != SDV2_OK) return rc;
  if ((rc = check_view(v, 2, allow_kv_broadcast)) != SDV2_OK) return rc;
  if ((k->stride_row == 0) != (v->stride_row == 0)) return SDV2_ERR_INVALID_ARG;
  if (!(softmax_scale > 0.f) || !isfinite(softmax_scale)) return SDV2_ERR_INVALID_ARG;

  sdv2::AttnParams p;
  memset(&p, 0, sizeof(p));
  for (int b = 0; b < rows; ++b) {
    const int len = seq_lens ? seq_lens[b] : uniform_len;
    if (len < 1 || len > kv_extent) return SDV2_ERR_INVALID_ARG;
    p.seq_lens[b] = len;
  }
  p.out = out->ptr;
  p.out_stride_row = out->stride_row;
  p.out_stride_tok = out->stride_tok;
  p.out_stride_head = out->stride_head;
  p.rows = rows;
  p.q_tokens = q_tokens;
  p.heads = heads;
  p.kv_row_broadcast = (k->stride_row == 0) ? 1 : 0;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = static_cast<int*>(workspace);
  // measurement aid: with SDV2_ATTN_TRACE set, CTA 0 writes cycle stamps into the scratch area instead (no tail split)
  static const int trace = getenv("SDV2_ATTN_TRACE") ? atoi(getenv("SDV2_ATTN_TRACE")) : 0;
  p.trace_mode = trace;
  if (trace && workspace_bytes >= kStatusBytes + 256 * 32 * sizeof(long long)) {
    p.trace = reinterpret_cast<long long*>(static_cast<char*>(workspace) + kStatusBytes);
  } else if (workspace_bytes >= kStatusBytes + sdv2::kAttnMaxPartialSlots * sdv2::kAttnPartialBytesPerSlot) {
    p.part_ml = reinterpret_cast<float*>(static_cast<char*>(workspace) + kStatusBytes);
    p.part_o = p.part_ml + static_cast<size_t>(sdv2::kAttnMaxPartialSlots) * 2 * 2 * 128;
  }

  CUtensorMap tm_q, tm_k, tm_v;
  if ((rc = make_tile_map(&tm_q, q, rows, q_tokens, heads)) != SDV2_OK) return rc;
  const int kv_rows = p.kv_row_broadcast ? 1 : rows;
  if ((rc = make_tile_map(&tm_k, k, kv_rows, kv_extent, heads)) != SDV2_OK) return rc;
  if ((rc = make_tile_map(&tm_v, v, kv_rows, kv_extent, heads)) != SDV2_OK) return rc;
  cudaError_t e = sdv2::launch_attn_tcgen05(tm_q, tm_k, tm_v, p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? SDV2_OK : cuda_fail(e);
}

}  // namespace

extern "C" {

int sdv2_abi_version(void) { return SDV2_ABI_VERSION; }

const char* sdv2_strerror(int code) {
  switch (code) {
    case SDV2_OK: return "ok";
    case SDV2_ERR_INVALID_ARG: return "invalid argument";
    case SDV2_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
    case SDV2_ERR_MISALIGNED: return "pointer or stride not 16-byte aligned";
    case SDV2_ERR_CUDA: return "CUDA call failed";
    case SDV2_ERR_TIMEOUT: return "device-side wait timed out";
    case SDV2_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown error";
  }
}

int sdv2_last_cuda_error(void) { return g_last_cuda_error; }

// Shared by the two append entry points: slot parameters either in the four host arrays or in
// `step_params_dev` (device, [4][rows]).
static int append_common(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v, const sdv2_view* q_out,
                         const sdv2_view* k_cache, const sdv2_view* v_cache, int rows, int new_tokens, int heads,
                         int head_dim, int64_t cache_tokens, const double* rope_table_dev, int table_rows,
                         int grid_f, int grid_h, int grid_w, const int64_t* start_frame,
                         const int64_t* dst_begin, int64_t* global_end_dev, int64_t* local_end_dev,
                         const int64_t* global_end_val, const int64_t* local_end_val,
                         const int64_t* step_params_dev, int dtype, int* status_dev, void* stream,
                         const void* norm_q_weight_dev = nullptr, const void* norm_k_weight_dev = nullptr,
                         float norm_eps = 0.f) {
  if (rows <= 0 || new_tokens <= 0 || heads <= 0 || cache_tokens <= 0 || table_rows <= 0) return SDV2_ERR_INVALID_ARG;
  if (grid_f <= 0 || grid_h <= 0 || grid_w <= 0) return SDV2_ERR_INVALID_ARG;
  if (static_cast<int64_t>(grid_f) * grid_h * grid_w != new_tokens) return SDV2_ERR_INVALID_ARG;
  if (dtype != SDV2_DTYPE_BF16 && dtype != SDV2_DTYPE_F32) return SDV2_ERR_INVALID_ARG;
  if (rows > SDV2_MAX_ROWS) return SDV2_ERR_UNSUPPORTED_SHAPE;
  const int esize = dtype == SDV2_DTYPE_BF16 ? 2 : 4;
  if (head_dim <= 0 || head_dim % (16 / esize) || head_dim % 2) return SDV2_ERR_UNSUPPORTED_SHAPE;
  const bool indirect = step_params_dev != nullptr;
  if (rope_table_dev == nullptr) return SDV2_ERR_INVALID_ARG;
  if (!indirect && (start_frame == nullptr || dst_begin == nullptr)) return SDV2_ERR_INVALID_ARG;
  if (indirect && (reinterpret_cast<uintptr_t>(step_params_dev) & 7u)) return SDV2_ERR_MISALIGNED;
  if (!aligned16(rope_table_dev)) return SDV2_ERR_MISALIGNED;
  if ((global_end_dev == nullptr) != (local_end_dev == nullptr)) return SDV2_ERR_INVALID_ARG;
  if (!indirect && global_end_dev != nullptr && (global_end_val == nullptr || local_end_val == nullptr))
    return SDV2_ERR_INVALID_ARG;
  int rc;
  const sdv2_view* views[6] = {q, k, v, q_out, k_cache, v_cache};
  for (const sdv2_view* vw : views)
    if ((rc = check_view(vw, esize, false)) != SDV2_OK) return rc;
  if (grid_h > table_rows || grid_w > table_rows) return SDV2_ERR_INVALID_ARG;
  if ((norm_q_weight_dev == nullptr) != (norm_k_weight_dev == nullptr)) return SDV2_ERR_INVALID_ARG;
  if (norm_q_weight_dev != nullptr) {
    if (dtype != SDV2_DTYPE_BF16) return SDV2_ERR_UNSUPPORTED_SHAPE;
    if (!aligned16(norm_q_weight_dev) || !aligned16(norm_k_weight_dev)) return SDV2_ERR_MISALIGNED;
    if (!(norm_eps >= 0.f) || !isfinite(norm_eps)) return SDV2_ERR_INVALID_ARG;
  }

  sdv2::AppendParams p;
  memset(&p, 0, sizeof(p));
  p.norm_q_weight = norm_q_weight_dev;
  p.norm_k_weight = norm_k_weight_dev;
  p.norm_eps = norm_eps;
  for (int b = 0; b < rows && !indirect; ++b) {
    // the reference fails with a shape mismatch where these hold; fail loudly instead of writing
    // outside the cache or reading past the rope table
    if (dst_begin[b] < 0 || dst_begin[b] + new_tokens > cache_tokens) return SDV2_ERR_INVALID_ARG;
    if (start_frame[b] < 0 || start_frame[b] + grid_f > table_rows) return SDV2_ERR_INVALID_ARG;
    p.start_frame[b] = start_frame[b];
    p.dst_begin[b] = dst_begin[b];
    if (global_end_dev != nullptr) {
      p.global_end_val[b] = global_end_val[b];
      p.local_end_val[b] = local_end_val[b];
    }
  }
  p.q = *q; p.k = *k; p.v = *v; p.q_out = *q_out; p.k_cache = *k_cache; p.v_cache = *v_cache;
  p.table = reinterpret_cast<const double2*>(rope_table_dev);
  p.rows = rows;
  p.tokens = new_tokens;
  p.heads = heads;
  p.head_dim = head_dim;
  p.half = head_dim / 2;
  p.grid_h = grid_h;
  p.grid_w = grid_w;
  p.cols_t = p.half - 2 * (p.half / 3);
  p.cols_h = p.half / 3;
  p.global_end_dev = global_end_dev;
  p.local_end_dev = local_end_dev;
  p.step_dev = step_params_dev;
  p.cache_tokens = cache_tokens;
  p.table_rows = table_rows;
  p.grid_f = grid_f;
  p.status = status_dev;
  cudaError_t e = sdv2::launch_rope_kv_append(p, dtype, static_cast<cudaStream_t>(stream));
  if (e == cudaErrorNotSupported) return SDV2_ERR_UNSUPPORTED_SHAPE;
  return e == cudaSuccess ? SDV2_OK : cuda_fail(e);
}

int sdv2_norm_rope_kv_append(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v, const sdv2_view* q_out,
                             const sdv2_view* k_cache, const sdv2_view* v_cache, int rows, int new_tokens, int heads,
                             int head_dim, int64_t cache_tokens, const double* rope_table_dev, int table_rows,
                             int grid_f, int grid_h, int grid_w, const int64_t* start_frame,
                             const int64_t* dst_begin, const int64_t* step_params_dev, int64_t* global_end_dev,
                             int64_t* local_end_dev, const int64_t* global_end_val, const int64_t* local_end_val,
                             const void* norm_q_weight_dev, const void* norm_k_weight_dev, float norm_eps,
                             int* status_dev, void* stream) {
  if (norm_q_weight_dev == nullptr || norm_k_weight_dev == nullptr) return SDV2_ERR_INVALID_ARG;
  return append_common(q, k, v, q_out, k_cache, v_cache, rows, new_tokens, heads, head_dim, cache_tokens,
                       rope_table_dev, table_rows, grid_f, grid_h, grid_w, start_frame, dst_begin, global_end_dev,
                       local_end_dev, global_end_val, local_end_val, step_params_dev, SDV2_DTYPE_BF16, status_dev,
                       stream, norm_q_weight_dev, norm_k_weight_dev, norm_eps);
}

int sdv2_rope_kv_append(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v, const sdv2_view* q_out,
                        const sdv2_view* k_cache, const sdv2_view* v_cache, int rows, int new_tokens, int heads,
                        int head_dim, int64_t cache_tokens, const double* rope_table_dev, int table_rows,
                        int grid_f, int grid_h, int grid_w, const int64_t* start_frame,
                        const int64_t* dst_begin, int64_t* global_end_dev, int64_t* local_end_dev,
                        const int64_t* global_end_val, const int64_t* local_end_val, int dtype, int* status_dev,
                        void* stream) {
  return append_common(q, k, v, q_out, k_cache, v_cache, rows, new_tokens, heads, head_dim, cache_tokens,
                       rope_table_dev, table_rows, grid_f, grid_h, grid_w, start_frame, dst_begin, global_end_dev,
                       local_end_dev, global_end_val, local_end_val, nullptr, dtype, status_dev, stream);
}

int sdv2_rope_kv_append_indirect(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v,
                                 const sdv2_view* q_out, const sdv2_view* k_cache, const sdv2_view* v_cache,
                                 int rows, int new_tokens, int heads, int head_dim, int64_t cache_tokens,
                                 const double* rope_table_dev, int table_rows, int grid_f, int grid_h, int grid_w,
                                 const int64_t* step_params_dev, int64_t* global_end_dev, int64_t* local_end_dev,
                                 int dtype, int* status_dev, void* stream) {
  if (step_params_dev == nullptr) return SDV2_ERR_INVALID_ARG;
  return append_common(q, k, v, q_out, k_cache, v_cache, rows, new_tokens, heads, head_dim, cache_tokens,
                       rope_table_dev, table_rows, grid_f, grid_h, grid_w, nullptr, nullptr, global_end_dev,
                       local_end_dev, nullptr, nullptr, step_params_dev, dtype, status_dev, stream);
}

size_t sdv2_attn_workspace_bytes(int rows, int q_tokens, int heads, int head_dim) {
  (void)rows; (void)q_tokens; (void)heads; (void)head_dim;
  // status block + scratch for the partial results of split tail tiles (at most one per SM)
  return kStatusBytes + sdv2::kAttnMaxPartialSlots * sdv2::kAttnPartialBytesPerSlot;
}

int sdv2_attn_partial_slots(int rows, int q_tokens, int heads, int min_seq_len, int sm_count) {
  if (rows <= 0 || q_tokens <= 0 || heads <= 0 || min_seq_len <= 0 || sm_count <= 0) return 0;
  int n_tail = 0;
  const int split = sdv2::attn_tail_split(static_cast<int64_t>((q_tokens + 255) / 256) * heads * rows, sm_count,
                                          (min_seq_len + 127) / 128, true, &n_tail);
  return n_tail * split;
}

int sdv2_attn_kvcache(const sdv2_view* q, const sdv2_view* k_cache, const sdv2_view* v_cache,
                      const sdv2_view* out, int rows, int q_tokens, int heads, int head_dim, int64_t cache_tokens,
                      const int32_t* seq_lens, float softmax_scale, void* workspace_dev, size_t workspace_bytes,
                      void* stream) {
  if (seq_lens == nullptr) return SDV2_ERR_INVALID_ARG;
  return attn_common(q, k_cache, v_cache, out, rows, q_tokens, heads, head_dim, cache_tokens, seq_lens, 0,
                     softmax_scale, workspace_dev, workspace_bytes, false, stream);
}

int sdv2_cross_attn(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v, const sdv2_view* out, int rows,
                    int q_tokens, int heads, int head_dim, int kv_tokens, float softmax_scale,
                    void* workspace_dev, size_t workspace_bytes, void* stream) {
  return attn_common(q, k, v, out, rows, q_tokens, heads, head_dim, kv_tokens, nullptr, kv_tokens,
                     softmax_scale, workspace_dev, workspace_bytes, true, stream);
}

int sdv2_attn_kvcache_simt(const sdv2_view* q, const sdv2_view* k_cache, const sdv2_view* v_cache,
                           const sdv2_view* out, int rows, int q_tokens, int heads, int head_dim,
                           int64_t cache_tokens, const int32_t* seq_lens, float softmax_scale, int dtype,
                           void* stream) {
  if (rows <= 0 || q_tokens <= 0 || heads <= 0 || cache_tokens <= 0 || seq_lens == nullptr) return SDV2_ERR_INVALID_ARG;
  if (dtype != SDV2_DTYPE_BF16 && dtype != SDV2_DTYPE_F32) return SDV2_ERR_INVALID_ARG;
  if (head_dim != 128 || rows > SDV2_MAX_ROWS) return SDV2_ERR_UNSUPPORTED_SHAPE;
  const int esize = dtype == SDV2_DTYPE_BF16 ? 2 : 4;
  int rc;
  if ((rc = check_view(q, esize, false)) != SDV2_OK) return rc;
  if ((rc = check_view(out, esize, false)) != SDV2_OK) return rc;
  if ((rc = check_view(k_cache, esize, true)) != SDV2_OK) return rc;
  if ((rc = check_view(v_cache, esize, true)) != SDV2_OK) return rc;
  sdv2::SimtAttnParams p;
  memset(&p, 0, sizeof(p));
  for (int b = 0; b < rows; ++b) {
    if (seq_lens[b] < 1 || seq_lens[b] > cache_tokens) return SDV2_ERR_INVALID_ARG;
    p.seq_lens[b] = seq_lens[b];
  }
  p.q = *q; p.k = *k_cache; p.v = *v_cache; p.out = *out;
  p.rows = rows; p.q_tokens = q_tokens; p.heads = heads;
  p.scale = softmax_scale;
  cudaError_t e = sdv2::launch_attn_simt(p, dtype, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? SDV2_OK : cuda_fail(e);
}

int sdv2_read_status(void* workspace_dev, int* detail, void* stream) {
  if (workspace_dev == nullptr) return SDV2_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, workspace_dev, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return cuda_fail(e);
  if (detail) *detail = word;
  if (word == 0) return SDV2_OK;
  e = cudaMemsetAsync(workspace_dev, 0, sizeof(int), s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return cuda_fail(e);
  return (word & 0xFF) == 10 ? SDV2_ERR_INVALID_ARG : SDV2_ERR_TIMEOUT;  // 10: BAD_STEP_PARAMS
}

int sdv2_selftest_umma(const void* a_dev, const void* b_dev, const void* p_dev, const void* v_dev,
                       float* s_out_dev, float* o_out_dev, int* status_dev, void* stream) {
  if (!a_dev || !b_dev || !p_dev || !v_dev || !s_out_dev || !o_out_dev || !status_dev) return SDV2_ERR_INVALID_ARG;
  if (!aligned16(a_dev) || !aligned16(b_dev) || !aligned16(p_dev) || !aligned16(v_dev)) return SDV2_ERR_MISALIGNED;
  CUtensorMap ta, tb, tv;
  int rc;
  if ((rc = make_square_map(&ta, a_dev)) != SDV2_OK) return rc;
  if ((rc = make_square_map(&tb, b_dev)) != SDV2_OK) return rc;
  if ((rc = make_square_map(&tv, v_dev)) != SDV2_OK) return rc;
  cudaError_t e = sdv2::launch_umma_selftest(ta, tb, tv, p_dev, s_out_dev, o_out_dev, status_dev,
                                             static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? SDV2_OK : cuda_fail(e);
}

size_t sdv2_frame_means_scratch_bytes(int rows, int sink_frames, int heads, int head_dim) {
  if (rows <= 0 || sink_frames < 0 || heads <= 0 || head_dim <= 0) return 0;
  return static_cast<size_t>(rows) * (sink_frames + 1) * 2 * sdv2::kFrameMeanChunks * heads * head_dim * sizeof(float);
}

int sdv2_frame_means(const sdv2_view* k_cache, const sdv2_view* v_cache, const sdv2_view* k_new, const sdv2_view* v_new,
                     int rows, int sink_frames, int frame_tokens, int heads, int head_dim, int64_t cache_tokens,
                     int dtype, void* means_dev, void* scratch_dev, size_t scratch_bytes, void* stream) {
  if (rows <= 0 || sink_frames < 0 || frame_tokens <= 0 || heads <= 0 || head_dim <= 0) return SDV2_ERR_INVALID_ARG;
  if (dtype != SDV2_DTYPE_BF16 && dtype != SDV2_DTYPE_F32) return SDV2_ERR_INVALID_ARG;
  if (rows > SDV2_MAX_ROWS || sink_frames > 64) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (static_cast<int64_t>(sink_frames) * frame_tokens > cache_tokens) return SDV2_ERR_INVALID_ARG;
  if (means_dev == nullptr || scratch_dev == nullptr) return SDV2_ERR_INVALID_ARG;
  if (scratch_bytes < sdv2_frame_means_scratch_bytes(rows, sink_frames, heads, head_dim)) return SDV2_ERR_WORKSPACE;
  const int esize = dtype == SDV2_DTYPE_BF16 ? 2 : 4;
  if ((heads * head_dim) % (16 / esize)) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (!aligned16(means_dev) || !aligned16(scratch_dev)) return SDV2_ERR_MISALIGNED;
  int rc;
  const sdv2_view* views[4] = {k_cache, v_cache, k_new, v_new};
  for (const sdv2_view* vw : views) {
    if ((rc = check_view(vw, esize, false)) != SDV2_OK) return rc;
    if (vw->stride_head != head_dim) return SDV2_ERR_UNSUPPORTED_SHAPE;   // a token's heads as one run
  }
  sdv2::FrameMeansParams p;
  memset(&p, 0, sizeof(p));
  p.k_cache = *k_cache; p.v_cache = *v_cache; p.k_new = *k_new; p.v_new = *v_new;
  p.rows = rows; p.sink_frames = sink_frames; p.frame_tokens = frame_tokens; p.row_elems = heads * head_dim;
  p.dtype = dtype; p.chunks = sdv2::kFrameMeanChunks;
  p.partial = static_cast<float*>(scratch_dev);
  p.means = means_dev;
  cudaError_t e = sdv2::launch_frame_means(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? SDV2_OK : cuda_fail(e);
}

int sdv2_ring_plan_adaptive(const void* sim_dev, int sim_dtype, int rows, int sink_frames, float threshold,
                            int64_t* queue_dev, int queue_cap, int64_t frame_tokens, int64_t new_tokens,
                            const int64_t* host_inputs, const int64_t* host_inputs_dev, int64_t* step_params_dev,
                            int* status_dev, void* stream) {
  if (queue_dev == nullptr || step_params_dev == nullptr) return SDV2_ERR_INVALID_ARG;
  if ((host_inputs == nullptr) == (host_inputs_dev == nullptr)) return SDV2_ERR_INVALID_ARG;
  if (rows <= 0 || queue_cap <= 0 || frame_tokens <= 0 || new_tokens <= 0 || sink_frames < 0) return SDV2_ERR_INVALID_ARG;
  if (rows > SDV2_MAX_ROWS) return SDV2_ERR_UNSUPPORTED_SHAPE;
  if (sim_dev != nullptr && sim_dtype != SDV2_DTYPE_BF16 && sim_dtype != SDV2_DTYPE_F32) return SDV2_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(queue_dev) | reinterpret_cast<uintptr_t>(step_params_dev) |
       reinterpret_cast<uintptr_t>(host_inputs_dev)) & 7u)
    return SDV2_ERR_MISALIGNED;
  sdv2::RingPlanParams p;
  memset(&p, 0, sizeof(p));
  p.sim = sink_frames > 0 ? sim_dev : nullptr;
  p.dtype = sim_dtype;
  p.rows = rows;
  p.sink_frames = sink_frames;
  p.threshold = threshold;
  p.queue = queue_dev;
  p.queue_cap = queue_cap;
  p.frame_tokens = frame_tokens;
  p.sink_tokens = frame_tokens * sink_frames;
  p.new_tokens = new_tokens;
  p.host_dev = host_inputs_dev;
  if (host_inputs != nullptr)
    for (int w = 0; w < sdv2::kRingPlanInputs; ++w)
      for (int b = 0; b < rows; ++b) p.host_val[w][b] = host_inputs[w * rows + b];
  p.step_params = step_params_dev;
  p.status = status_dev;
  cudaError_t e = sdv2::launch_ring_plan(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? SDV2_OK : cuda_fail(e);
}

int sdv2_selftest_wait_timeout(int* status_dev, long long budget_cycles, void* stream) {
  if (status_dev == nullptr) return SDV2_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(status_dev) & 3u) return SDV2_ERR_MISALIGNED;
  if (budget_cycles < 10000LL) budget_cycles = 10000LL;
  if (budget_cycles > 2000000000LL) budget_cycles = 2000000000LL;
  cudaError_t e = sdv2::launch_wait_timeout_selftest(status_dev, budget_cycles, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? SDV2_OK : cuda_fail(e);
}

}  // extern "C"

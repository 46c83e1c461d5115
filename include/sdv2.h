/*
 * sdv2.h - C ABI of libsdv2.so: sm_100a kernels for the per-chunk causal self-attention of the
 * causal Wan DiT used by StreamDiffusionV2 (ring-buffer K/V cache with sink slots, attention
 * over the wrapped cache, text cross-attention from a persistent K/V cache).
 *
 * Conventions
 *   - every pointer named *_dev or held in an sdv2_view is a CUDA device pointer borrowed for the
 *     duration of the call; nothing is allocated, freed or retained by the library;
 *   - arrays documented as "host" are read during the call and copied into the launch parameters;
 *   - `stream` is a cudaStream_t passed as void*; calls enqueue work and return without
 *     synchronising (except sdv2_read_status);
 *   - return value: SDV2_OK or a negative SDV2_ERR_* code; the library never aborts or traps;
 *   - element strides are in elements of the tensor's dtype; the innermost (head_dim) stride is 1.
 *
 * "Reference" below is the upstream Python implementation; paths are relative to its root.
 */
#ifndef SDV2_H_
#define SDV2_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SDV2_ABI_VERSION 1
#define SDV2_MAX_ROWS 64 /* cache batch rows (denoise levels x streams) per call */

enum {
  SDV2_OK = 0,
  SDV2_ERR_INVALID_ARG = -1,       /* null pointer, negative size, slot outside the cache ... */
  SDV2_ERR_UNSUPPORTED_SHAPE = -2, /* head_dim != 128, too many rows ... */
  SDV2_ERR_MISALIGNED = -3,        /* pointer or stride not 16-byte aligned */
  SDV2_ERR_CUDA = -4,              /* a CUDA runtime/driver call failed; see sdv2_last_cuda_error */
  SDV2_ERR_TIMEOUT = -5,           /* a bounded device-side wait ran out (reported by sdv2_read_status) */
  SDV2_ERR_WORKSPACE = -6          /* workspace missing or too small */
};

enum { SDV2_DTYPE_BF16 = 0, SDV2_DTYPE_F32 = 1 };

/* A [rows, tokens, heads, head_dim] tensor view with head_dim contiguous. stride_row may be 0
 * (one row broadcast to all) where documented. */
typedef struct {
  void* ptr;
  int64_t stride_row;
  int64_t stride_tok;
  int64_t stride_head;
} sdv2_view;

int sdv2_abi_version(void);
const char* sdv2_strerror(int code);
/* cudaError_t of the most recent failing CUDA call made by this thread through the library. */
int sdv2_last_cuda_error(void);

/*
 * Fused 3D rotary embedding + K/V slot write.
 *
 * Replaces, per call of reference CausalWanSelfAttention.forward (models/wan/causal_model.py):
 *   causal_rope_apply on q and k ............ :253-266 (-> :94-108, multiplier :57-73)
 *   the K/V slice assignments ............... :321-322 and :336-337
 *   the four index fill_ calls per row ...... :303-304, :341-342
 * The slot positions themselves (dst_begin) come from the caller's integer mirror of :279-342.
 *
 * For every row b, token t (ordered frame-major over grid_f x grid_h x grid_w), head h:
 *   q_out[b,t,h,:]                 = rope(q[b,t,h,:])
 *   k_cache[b, dst_begin[b]+t,h,:] = rope(k[b,t,h,:])
 *   v_cache[b, dst_begin[b]+t,h,:] = v[b,t,h,:]
 * rope multiplies pair (2j,2j+1) of the head dim, as a complex number, by
 * rope_table_dev[row_j][j] where row_j = start_frame[b]+frame(t) for the first
 * half-2*(half/3) pairs, grid row of t for the next half/3 and grid column for the last half/3
 * (half = head_dim/2). Arithmetic is IEEE double with separately rounded products
 * (re = a*c - b*d, im = a*d + b*c), then rounded to float and, for bf16 storage, rounded again
 * to bf16: bit-identical to the reference's complex128 path on CPU.
 *
 * rope_table_dev: device, double [table_rows][head_dim/2][2] (re, im) = the reference's
 *   model.freqs (models/wan/causal_model.py:631-638) viewed as real.
 * start_frame, dst_begin: host int64[rows].
 * global_end_dev/local_end_dev: device int64[rows] index tensors of the cache dict, or NULL; when
 *   given, global_end_val/local_end_val (host int64[rows]) are stored into them by the kernel.
 * status_dev: optional device int (NULL to skip); written only if a bounded device-side wait of
 *   the staging pipeline runs out, in the format sdv2_read_status decodes. The attention
 *   workspace's first word may be passed.
 * q_out, k_cache and v_cache must not overlap q, k or v.
 */
int sdv2_rope_kv_append(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v,
                        const sdv2_view* q_out, const sdv2_view* k_cache, const sdv2_view* v_cache,
                        int rows, int new_tokens, int heads, int head_dim, int64_t cache_tokens,
                        const double* rope_table_dev, int table_rows,
                        int grid_f, int grid_h, int grid_w,
                        const int64_t* start_frame, const int64_t* dst_begin,
                        int64_t* global_end_dev, int64_t* local_end_dev,
                        const int64_t* global_end_val, const int64_t* local_end_val,
                        int dtype, int* status_dev, void* stream);

/*
 * Same operation with the per-row slot parameters in device memory, for launches that must not
 * carry per-step values - a launch recorded in a CUDA graph is replayed with the values the host
 * wrote into the array since.  No reference counterpart (the reference passes Python ints).
 *
 * step_params_dev: device int64 [4][rows], 8-byte aligned: start_frame | dst_begin |
 *   global_end value | local_end value, read by the kernel when it runs.  The host cannot check
 *   them, so the kernel does: if a slot would leave the cache or a frame the rope table, the
 *   launch writes nothing and records that in *status_dev, and sdv2_read_status then returns
 *   SDV2_ERR_INVALID_ARG.  The caller orders its update of the array before the launch (same
 *   stream) and must not overwrite it while a launch that reads it is still pending.
 * Everything else as for sdv2_rope_kv_append.
 */
int sdv2_rope_kv_append_indirect(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v,
                                 const sdv2_view* q_out, const sdv2_view* k_cache, const sdv2_view* v_cache,
                                 int rows, int new_tokens, int heads, int head_dim, int64_t cache_tokens,
                                 const double* rope_table_dev, int table_rows,
                                 int grid_f, int grid_h, int grid_w,
                                 const int64_t* step_params_dev,
                                 int64_t* global_end_dev, int64_t* local_end_dev,
                                 int dtype, int* status_dev, void* stream);

/*
 * The same operation with the RMS norm of q and k folded in: q and k arrive as the raw outputs of
 * their projections (slices of one fused q|k|v projection are fine: only head_dim and the heads of
 * a token must be contiguous) and are normalised over the whole token row of heads * head_dim
 * elements before the rope,
 *   x_n = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * weight)
 * which is WanRMSNorm.forward (models/wan/wan_base/modules/model.py:70-86) as applied to the q and k
 * projections at models/wan/causal_model.py:212-214, with the same intermediate roundings; the row
 * statistics are summed in the order sdv2_rmsnorm uses, so the result equals sdv2_rmsnorm followed
 * by sdv2_rope_kv_append bit for bit.  v is copied as it is.
 * bf16 tensors only; heads * head_dim <= 8192; heads of a token back to back (stride_head ==
 * head_dim) - otherwise SDV2_ERR_UNSUPPORTED_SHAPE, and the caller runs sdv2_rmsnorm first.
 * norm_q_weight_dev / norm_k_weight_dev: device bf16 [heads * head_dim], 16-byte aligned.
 * Slot parameters: either the host arrays start_frame / dst_begin (+ global_end_val / local_end_val)
 * with step_params_dev NULL, or step_params_dev (device int64 [4][rows], as for
 * sdv2_rope_kv_append_indirect) with the host arrays NULL.
 */
int sdv2_norm_rope_kv_append(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v,
                             const sdv2_view* q_out, const sdv2_view* k_cache, const sdv2_view* v_cache,
                             int rows, int new_tokens, int heads, int head_dim, int64_t cache_tokens,
                             const double* rope_table_dev, int table_rows,
                             int grid_f, int grid_h, int grid_w,
                             const int64_t* start_frame, const int64_t* dst_begin,
                             const int64_t* step_params_dev,
                             int64_t* global_end_dev, int64_t* local_end_dev,
                             const int64_t* global_end_val, const int64_t* local_end_val,
                             const void* norm_q_weight_dev, const void* norm_k_weight_dev, float norm_eps,
                             int* status_dev, void* stream);

/*
 * Per-frame means for the adaptive sink test: for every cache row, the mean over the tokens of each of
 * the first sink_frames frames of the K and V cache and of the new frame's roped K and V
 * (k_new / v_new: [rows, frame_tokens, heads, head_dim]) - the four `.mean(1)` reductions of
 * models/wan/causal_model.py:286-293 for all rows in two launches, without the reshaped copies.
 * means_dev: out, [rows][sink_frames + 1][2 (K, V)][heads * head_dim] in the tensors' type (fp32 sums,
 * scaled by 1 / frame_tokens, rounded once); entry sink_frames is the new frame.
 * scratch_dev: at least sdv2_frame_means_scratch_bytes() bytes, 16-byte aligned, no initialisation needed.
 * The heads of a token must be back to back (stride_head == head_dim).
 */
int sdv2_frame_means(const sdv2_view* k_cache, const sdv2_view* v_cache, const sdv2_view* k_new,
                     const sdv2_view* v_new, int rows, int sink_frames, int frame_tokens, int heads, int head_dim,
                     int64_t cache_tokens, int dtype, void* means_dev, void* scratch_dev, size_t scratch_bytes,
                     void* stream);
size_t sdv2_frame_means_scratch_bytes(int rows, int sink_frames, int heads, int head_dim);

/*
 * Data-dependent half of the sink + ring slot logic, on the device, for the adaptive sink refresh
 * (models/wan/causal_model.py:284-299 for the test, :302-337 for the queue): one launch per layer
 * decides for every cache row whether a sink frame is refreshed, updates the row's evict queue and
 * writes the parameter array that sdv2_rope_kv_append_indirect reads, so that no similarity, queue
 * entry or slot is ever read back by the host.
 *
 * sim_dev: device [rows][sink_frames], bf16 or f32 (sim_dtype): (cos(K sink mean, K new mean) +
 *   cos(V sink mean, V new mean)) / 2 as the caller computed it; NULL or sink_frames == 0: no test.
 *   A row whose smallest entry is below `threshold` (compared in sim_dtype, first minimum wins) gets
 *   (argmin + 1) * frame_tokens pushed at the head of its queue.
 * queue_dev: device int64 [rows][1 + queue_cap]: length, then the entries; updated in place.
 * host_inputs / host_inputs_dev: the data-independent inputs, int64 [7][rows] - start frame | global
 *   end value | local end value | evict branch (0/1) | pop the head (0/1) | rolling end to register or
 *   -1 | slot of the append branch - on the host (copied into the launch) or on the device (read when
 *   the kernel runs: for launches recorded in a CUDA graph); exactly one of the two is given.
 * step_params_dev: out, device int64 [4][rows]: start frame | slot | global end | local end.
 * An empty queue in the evict branch (the reference raises there) or a queue overflow writes slot -1,
 * which the append kernel refuses, and reports through *status_dev (sdv2_read_status answers
 * SDV2_ERR_INVALID_ARG).
 */
int sdv2_ring_plan_adaptive(const void* sim_dev, int sim_dtype, int rows, int sink_frames, float threshold,
                            int64_t* queue_dev, int queue_cap, int64_t frame_tokens, int64_t new_tokens,
                            const int64_t* host_inputs, const int64_t* host_inputs_dev,
                            int64_t* step_params_dev, int* status_dev, void* stream);

/*
 * Attention of the new queries over the wrapped cache: out[b] = softmax(q[b] k[b,:L_b]^T * scale)
 * v[b,:L_b] with L_b = seq_lens[b], no causal or window mask (the window is the cache content).
 *
 * Replaces flash_attn_interface.flash_attn_with_kvcache(q, k_cache, v_cache, cache_seqlens) at
 * models/wan/causal_model.py:353-358 and its fallback attention_with_kvcache_fallback (:111-157).
 *
 * bf16 in, fp32 accumulate, bf16 out; head_dim must be 128. tcgen05 tensor-core kernel with
 * TMA-staged K/V tiles. seq_lens: host int32[rows], 1 <= seq_lens[b] <= cache_tokens.
 * workspace_dev: at least sdv2_attn_workspace_bytes() bytes, 256-byte aligned; its first word is
 * a status flag written only when a bounded device-side wait runs out (read with sdv2_read_status;
 * zero it once after allocation).
 * Cache rows at and beyond seq_lens[b] are never attended and may hold anything (uninitialised
 * memory, NaN): their scores are masked and their V rows are cleared on chip before use, like
 * flash_attn_with_kvcache's handling of rows past cache_seqlens.
 */
int sdv2_attn_kvcache(const sdv2_view* q, const sdv2_view* k_cache, const sdv2_view* v_cache,
                      const sdv2_view* out, int rows, int q_tokens, int heads, int head_dim,
                      int64_t cache_tokens, const int32_t* seq_lens, float softmax_scale,
                      void* workspace_dev, size_t workspace_bytes, void* stream);

size_t sdv2_attn_workspace_bytes(int rows, int q_tokens, int heads, int head_dim);

/* Partial-result slots (133,120 bytes each, after the 256-byte status block) that the attention
 * launch for this problem writes on a device with `sm_count` multiprocessors: 0 when the grid
 * fills whole waves or the key range is short, never more than 192.  min_seq_len = the smallest
 * seq_lens[b].  Pure host arithmetic (no CUDA call); no reference counterpart. */
int sdv2_attn_partial_slots(int rows, int q_tokens, int heads, int min_seq_len, int sm_count);

/*
 * Text cross-attention core: every query attends all kv_tokens context slots, no mask.
 * Replaces flash_attention(q, k, v, k_lens=None) as called from WanT2VCrossAttention.forward
 * (models/wan/wan_base/modules/model.py:189 -> models/wan/wan_base/modules/attention.py:138-261),
 * reading K/V straight from crossattn_cache["k"/"v"]; k/v stride_row may be 0 (the reference
 * expands one row over the batch, models/wan/causal_stream_inference.py:227-228).
 */
int sdv2_cross_attn(const sdv2_view* q, const sdv2_view* k, const sdv2_view* v, const sdv2_view* out,
                    int rows, int q_tokens, int heads, int head_dim, int kv_tokens,
                    float softmax_scale, void* workspace_dev, size_t workspace_bytes, void* stream);

/*
 * Same contraction as sdv2_attn_kvcache on CUDA cores (one warp per query row, fp32 math), for
 * bf16 or fp32 tensors. It exists to check the tensor-core kernel on the device at sizes where a
 * CPU check takes minutes, and to serve fp32 caches (the reference's CPU configuration uses fp32,
 * models/wan/causal_model.py:115-120). out has q's dtype.
 */
int sdv2_attn_kvcache_simt(const sdv2_view* q, const sdv2_view* k_cache, const sdv2_view* v_cache,
                           const sdv2_view* out, int rows, int q_tokens, int heads, int head_dim,
                           int64_t cache_tokens, const int32_t* seq_lens, float softmax_scale,
                           int dtype, void* stream);

/*
 * sdv2_attn_kvcache without a caller-provided workspace.  No counterpart in the reference (which
 * lets PyTorch allocate whatever its kernels need): this entry point exists for hosts that cannot
 * give the library scratch memory - embedders that only hold borrowed tensor pointers, workers
 * whose device memory was fully partitioned at start-up, loops where a cudaMalloc in the per-chunk
 * path would serialise the GPU.  The status block and the partial results of the split tail tiles
 * live in a device array built into the library (24.4 MiB per GPU, 192 partial slots).
 *
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - The first call on each device looks up the array's device address (a host-side query: nothing
 *    is launched or synchronised).  Make that first call before any stream capture starts.
 *  - The array always suffices: the kernel's tail split is lowered until it fits 192 partial slots
 *    (see sdv2_attn_partial_slots), so no shape is refused for lack of scratch; SDV2_ERR_WORKSPACE is
 *    kept as a defensive check only.  rows > SDV2_MAX_ROWS is refused with SDV2_ERR_UNSUPPORTED_SHAPE.
 *  - All calls on a device share the array and it keeps the previous call's contents (every slot is
 *    rewritten before it is read; the status block starts as zeros and is cleared by
 *    sdv2_read_status).  Calls that overlap on the GPU race on it: order them.
 *  - status_dev_out (optional) receives the device address of the status block, valid for
 *    sdv2_read_status.
 * Results are identical to sdv2_attn_kvcache on the same inputs.
 */
int sdv2_attn_kvcache_static(const sdv2_view* q, const sdv2_view* k_cache, const sdv2_view* v_cache,
                             const sdv2_view* out, int rows, int q_tokens, int heads, int head_dim,
                             int64_t cache_tokens, const int32_t* seq_lens, float softmax_scale,
                             void** status_dev_out, void* stream);

/*
 * Fused element-wise steps directly around the attention path of a DiT block (bf16 tensors, fp32
 * statistics).  Each reproduces the intermediate bf16 roundings of the reference's op chain.
 *
 * sdv2_rmsnorm: out[r,:] = bf16(bf16(x[r,:] * rsqrt(mean(x[r,:]^2) + eps)) * weight) - WanRMSNorm.forward
 *   (models/wan/wan_base/modules/model.py:70-86) applied to the q / k projections
 *   (models/wan/causal_model.py:212-214).  Row strides in elements (a slice of a fused projection is fine).
 * sdv2_ln_modulate: out = bf16(bf16(bf16(LayerNorm(x)) * bf16(1 + scale[b,f])) + shift[b,f]) for x [batch,
 *   frames * tokens_per_frame, dim] - the adaLN modulation in front of self-attention and the FFN
 *   (models/wan/causal_model.py:463-467, 477-480).  scale / shift point at the first row of their
 *   chunk of the [batch, frames, 6, dim] modulation tensor; row (b * frames + f) starts
 *   mod_row_stride elements after the previous one (6 * dim in place, dim if copied out).
 * sdv2_gate_residual: out = bf16(x + bf16(y * gate[b,f])) - the gated residual after them
 *   (models/wan/causal_model.py:470-471, 482-483); gate addressed like scale.  out may alias x.
 * sdv2_layernorm_affine: out[r,:] = bf16(weight * ((x[r,:] - mean) * rstd) + bias) in fp32 - torch.nn.LayerNorm
 *   with elementwise_affine on bf16 tensors, the block's norm3 in front of the text cross-attention
 *   (models/wan/causal_model.py:473-476; WanLayerNorm, models/wan/wan_base/modules/model.py:89-100);
 *   x, out contiguous [n_rows, dim], dim at most 5120.
 * sdv2_residual_layernorm: x_out = bf16(x + bf16(y * gate[b,f])) (gate null: bf16(x + y)), then out = the
 *   modulated LayerNorm (affine = 0: mul / add are scale / shift addressed like sdv2_ln_modulate's) or the affine
 *   LayerNorm (affine = 1: mul / add are weight / bias) of x_out, in one pass over the rows: the residual
 *   addition after self-attention together with norm3 (models/wan/causal_model.py:470-476), and the one
 *   after the text cross-attention together with norm2 and its modulation (:473-480).  Bit for bit the
 *   result of sdv2_gate_residual (or a bf16 addition) followed by sdv2_layernorm_affine / sdv2_ln_modulate.
 *   x_out may alias x; dim at most 5120.
 * sdv2_gelu_tanh: out = bf16(gelu(x)) with the tanh approximation (torch.nn.GELU(approximate="tanh"), the
 *   activation between the block's two FFN projections, models/wan/causal_model.py:424-427), n bf16 elements
 *   (a multiple of 8); out may alias x.  Evaluated as x * sigmoid(2u), which equals 0.5 x (1 + tanh(u)); for
 *   x > -2.9 the rounded results are the op chain's (isolated single-step differences); below that the chain's
 *   1 + tanh(u) cancels and its fp32 results are off by up to 3e-7, which is whole bf16 steps of values that
 *   small, while this form stays within rounding of the exact function.
 * dim must be a multiple of 8 and at most 8192; all pointers 16-byte aligned.
 */
int sdv2_rmsnorm(const void* x, int64_t x_row_stride, const void* weight, void* out, int64_t out_row_stride,
                 int64_t n_rows, int dim, float eps, void* stream);
int sdv2_ln_modulate(const void* x, const void* scale, const void* shift, int64_t mod_row_stride, void* out,
                     int batch, int frames, int tokens_per_frame, int dim, float eps, void* stream);
int sdv2_gate_residual(const void* x, const void* y, const void* gate, int64_t mod_row_stride, void* out, int batch,
                       int frames, int tokens_per_frame, int dim, void* stream);
int sdv2_layernorm_affine(const void* x, const void* weight, const void* bias, void* out, int64_t n_rows, int dim,
                          float eps, void* stream);
int sdv2_gelu_tanh(const void* x, void* out, int64_t n, void* stream);
int sdv2_residual_layernorm(const void* x, const void* y, const void* gate, int64_t gate_row_stride, void* x_out,
                            int affine, const void* mul, const void* add, int64_t mod_row_stride, void* out,
                            int batch, int frames, int tokens_per_frame, int dim, float eps, void* stream);

/* Synchronises `stream`, reads the status word at the start of a workspace and clears it.
 * Returns SDV2_OK, SDV2_ERR_TIMEOUT (a device-side wait ran out; *detail = where),
 * SDV2_ERR_INVALID_ARG (device-resident slot parameters were out of range; nothing was written) or
 * SDV2_ERR_CUDA. */
int sdv2_read_status(void* workspace_dev, int* detail, void* stream);

/*
 * Device self-test of the two tensor-core contractions the attention kernel is built from:
 *   s_out[128][128] = a[128][128] * b[128][128]^T      (both operands K-major in shared memory)
 *   o_out[128][128] = p[128][128] * v[128][128]        (p from tensor memory, v MN-major)
 * a, b, p, v: device bf16 row-major; s_out, o_out: device float row-major. No reference
 * counterpart; used by the tests to localise a failure.
 */
int sdv2_selftest_umma(const void* a_dev, const void* b_dev, const void* p_dev, const void* v_dev,
                       float* s_out_dev, float* o_out_dev, int* status_dev, void* stream);

/*
 * Device self-test of the bounded waits: one thread block waits on an on-chip barrier that nothing
 * ever completes, gives up after `budget_cycles` SM clock cycles (clamped to [1e4, 2e9]), records
 * the site in *status_dev and returns normally - the context stays usable.  A following
 * sdv2_read_status(status_dev, ...) must answer SDV2_ERR_TIMEOUT with site 7 (probe) in the low
 * byte of *detail.  This is how the error path of every wait in the attention and append kernels
 * (same wait routine, budget 1.5e9 cycles) is exercised without hanging or faulting a GPU.
 * No reference counterpart (the reference's communication_timeout,
 * streamv2v/communication/data_containers.py:77, is never read).
 */
int sdv2_selftest_wait_timeout(int* status_dev, long long budget_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SDV2_H_ */

// Device side of the sink + ring slot logic for the adaptive sink refresh.
//
// The reference tests, per cache row and per layer, how similar the new frame's mean K / V are to
// those of every sink frame and, when the least similar one falls below a threshold, pushes that
// sink frame's slot at the FRONT of the row's evict queue (models/wan/causal_model.py:284-299), so
// the queue - and with it the slot the new K/V go to - depends on the data.  Deciding that on the
// host costs a device read-back per row per layer.  Here the queue lives in device memory and one
// small launch per layer does the data-dependent half of the slot logic for all rows:
//
//   front   = (argmin_s sim[row][s] + 1) * frame_tokens   if min_s sim[row][s] < threshold
//   queue   : insert front at the head; evict branch: slot = queue[0] - new_tokens, pop the head when
//             the host says so and re-append it if it lies beyond the sink; append branch: register
//             the rolling end unless it is already the tail (causal_model.py:302-337)
//   output  : the [4][rows] parameter array sdv2_rope_kv_append_indirect reads (start frame | slot |
//             global end | local end)
//
// Everything that does not depend on the data (which branch, whether the head is popped, the
// rolling end, both index values) is computed by the host and handed in, by value or - for launches
// recorded in a CUDA graph - through a device array.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "sdv2_internal.h"

namespace sdv2 {

__device__ __forceinline__ float sim_value(const void* sim, int dtype, int idx) {
  return dtype == SDV2_DTYPE_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(sim)[idx])
                                  : static_cast<const float*>(sim)[idx];
}

__global__ void __launch_bounds__(64) ring_plan_kernel(const __grid_constant__ RingPlanParams p) {
  const int row = threadIdx.x;
  if (row >= p.rows) return;
  const int64_t* in = p.host_dev;  // [kRingPlanInputs][rows] when given, else the by-value copy
  auto input = [&](int which) { return in != nullptr ? in[which * p.rows + row] : p.host_val[which][row]; };
  const int64_t start_frame = input(0), global_end = input(1), local_end = input(2);
  const bool evict = input(3) != 0, pop = input(4) != 0;
  const int64_t push_value = input(5), append_begin = input(6);

  int64_t* q = p.queue + static_cast<int64_t>(row) * (1 + p.queue_cap);
  int64_t len = q[0];
  bool bad = len < 0 || len > p.queue_cap;

  // adaptive test: the comparison runs in the similarities' own type, as a tensor-vs-scalar compare does
  int64_t front = -1;
  if (p.sim != nullptr && p.sink_frames > 0) {
    float lo = sim_value(p.sim, p.dtype, row * p.sink_frames);
    int arg = 0;
    for (int s = 1; s < p.sink_frames; ++s) {
      const float v = sim_value(p.sim, p.dtype, row * p.sink_frames + s);
      if (v < lo) {  // first minimum wins, NaN never does
        lo = v;
        arg = s;
      }
    }
    const float thr = p.dtype == SDV2_DTYPE_BF16 ? __bfloat162float(__float2bfloat16_rn(p.threshold)) : p.threshold;
    if (lo < thr) front = static_cast<int64_t>(arg + 1) * p.frame_tokens;
  }
  if (!bad && front >= 0) {
    if (len >= p.queue_cap) {
      bad = true;
    } else {
      for (int64_t i = len; i > 0; --i) q[1 + i] = q[i];
      q[1] = front;
      ++len;
    }
  }
  int64_t slot = -1;
  if (!bad) {
    if (evict) {
      if (len == 0) {
        bad = true;  // the reference raises here (indexing an empty queue)
      } else {
        const int64_t head = q[1];
        slot = head - p.new_tokens;
        if (pop) {
          for (int64_t i = 1; i < len; ++i) q[i] = q[i + 1];
          --len;
          if (head > p.sink_tokens) q[1 + len++] = head;
        }
      }
    } else {
      if (push_value >= 0 && (len == 0 || q[len] != push_value)) {
        if (len >= p.queue_cap) bad = true;
        else q[1 + len++] = push_value;
      }
      slot = append_begin;
    }
  }
  if (bad) {
    slot = -1;  // the append kernel refuses a negative slot and writes nothing
    if (p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(BAD_STEP_PARAMS));
  } else {
    q[0] = len;
  }
  p.step_params[0 * p.rows + row] = start_frame;
  p.step_params[1 * p.rows + row] = slot;
  p.step_params[2 * p.rows + row] = global_end;
  p.step_params[3 * p.rows + row] = local_end;
}

// ------------------------------------------------------------------------------------------
// per-frame means of K and V for the adaptive test: every sink frame of the cache and the new frame
// ------------------------------------------------------------------------------------------
// Pass 1: grid (token chunks, (sink + 1) frames x 2 tensors, rows); a thread owns 16-byte vectors of
// the token row and sums them over its chunk of the frame's tokens in fp32.  Pass 2 adds the chunk
// partials in chunk order (so the result does not depend on scheduling), scales by 1 / tokens and
// rounds to the tensors' type - what a mean over the token dimension of a [frames, tokens, C] tensor
// gives up to the order of the fp32 additions.
template <typename T>
__global__ void __launch_bounds__(256) frame_sum_kernel(const __grid_constant__ FrameMeansParams p) {
  constexpr int kElems = 16 / sizeof(T);
  const int chunk = blockIdx.x, row = blockIdx.z;
  const int frame = blockIdx.y >> 1, tensor = blockIdx.y & 1;   // frame == sink_frames: the new frame
  const bool is_new = frame == p.sink_frames;
  const sdv2_view& vw = is_new ? (tensor ? p.v_new : p.k_new) : (tensor ? p.v_cache : p.k_cache);
  const int t0 = static_cast<int>(static_cast<int64_t>(chunk) * p.frame_tokens / gridDim.x);
  const int t1 = static_cast<int>(static_cast<int64_t>(chunk + 1) * p.frame_tokens / gridDim.x);
  const int64_t tok0 = is_new ? 0 : static_cast<int64_t>(frame) * p.frame_tokens;
  const T* base = static_cast<const T*>(vw.ptr) + row * vw.stride_row + tok0 * vw.stride_tok;
  const int row_vecs = p.row_elems / kElems;
  float* out = p.partial + ((static_cast<size_t>(row) * (p.sink_frames + 1) + frame) * 2 + tensor) * gridDim.x * p.row_elems +
               static_cast<size_t>(chunk) * p.row_elems;
  for (int c = threadIdx.x; c < row_vecs; c += blockDim.x) {
    float acc[kElems];
#pragma unroll
    for (int i = 0; i < kElems; ++i) acc[i] = 0.f;
    for (int t = t0; t < t1; ++t) {
      const uint4 v = *reinterpret_cast<const uint4*>(base + t * vw.stride_tok + c * kElems);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      if (sizeof(T) == 2) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] += __uint_as_float(w[i] << 16);
          acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] += __uint_as_float(w[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < kElems; ++i) out[c * kElems + i] = acc[i];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) frame_mean_kernel(const __grid_constant__ FrameMeansParams p) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= p.row_elems) return;
  const size_t item = (static_cast<size_t>(blockIdx.z) * (p.sink_frames + 1) + (blockIdx.y >> 1)) * 2 + (blockIdx.y & 1);
  const float* part = p.partial + item * p.chunks * p.row_elems + e;
  float s = 0.f;
  for (int c = 0; c < p.chunks; ++c) s += part[static_cast<size_t>(c) * p.row_elems];
  const float m = s * (1.0f / static_cast<float>(p.frame_tokens));
  T* out = static_cast<T*>(p.means) + item * p.row_elems + e;
  if (sizeof(T) == 2) *reinterpret_cast<__nv_bfloat16*>(out) = __float2bfloat16_rn(m);
  else *reinterpret_cast<float*>(out) = m;
}

cudaError_t launch_frame_means(const FrameMeansParams& p, cudaStream_t stream) {
  const dim3 g1(p.chunks, (p.sink_frames + 1) * 2, p.rows), g2((p.row_elems + 255) / 256, (p.sink_frames + 1) * 2, p.rows);
  if (p.dtype == SDV2_DTYPE_BF16) {
    frame_sum_kernel<__nv_bfloat16><<<g1, 256, 0, stream>>>(p);
    frame_mean_kernel<__nv_bfloat16><<<g2, 256, 0, stream>>>(p);
  } else {
    frame_sum_kernel<float><<<g1, 256, 0, stream>>>(p);
    frame_mean_kernel<float><<<g2, 256, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

cudaError_t launch_ring_plan(const RingPlanParams& p, cudaStream_t stream) {
  ring_plan_kernel<<<1, 64, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace sdv2

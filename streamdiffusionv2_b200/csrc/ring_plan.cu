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

cudaError_t launch_ring_plan(const RingPlanParams& p, cudaStream_t stream) {
  ring_plan_kernel<<<1, 64, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace sdv2

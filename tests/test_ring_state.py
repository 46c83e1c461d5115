"""The host-integer slot mirror used by the product path, against index traces recorded from the
reference at 1560 tokens per latent frame, driven through cache dicts with CPU index tensors."""
import pytest
import torch

import cases
from streamdiffusionv2_b200.ring_state import RingState


class _Mod:
    def __init__(self, sink):
        self.sink_size, self.adapt_sink_thr, self.evict_idx = sink, -1, None


@pytest.mark.parametrize("name", sorted(cases.TRACE_CASES))
def test_ring_state_follows_reference_trace(name):
    case = cases.TRACE_CASES[name]
    trace = cases.load_traces()[name]
    h, w = case["grid_hw"]
    fs = h * w
    smax = case["cache_frames"] * fs
    kv = {"k": torch.empty(1, smax, 1, 0), "v": torch.empty(1, smax, 1, 0),
          "global_end_index": torch.tensor([0]), "local_end_index": torch.tensor([0]),
          "total_steps": case["total_steps"], "current_step": case["total_steps"]}
    mod = _Mod(case["sink_size"])
    i = 0
    for call in cases.schedule(case):
        if call["op"] == "replicate":
            b = call["rows"]
            kv["k"] = kv["k"].repeat(b, 1, 1, 1)
            kv["v"] = kv["v"].repeat(b, 1, 1, 1)
            kv["global_end_index"] = kv["global_end_index"].repeat(b)
            kv["local_end_index"] = kv["local_end_index"].repeat(b)
            continue
        st = RingState.of(kv)
        n_new = call["frames"] * fs
        dst, sl = st.plan(kv, mod, call["starts"], n_new, fs)
        # what the append kernel does with the values it is handed
        kv["global_end_index"].data[:] = torch.tensor(st.global_end)
        kv["local_end_index"].data[:] = torch.tensor(st.local_end)
        g = trace[i]
        assert st.global_end == g["global_end"] and st.local_end == g["local_end"], (name, i)
        assert mod.evict_idx == g["evict_idx"], (name, i)
        assert kv["current_step"] == g["current_step"], (name, i)
        assert sl == g["local_end"]
        assert all(0 <= d and d + n_new <= smax for d in dst)
        i += 1
    assert i == len(trace)


def test_slot_outside_cache_raises():
    kv = {"k": torch.empty(1, 24, 1, 0), "v": torch.empty(1, 24, 1, 0),
          "global_end_index": torch.tensor([24]), "local_end_index": torch.tensor([24]),
          "total_steps": 1, "current_step": 1}
    mod = _Mod(0)
    mod.evict_idx = [[6]]          # a queue entry smaller than the chunk: slot would start at -6
    with pytest.raises(RuntimeError, match="outside"):
        RingState.of(kv).plan(kv, mod, [24], 12, 6)

"""Replay of a steady-state chunk step from a CUDA graph.

Once every cache row has wrapped, a chunk step launches the same kernels with the same shapes and
the same attention lengths every time; the only values that change are each row's rope start frame,
its ring slot and the two index values the append kernel stores.  Those are read by the kernel from
a small device array (`ops.rope_kv_append(step_params=...)`), so the whole DiT forward of a step
(~500 launches for 30 blocks) is recorded once and replayed with a single launch, after one
host->device copy of that array.  The host slot state is still advanced layer by layer with the
same `RingState.plan` calls the eager path makes, so cache dicts, evict queues and host mirrors
end up exactly as without graphs, and any step that does not match the recorded one (a row that
has not wrapped yet, another shape, the adaptive sink test) simply runs eagerly.

The reference has no counterpart: it launches every op from Python each step and reads device
indices back in between (models/wan/causal_model.py:279-342).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from . import causal_attention as CA
from . import ops
from .ring_state import RingState

_PINNED_SLOTS = 4
# per layer and row: 4 values the append kernel reads, 7 inputs of the adaptive plan kernel, 4 values for the
# append launch that ropes into the staging chunk in front of the adaptive test (start frame, slot 0, unused)
_STEP, _PLAN, _STAGE = 4, 7, 4
_ALL = _STEP + _PLAN + _STAGE


class _Recorder:
    """Active while a forward is being captured: hands every layer its slice of the parameter
    array and notes which (attention module, cache dict) pairs ran, in order."""

    def __init__(self, params_dev: torch.Tensor, host: torch.Tensor):
        self.params_dev, self.host = params_dev, host
        self.layers: List[Tuple[object, dict]] = []
        self.seq_lens: Optional[List[int]] = None
        self.n_new = self.frame_tokens = 0

    def layer_params(self, attn_module, kv_cache, start_frames, dst, state: RingState, seq_lens, n_new, frame_tokens):
        i = len(self.layers)
        if i >= self.params_dev.shape[0]:
            raise RuntimeError("more attention layers ran than the graph was sized for")
        if self.seq_lens is None:
            self.seq_lens, self.n_new, self.frame_tokens = list(seq_lens), n_new, frame_tokens
        elif list(seq_lens) != self.seq_lens:
            raise RuntimeError("layers disagree on the attention lengths; step cannot be recorded")
        self.layers.append((attn_module, kv_cache, False))
        rows = len(dst)
        self.host[i, :_STEP] = torch.tensor([start_frames, dst, state.global_end[:rows], state.local_end[:rows]],
                                            dtype=torch.int64)
        return self.params_dev[i, :_STEP]

    def adaptive_layer_params(self, attn_module, kv_cache, inputs, seq_lens, n_new, frame_tokens):
        """A layer with the adaptive sink test: its slots are decided on the device by the plan kernel,
        which reads the data-independent inputs from this layer's slice of the parameter array and
        writes the four values the append kernel reads into the slice in front of it; the append
        launch that ropes the new frame into the staging chunk reads its start frames from a third
        slice.  Returns (step_params, keyword for the plan kernel, staging step_params)."""
        i = len(self.layers)
        if i >= self.params_dev.shape[0]:
            raise RuntimeError("more attention layers ran than the graph was sized for")
        if self.seq_lens is None:
            self.seq_lens, self.n_new, self.frame_tokens = list(seq_lens), n_new, frame_tokens
        elif list(seq_lens) != self.seq_lens:
            raise RuntimeError("layers disagree on the attention lengths; step cannot be recorded")
        self.layers.append((attn_module, kv_cache, True))
        rows = len(inputs[0])
        self.host[i, _STEP:_STEP + _PLAN] = torch.tensor(inputs, dtype=torch.int64)
        self.host[i, _STEP + _PLAN:] = torch.tensor([inputs[0], [0] * rows, [0] * rows, [0] * rows], dtype=torch.int64)
        return (self.params_dev[i, :_STEP], {"host_inputs_dev": self.params_dev[i, _STEP:_STEP + _PLAN]},
                self.params_dev[i, _STEP + _PLAN:])


class _Recorded:
    __slots__ = ("graph", "layers", "seq_lens", "n_new", "frame_tokens", "outputs", "launch_counts", "launch_work",
                 "pointers")


def _cache_pointers(layers: Sequence[tuple]) -> List[int]:
    """Addresses a recorded step has baked in for these layers: (attention module, kv_cache dict) or
    (attention module, kv_cache dict, crossattn_cache dict) per layer."""
    out: List[int] = []
    for entry in layers:
        kv = entry[1]
        if kv is not None:            # None: a block of which only the cross-attention half runs here
            out += [kv["k"].data_ptr(), kv["v"].data_ptr(), kv["global_end_index"].data_ptr(),
                    kv["local_end_index"].data_ptr()]
        if len(entry) > 2 and entry[2] is not None and entry[2].get("is_init"):
            out += [entry[2]["k"].data_ptr(), entry[2]["v"].data_ptr()]
    return out


class StepGraphs:
    """Per-pipeline cache of recorded steps, keyed by what the caller says distinguishes them
    (entry point, block range, shapes)."""

    def __init__(self, device: torch.device, max_layers: int, rows: int):
        self.device = torch.device(device)
        self.rows = rows
        self.params_dev = torch.zeros((max_layers, _ALL, rows), dtype=torch.int64, device=self.device)
        self._pinned = [torch.zeros((max_layers, _ALL, rows), dtype=torch.int64).pin_memory()
                        for _ in range(_PINNED_SLOTS)]
        self._pinned_done: List[Optional[torch.cuda.Event]] = [None] * _PINNED_SLOTS
        self._turn = 0
        self._graphs: Dict[tuple, _Recorded] = {}
        self.replays = 0
        self.eager_steps = 0

    def forget(self) -> None:
        """Drop every recording (their block ranges or tensors are no longer the pipeline's)."""
        self._graphs.clear()

    # ------------------------------------------------------------------ host side of a step
    @staticmethod
    def steady(layers: Sequence[tuple], starts: Sequence[int], n_new: int) -> bool:
        """True when every row of every layer takes the wrapped-cache branch of the slot logic,
        i.e. attends the whole cache (causal_model.py:301-322), and (where the layer's crossattn_cache
        is given as a third entry) the text K/V are cached, so that the step launches exactly what a
        recorded one launched.  Layers with the adaptive sink test qualify too: their data-dependent
        slot choice runs on the device, inside the recording.  Nothing is modified."""
        for entry in layers:
            module, kv = entry[0], entry[1]
            if len(entry) > 2 and entry[2] is not None and not entry[2].get("is_init", False):
                return False
            if kv is None:
                continue
            st = RingState.of(kv)
            smax = kv["k"].shape[1]
            for i, cs in enumerate(starts):
                if not (int(cs) + n_new > smax or st.local_end[i] >= smax):
                    return False
        return True

    def _stage_params(self, rec: _Recorded, starts: Sequence[int]) -> None:
        """Advance every layer's slot state by one chunk (as the eager forward would) and send
        the resulting parameters to the device array, ordered before the replay."""
        slot = self._turn % _PINNED_SLOTS
        self._turn += 1
        done = self._pinned_done[slot]
        if done is not None:
            done.synchronize()                 # the copy that last read this staging buffer
        host = self._pinned[slot]
        ft = rec.frame_tokens
        start_frames = [int(s) // ft for s in starts]
        rows = len(starts)
        flat: List[List[int]] = []
        zeros4, zeros11, zeros3 = [0] * (_STEP * rows), [0] * ((_PLAN + _STAGE) * rows), [0] * (3 * rows)
        for module, kv, adaptive in rec.layers:
            st = RingState.of(kv)
            if adaptive:
                cols = [st.plan_row_split(kv, module, i, int(starts[i]), rec.n_new, ft) for i in range(rows)]
                lens = [c[4] for c in cols]
                flat.append(zeros4 + start_frames + st.global_end[:rows] + lens + [int(c[0]) for c in cols]
                            + [int(c[1]) for c in cols] + [c[2] for c in cols] + [c[3] for c in cols]
                            + start_frames + zeros3)
            else:
                dst, lens = st.plan(kv, module, starts, rec.n_new, ft)
                flat.append(start_frames + dst + st.global_end[:rows] + st.local_end[:rows] + zeros11)
            if lens != rec.seq_lens:
                raise RuntimeError("slot state left the recorded steady state during a replayed step")
        n = len(flat)
        host[:n] = torch.tensor(flat, dtype=torch.int64).view(n, _ALL, rows)
        self.params_dev[:n].copy_(host[:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pinned_done[slot] = ev

    # ------------------------------------------------------------------ record / replay
    def run(self, key: tuple, fn: Callable[[], object], layers_hint: Sequence[Tuple[object, dict]],
            starts: Sequence[int], n_new: int, allow_record: bool = True):
        """Run `fn` (a forward whose tensor arguments all live at fixed addresses) for a chunk whose
        rows start at `starts`: replayed from the graph recorded under `key` when the step is in
        steady state, recorded first if there is none yet, eagerly otherwise.  Recording
        synchronises the device, so a caller with transfers in flight that a peer must complete
        passes allow_record=False until it is quiescent.  Returns fn's result; for a graph step
        these are the graph's own output tensors, overwritten by the next replay."""
        rec = self._graphs.get(key)
        if rec is not None and rec.pointers != _cache_pointers(layers_hint):
            del self._graphs[key]          # somebody replaced a cache tensor: the recording is stale
            rec = None
        if (rec is None and not allow_record) or not self.steady(layers_hint, starts, n_new):
            self.eager_steps += 1
            return fn()
        if rec is None:
            rec = self._record(key, fn, starts)
            rec.pointers = _cache_pointers(layers_hint)
        else:
            self._stage_params(rec, starts)
        rec.graph.replay()
        self.replays += 1
        ops.poll_status(self.device)       # replays bypass the attention forwards, which poll on the eager path
        log = ops.current_launch_log()
        if log is not None:
            for name, c in rec.launch_counts.items():
                log.counts[name] = log.counts.get(name, 0) + c
                log.work[name] = log.work.get(name, 0.0) + rec.launch_work[name]
        return rec.outputs

    def _record(self, key: tuple, fn: Callable[[], object], starts: Sequence[int]) -> _Recorded:
        slot = self._turn % _PINNED_SLOTS
        self._turn += 1
        done = self._pinned_done[slot]
        if done is not None:
            done.synchronize()
        recorder = _Recorder(self.params_dev, self._pinned[slot])
        graph = torch.cuda.CUDAGraph()
        counter = ops.LaunchLog(timed=False)
        outer = ops.current_launch_log()
        ops.set_launch_log(counter)
        CA.set_step_recorder(recorder)
        try:
            # thread_local: other threads (a process group's watchdog) may touch the CUDA API
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                outputs = fn()
        finally:
            CA.set_step_recorder(None)
            ops.set_launch_log(outer)
        if not recorder.layers:
            raise RuntimeError("the recorded forward ran no cached attention layer")
        rec = _Recorded()
        rec.graph, rec.layers, rec.seq_lens = graph, recorder.layers, recorder.seq_lens
        rec.n_new, rec.frame_tokens, rec.outputs = recorder.n_new, recorder.frame_tokens, outputs
        rec.launch_counts, rec.launch_work = dict(counter.counts), dict(counter.work)
        rec.pointers = []
        n = len(rec.layers)
        # the capture pass already advanced the slot state for this step and filled the staging buffer
        self.params_dev[:n].copy_(self._pinned[slot][:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pinned_done[slot] = ev
        self._graphs[key] = rec
        return rec

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


def test_step_graph_steady_state_predicate_matches_the_slot_logic():
    """StepGraphs.steady must say "every row attends the whole cache" exactly when the slot logic
    then takes its wrapped branch for every row, and must not modify any state."""
    import copy

    import torch

    from streamdiffusionv2_b200.ring_state import RingState
    from streamdiffusionv2_b200.step_graph import StepGraphs

    class Mod:
        sink_size, adapt_sink_thr, evict_idx = 1, -1, None

    fs, frames, cache_frames, rows = 6, 2, 7, 2
    n_new, smax = frames * fs, cache_frames * fs
    mod = Mod()
    kv = {"k": torch.zeros(rows, smax, 1, 8), "v": torch.zeros(rows, smax, 1, 8),
          "global_end_index": torch.zeros(rows, dtype=torch.long),
          "local_end_index": torch.zeros(rows, dtype=torch.long), "total_steps": 2, "current_step": 2}
    start, history, seen_steady = 0, [0] * rows, 0
    for step in range(14):
        history = [start] + history[:-1]
        st = RingState.of(kv)
        before = (copy.deepcopy(st.global_end), copy.deepcopy(st.local_end), copy.deepcopy(mod.evict_idx))
        steady = StepGraphs.steady([(mod, kv)], history, n_new)
        assert (st.global_end, st.local_end, mod.evict_idx) == before
        _, lens = st.plan(kv, mod, history, n_new, fs)
        if steady:                                  # a recorded step attends the whole cache in every row
            assert all(le == smax for le in lens), (step, lens)
        elif step > 6:
            assert False, "a stream that has wrapped must be reported steady"
        seen_steady += steady
        start += n_new
    assert seen_steady >= 8
    mod.adapt_sink_thr = 0.5                      # the adaptive sink test runs on the device: it records too
    assert StepGraphs.steady([(mod, kv)], history, n_new)


# ---------------------------------------------------------------------------------------------
# writers that bypass the version counter (collectives)
# ---------------------------------------------------------------------------------------------
import os  # noqa: E402
import socket  # noqa: E402
import traceback  # noqa: E402

import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


class _FakePipeline:
    def __init__(self, kv):
        self.kv_cache1 = [kv]


class _ManagerLike:
    """The part of the reference's KVCacheManager that matters here
    (streamv2v/communication/kv_cache_manager.py:48-86): broadcast the index tensors in place."""

    def __init__(self, kv):
        self.pipeline = _FakePipeline(kv)

    def broadcast_kv_blocks(self, block_indices, donor_rank):
        for bi in block_indices:
            dist.broadcast(self.pipeline.kv_cache1[bi]["global_end_index"], src=donor_rank)
            dist.broadcast(self.pipeline.kv_cache1[bi]["local_end_index"], src=donor_rank)


def _broadcast_worker(rank, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.set_num_threads(1)
        dist.init_process_group("gloo", rank=rank, world_size=2)
        from streamdiffusionv2_b200.causal_attention import watch_cache_manager
        fs, smax, n_new = 6, 42, 12
        kv = {"k": torch.empty(1, smax, 1, 0), "v": torch.empty(1, smax, 1, 0),
              "global_end_index": torch.tensor([0]), "local_end_index": torch.tensor([0]),
              "total_steps": 1, "current_step": 1}
        mod = _Mod(1)
        steps = 2 if rank == 0 else 1          # the donor (rank 0) is one chunk ahead
        for s in range(steps):
            st = RingState.of(kv)
            st.plan(kv, mod, [s * n_new], n_new, fs)
            kv["global_end_index"].data[:] = torch.tensor(st.global_end)
            kv["local_end_index"].data[:] = torch.tensor(st.local_end)
        version = kv["global_end_index"]._version
        mgr = _ManagerLike(kv)
        plain_stale = None
        if rank == 1:
            # without the hook: the collective changes the values, not the version, and the mirror stays stale
            mgr.broadcast_kv_blocks([0], 0)
            assert kv["global_end_index"].tolist() == [24] and kv["global_end_index"]._version == version
            plain_stale = RingState.of(kv).global_end == [12]
            kv["global_end_index"].data[:] = torch.tensor([12])      # put the old values back for the second round
            kv["local_end_index"].data[:] = torch.tensor([12])
        else:
            mgr.broadcast_kv_blocks([0], 0)
        watch_cache_manager(mgr)
        watch_cache_manager(mgr)               # idempotent
        mgr.broadcast_kv_blocks([0], 0)
        st = RingState.of(kv)
        dst, lens = st.plan(kv, mod, [24], n_new, fs)
        q.put((rank, "ok", (plain_stale, st.global_end, dst, lens)))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def test_collective_writes_to_index_tensors_need_and_get_invalidation():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_broadcast_worker, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in procs:
        r = q.get(timeout=120)
        res[r[0]] = r
    for p in procs:
        p.join(30)
    for r in (0, 1):
        assert res[r][1] == "ok", res[r][2]
    plain_stale, ge, dst, lens = res[1][2]
    assert plain_stale is True                 # the failure mode exists: version counters do not see collectives
    # after the hooked broadcast the receiver plans its next chunk from the donor's values
    assert ge == [36] and dst == [24] and lens == [36]
    assert res[0][2][1:] == ([36], [24], [36])


def test_split_slot_logic_equals_the_whole_one_with_adaptive_fronts():
    """With the adaptive sink test the queue is updated on the device and the rest of the slot logic
    on the host.  The two halves together (`plan_row_split` + `queue_step`, the latter being the
    host statement of what the plan kernel does) must equal the reference logic (`plan_row`, pinned
    by the traces above) for any pattern of adaptive insertions."""
    import random
    from oracle import causal_attention_oracle as orc
    rnd = random.Random(3)
    for rows, frames, cache_frames, sink, total in ((2, 1, 6, 3, 2), (1, 1, 6, 3, 2), (3, 1, 8, 2, 3), (2, 1, 9, 1, 2)):
        fs, n_new = 6, frames * 6
        smax = cache_frames * fs
        mk = lambda: {"k": torch.empty(rows, smax, 1, 0), "v": torch.empty(rows, smax, 1, 0),
                      "global_end_index": torch.zeros(rows, dtype=torch.long),
                      "local_end_index": torch.zeros(rows, dtype=torch.long), "total_steps": total, "current_step": total}
        kv_a, kv_b = mk(), mk()
        mod_a, mod_b = _Mod(sink), _Mod(sink)
        st_ref = orc.RingLayerState(smax, rows, total_steps=total, current_step=total)
        orc._ensure_queues(st_ref)
        start, starts = 0, [0] * rows
        for step in range(60):
            if start // fs >= 20:
                start = smax - fs
            starts = [start] + starts[:-1]
            fronts = [((rnd.randrange(sink) + 1) * fs if rnd.random() < 0.3 else None) for _ in range(rows)]
            sa, sb = RingState.of(kv_a), RingState.of(kv_b)
            RingState._ensure_queues(kv_a, mod_a)
            RingState._ensure_queues(kv_b, mod_b)
            for i in range(rows):
                want = sa.plan_row(kv_a, mod_a, i, starts[i], n_new, fs, fronts[i])
                ev, pop, push, begin, le = sb.plan_row_split(kv_b, mod_b, i, starts[i], n_new, fs)
                dst = RingState.queue_step(mod_b.evict_idx[i], fronts[i], ev, pop, push, begin, n_new, sink * fs)
                assert (dst, le) == want, (step, i)
                assert orc.ring_plan_row(st_ref, i, starts[i], n_new, fs, sink, fronts[i]) == want
            assert mod_a.evict_idx == mod_b.evict_idx == st_ref.evict_idx
            assert sa.global_end == sb.global_end and sa.local_end == sb.local_end
            assert kv_a["current_step"] == kv_b["current_step"] == st_ref.current_step
            start += n_new

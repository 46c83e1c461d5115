"""Steady-state chunk steps replayed from a CUDA graph must leave exactly what the eager path leaves:
outputs, cache contents, index tensors, evict queues.  Also the append entry point that reads its
per-row slot parameters from device memory, which the recorded launches use."""
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def _append_inputs(B=2, N=24, H=2, S=96, seed=3):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    q, k, v = mk(B, N, H, 128), mk(B, N, H, 128), mk(B, N, H, 128)
    kc, vc = mk(B, S, H, 128), mk(B, S, H, 128)
    return q, k, v, kc, vc


def test_indirect_append_equals_the_host_parameter_entry_point():
    from streamdiffusionv2_b200 import ops
    from streamdiffusionv2_b200.wan_model import build_rope_table
    dev = torch.device("cuda")
    table = ops.rope_table_device(build_rope_table(128), dev)
    q, k, v, kc, vc = _append_inputs()
    kc2, vc2 = kc.clone(), vc.clone()
    grid, frames, dst, ge, le = (2, 3, 4), [5, 9], [24, 72], [1000, 2000], [48, 96]
    idx = [torch.zeros(2, dtype=torch.int64, device=dev) for _ in range(4)]
    ref = ops.rope_kv_append(q, k, v, kc, vc, table, grid, frames, dst, index_tensors=(idx[0], idx[1]),
                             index_values=(ge, le))
    params = torch.tensor([frames, dst, ge, le], dtype=torch.int64, device=dev)
    out = ops.rope_kv_append(q, k, v, kc2, vc2, table, grid, [0, 0], [0, 0], index_tensors=(idx[2], idx[3]),
                             index_values=([0, 0], [0, 0]), step_params=params)
    ops.read_status(dev)
    assert torch.equal(out, ref) and torch.equal(kc, kc2) and torch.equal(vc, vc2)
    assert idx[2].tolist() == ge and idx[3].tolist() == le
    # the same launch parameters, new values in the array: another slot is written
    params.copy_(torch.tensor([[6, 10], [0, 48], [1, 2], [3, 4]], dtype=torch.int64))
    kc3, vc3 = kc.clone(), vc.clone()
    ops.rope_kv_append(q, k, v, kc3, vc3, table, grid, [0, 0], [0, 0], index_tensors=(idx[2], idx[3]),
                       index_values=([0, 0], [0, 0]), step_params=params)
    kc4, vc4 = kc.clone(), vc.clone()
    ops.rope_kv_append(q, k, v, kc4, vc4, table, grid, [6, 10], [0, 48])
    ops.read_status(dev)
    assert torch.equal(kc3, kc4) and torch.equal(vc3, vc4) and idx[2].tolist() == [1, 2]


@pytest.mark.parametrize("bad", [[[5, 9], [24, 80], [0, 0], [0, 0]],       # slot runs past the cache
                                 [[5, 9], [-1, 0], [0, 0], [0, 0]],        # negative slot
                                 [[5, 2000], [0, 0], [0, 0], [0, 0]]])     # frame beyond the rope table
def test_indirect_append_refuses_out_of_range_device_parameters(bad):
    from streamdiffusionv2_b200 import _native, ops
    from streamdiffusionv2_b200.wan_model import build_rope_table
    dev = torch.device("cuda")
    table = ops.rope_table_device(build_rope_table(128), dev)
    q, k, v, kc, vc = _append_inputs()
    kc0, vc0 = kc.clone(), vc.clone()
    idx = [torch.full((2,), 7, dtype=torch.int64, device=dev) for _ in range(2)]
    params = torch.tensor(bad, dtype=torch.int64, device=dev)
    ops.read_status(dev)
    ops.rope_kv_append(q, k, v, kc, vc, table, (2, 3, 4), [0, 0], [0, 0], index_tensors=tuple(idx),
                       index_values=([0, 0], [0, 0]), step_params=params)
    with pytest.raises(_native.NativeError, match="out of range"):
        ops.read_status(dev)
    assert torch.equal(kc, kc0) and torch.equal(vc, vc0) and idx[0].tolist() == [7, 7]
    ops.read_status(dev)     # the report was cleared


def _run_stream(case_name, graphs, swap_at=None, reprompt_at=None, adapt_sink_threshold=-1):
    from model_harness import build_pipeline, snapshot
    case = cases.MODEL_CASES[case_name]
    fs, sched = cases.model_schedule(case)
    pipe, first, chunks = build_pipeline(case, device="cuda", dtype=torch.bfloat16,
                                         adapt_sink_threshold=adapt_sink_threshold)
    outs = []
    with torch.no_grad():
        torch.manual_seed(11)
        pipe.prepare(text_prompts=["p"], device=torch.device("cuda"), dtype=torch.bfloat16, noise=first,
                     current_start=0, current_end=fs * (1 + case["frames"]))
        if graphs:
            pipe.enable_step_graphs()
        torch.manual_seed(12)
        for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
            if i == swap_at:          # what a cache manager does: same contents, new tensors
                for kv in pipe.kv_cache1:
                    kv["k"], kv["v"] = kv["k"].clone(), kv["v"].clone()
            if i == reprompt_at:      # a new prompt mid-stream: the text K/V are recomputed on the next call
                pipe.conditional_dict["prompt_embeds"] = pipe.conditional_dict["prompt_embeds"].flip(1).contiguous()
                for cc in pipe.crossattn_cache:
                    cc["is_init"] = False
            outs.append(pipe.inference_stream(noise, cs, ce).clone())
    torch.cuda.synchronize()
    n_layers = cases.MODEL_KW["num_layers"]
    return outs, [snapshot(pipe, i) for i in range(n_layers)], pipe


def test_graph_replayed_stream_equals_the_eager_stream():
    from streamdiffusionv2_b200 import ops
    eager_out, eager_state, _ = _run_stream("m_stream", graphs=False)
    graph_out, graph_state, pipe = _run_stream("m_stream", graphs=True)
    ops.read_status(torch.device("cuda"))
    sg = pipe.step_graphs
    assert sg.replays >= 5 and sg.eager_steps >= 1, (sg.replays, sg.eager_steps)   # the fill steps run eagerly
    for i, (a, b) in enumerate(zip(eager_out, graph_out)):
        assert torch.equal(a, b), f"chunk {i}"
    assert eager_state == graph_state


def test_replaced_cache_tensors_invalidate_the_recording():
    eager_out, eager_state, _ = _run_stream("m_stream", graphs=False, swap_at=6)
    graph_out, graph_state, pipe = _run_stream("m_stream", graphs=True, swap_at=6)
    assert pipe.step_graphs.replays >= 4
    for i, (a, b) in enumerate(zip(eager_out, graph_out)):
        assert torch.equal(a, b), f"chunk {i}"
    assert eager_state == graph_state


def test_a_new_prompt_mid_stream_is_not_served_from_a_stale_recording():
    eager_out, eager_state, _ = _run_stream("m_stream", graphs=False, reprompt_at=6)
    graph_out, graph_state, pipe = _run_stream("m_stream", graphs=True, reprompt_at=6)
    plain_out, _, _ = _run_stream("m_stream", graphs=False)
    assert not torch.equal(plain_out[7], eager_out[7])          # the prompt does change the result
    for i, (a, b) in enumerate(zip(eager_out, graph_out)):
        assert torch.equal(a, b), f"chunk {i}"
    assert eager_state == graph_state


@pytest.mark.parametrize("thr", [0.2, 0.95])
def test_adaptive_sink_stream_records_and_replays(thr):
    """The default video-to-video shape (one frame per chunk, sink frames refreshed when the new frame
    drifts away from them): the data-dependent slot choice runs on the device, so steady steps are
    recorded and replayed like any other, and leave the outputs, caches, index tensors and evict
    queues of the launch-by-launch path.  The higher threshold makes the refresh fire often."""
    from streamdiffusionv2_b200 import ops
    eager_out, eager_state, _ = _run_stream("m_stream_1f", graphs=False, adapt_sink_threshold=thr)
    graph_out, graph_state, pipe = _run_stream("m_stream_1f", graphs=True, adapt_sink_threshold=thr)
    ops.read_status(torch.device("cuda"))
    assert pipe.step_graphs.replays >= 3, (pipe.step_graphs.replays, pipe.step_graphs.eager_steps)
    for i, (a, b) in enumerate(zip(eager_out, graph_out)):
        assert torch.equal(a, b), f"chunk {i}"
    assert eager_state == graph_state
    if thr > 0.9:      # refreshed sink slots show up as queue entries inside the sink region at some point
        assert any(st["evict_idx"] for st in graph_state)

"""Two pipeline stages on two GPUs (NCCL).  The same stream is run four ways - left alone on the
reference's split; with a block moved between the stages half-way; with the stage boundary inside a
block from the start; and with the ranges planned from costs measured on the GPUs and the blocks
moved accordingly.  All four must give bit-identical latents, and on every stage the index tensors,
evict queues and step counters must equal the fixture recorded from the reference's own two-stage
pipeline after every chunk.  Skipped on a single-GPU machine."""
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, mode, q):
    try:
        for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
            if p not in sys.path:
                sys.path.insert(0, p)
        import datetime

        import torch.distributed as dist

        import cases
        from model_harness import build_pipeline, snapshot
        from streamdiffusionv2_b200 import ops
        from streamdiffusionv2_b200.pipeline_runner import PipelineStageRunner
        from streamdiffusionv2_b200.stage_transport import StageLink
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        device = torch.device("cuda", rank)
        torch.cuda.set_device(device)
        dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
        case = cases.MODEL_CASES["m_stages"]
        fs, sched = cases.model_schedule(case)
        pipe, first, chunks = build_pipeline(case, device=device, dtype=torch.bfloat16)
        role = "input" if rank == 0 else "output"
        outs, states, planned = [], [], None
        with torch.no_grad():
            torch.manual_seed(21)
            pipe.prepare(text_prompts=["p"], device=device, dtype=torch.bfloat16, noise=first, current_start=0,
                         current_end=fs * (1 + case["frames"]), block_mode=role)
            torch.manual_seed(22)
            link = StageLink(rank, world, device, (len(case["levels"]), fs * case["frames"], cases.MODEL_KW["dim"]),
                             tuple(pipe.hidden_states.shape), dtype=torch.bfloat16, timeout_s=60)
            if mode == "half":
                runner = PipelineStageRunner(pipe, link, rank, world, half_ranges=[[0, 3], [3, 6]])
            else:
                runner = PipelineStageRunner(pipe, link, rank, world, [[0, 2], [2, 3]])
            for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
                if i == 1 and mode == "measured":
                    runner.measure_costs(3)
                if i == 4 and mode == "move":
                    runner.rebalance([[0, 1], [1, 3]])
                if i == 4 and mode == "measured":
                    planned = runner.plan_ranges("half")
                    runner.rebalance(planned, halves=True)
                o = runner.step(i, noise, cs, ce, None, last=(i == 3))
                if o is not None:
                    outs.append(o.float().cpu())
                if i == 3:
                    runner.quiesce()
                # index state of the block whose self-attention this stage runs first (stage 0) / last (stage 1)
                owned = list(runner.owned_blocks)
                if owned:
                    st = snapshot(pipe, owned[0] if rank == 0 else owned[-1])
                    states.append({k: st[k] for k in ("global_end", "local_end", "evict_idx", "current_step")})
                else:
                    states.append(None)
            runner.finish()
            ops.read_status(device)
        q.put((rank, "ok", outs, (runner.half_range, states, planned)))
        dist.destroy_process_group()
    except Exception:
        q.put((rank, "error", traceback.format_exc(), None))


def _run(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(2):
            r = q.get(timeout=150)
            res[r[0]] = r[1:]
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    return res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_pipeline_split_four_ways_gives_one_stream_and_the_reference_index_state():
    import cases
    meta, _ = cases.load_fixture("m_stages")
    runs = {mode: _run(mode) for mode in ("plain", "move", "half", "measured")}
    for mode, res in runs.items():
        for r, v in res.items():
            assert v[0] == "ok", (mode, v[1])
    plain = runs["plain"][1][1]
    assert len(plain) == cases.MODEL_CASES["m_stages"]["chunks"]
    for mode in ("move", "half", "measured"):
        outs = runs[mode][1][1]
        assert len(outs) == len(plain)
        for i, (a, b) in enumerate(zip(plain, outs)):
            assert torch.equal(a, b), f"{mode}: chunk {i} differs"
    assert runs["move"][0][2][0] == [0, 2] and runs["move"][1][2][0] == [2, 6]
    assert runs["half"][0][2][0] == [0, 3] and runs["half"][1][2][0] == [3, 6]
    planned = runs["measured"][0][2][2]
    assert planned == runs["measured"][1][2][2] and planned[0][0] == 0 and planned[1][1] == 6
    # index state is data independent: every run reproduces the reference's own two-stage pipeline
    for mode, res in runs.items():
        for rank, key in ((0, "stageA_layer0"), (1, "stageB_layerL")):
            for i, st in enumerate(res[rank][2][1]):
                if st is None:
                    continue
                want = meta["steps"][i][key]
                assert all(st[k] == want[k] for k in st), (mode, rank, i, st, want)

"""Two pipeline stages on two GPUs (NCCL): a stream whose blocks are moved between the stages half-way
equals, bit for bit, the same stream left alone.  Skipped on a single-GPU machine."""
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


def _worker(rank, world, port, move, q):
    try:
        for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
            if p not in sys.path:
                sys.path.insert(0, p)
        import datetime

        import torch.distributed as dist

        import cases
        from model_harness import build_pipeline
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
        outs = []
        with torch.no_grad():
            torch.manual_seed(21)
            pipe.prepare(text_prompts=["p"], device=device, dtype=torch.bfloat16, noise=first, current_start=0,
                         current_end=fs * (1 + case["frames"]), block_mode=role)
            torch.manual_seed(22)
            link = StageLink(rank, world, device, (len(case["levels"]), fs * case["frames"], cases.MODEL_KW["dim"]),
                             tuple(pipe.hidden_states.shape), dtype=torch.bfloat16, timeout_s=60)
            runner = PipelineStageRunner(pipe, link, rank, world, [[0, 2], [2, 3]])
            for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
                if i == 4 and move:
                    runner.rebalance([[0, 1], [1, 3]])
                o = runner.step(i, noise, cs, ce, None, last=(i == 3))
                if o is not None:
                    outs.append(o.float().cpu())
                if i == 3:
                    runner.quiesce()
            runner.finish()
            ops.read_status(device)
        q.put((rank, "ok", outs, runner.block_range))
        dist.destroy_process_group()
    except Exception:
        q.put((rank, "error", traceback.format_exc(), None))


def _run(move):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, move, q)) for r in range(2)]
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
def test_blocks_moved_between_two_gpus_leave_the_stream_unchanged():
    plain, moved = _run(False), _run(True)
    for res in (plain, moved):
        for r, v in res.items():
            assert v[0] == "ok", v[1]
    assert moved[0][2] == [0, 1] and moved[1][2] == [1, 3]
    assert len(moved[1][1]) == len(plain[1][1]) > 0
    for i, (a, b) in enumerate(zip(plain[1][1], moved[1][1])):
        assert torch.equal(a, b), f"chunk {i}"

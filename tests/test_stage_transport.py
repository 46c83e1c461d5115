"""Pipeline-parallel hand-off on CPU ranks (gloo): the ring transport and the per-rank runner
reproduce the two-stage fixture recorded from the reference, and survive failures injected on the
host (a peer that never sends; a packet of the wrong shape)."""
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port):
    for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)


class _Patch:
    """Minimal stand-in for pytest's monkeypatch inside a child process."""

    def setattr(self, obj, name, value):
        setattr(obj, name, value)


def _worker_pipeline(rank, world, port, ranges, quiesce_every, q, park_at=(), halves=False, replan_at=None):
    try:
        _init(rank, world, port)
        import fake_ops
        from model_harness import build_pipeline, snapshot
        from streamdiffusionv2_b200.pipeline_runner import PipelineStageRunner
        from streamdiffusionv2_b200.stage_transport import StageLink
        fake_ops.install(_Patch())
        case = cases.MODEL_CASES["m_stages"]
        fs, sched = cases.model_schedule(case)
        pipe, first, chunks = build_pipeline(case)
        role = "input" if rank == 0 else ("output" if rank == world - 1 else "middle")
        with torch.no_grad():
            torch.manual_seed(case["seed"] + 1)
            pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                         current_start=0, current_end=fs * (1 + case["frames"]), block_mode=role)
            torch.manual_seed(case["seed"] + 2)
            rows = len(case["levels"])
            link = StageLink(rank, world, torch.device("cpu"), (rows, fs * case["frames"], cases.MODEL_KW["dim"]),
                             tuple(pipe.hidden_states.shape), dtype=torch.float32, timeout_s=60)
            runner = (PipelineStageRunner(pipe, link, rank, world, half_ranges=ranges) if halves
                      else PipelineStageRunner(pipe, link, rank, world, ranges))
            outs, states, planned = [], [], None
            for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
                last = quiesce_every > 0 and i % quiesce_every == quiesce_every - 1
                if replan_at is not None and i == replan_at[0]:
                    runner.measure_costs(replan_at[1] - replan_at[0])
                if replan_at is not None and i == replan_at[1] - 1:
                    last = True
                if replan_at is not None and i == replan_at[1]:
                    # measured steps are over and the ring was emptied: plan from the gathered costs and move
                    planned = runner.plan_ranges(replan_at[2])
                    runner.rebalance(planned, halves=True)
                o = runner.step(i, noise, cs, ce, None, last=last)
                if o is not None:
                    outs.append(o.clone().numpy())
                if last:
                    runner.quiesce()       # ring emptied mid-stream; results must not change
                if planned is not None and i == replan_at[1]:
                    states.append({"planned": planned, "half_range": runner.half_range,
                                   "costs": runner.last_costs})
                    continue
                if i + rank in park_at:    # rank r is r chunks behind rank 0: the ring stays full
                    runner.park()
                    dist.barrier()
                states.append(snapshot(pipe, runner.block_range[0] if rank == 0 else runner.block_range[1] - 1))
            runner.finish()
        q.put((rank, "ok", outs, states))
    except Exception:
        q.put((rank, "error", traceback.format_exc(), None))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _worker_restart(rank, world, port, ranges, q):
    """3 chunks, a prompt restart from stage 0, 3 more chunks on the same links."""
    try:
        _init(rank, world, port)
        import fake_ops
        from model_harness import build_pipeline
        from streamdiffusionv2_b200.pipeline_runner import PipelineStageRunner, StreamRestart
        from streamdiffusionv2_b200.stage_transport import StageLink
        fake_ops.install(_Patch())
        case = cases.MODEL_CASES["m_stages"]
        fs, sched = cases.model_schedule(case)
        pipe, first, chunks = build_pipeline(case)
        role = "input" if rank == 0 else ("output" if rank == world - 1 else "middle")
        got, outs = [], 0
        with torch.no_grad():
            pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                         current_start=0, current_end=fs * (1 + case["frames"]), block_mode=role)
            link = StageLink(rank, world, torch.device("cpu"), (len(case["levels"]), fs * case["frames"],
                             cases.MODEL_KW["dim"]), tuple(pipe.hidden_states.shape), dtype=torch.float32, timeout_s=60)
            runner = PipelineStageRunner(pipe, link, rank, world, ranges)
            i = 0
            while i < 6:
                if rank == 0 and i == 3 and not got:
                    runner.restart("prompt two \u2713")
                    got.append("sent")
                noise, (cs, ce) = chunks[i], sched[i]
                try:
                    o = runner.step(i, noise, cs, ce, None)
                except StreamRestart as r:
                    got.append(r.prompt)
                    assert runner.items == 0
                    continue                     # the same chunk index arrives again after the restart
                outs += o is not None
                i += 1
            runner.finish()
        q.put((rank, "ok", got, outs))
    except Exception:
        q.put((rank, "error", traceback.format_exc(), None))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _worker_rebalance(rank, world, port, ranges_a, ranges_b, q):
    """4 chunks on one block split, the ring emptied, blocks (with their K/V state) moved, 4 more chunks."""
    try:
        _init(rank, world, port)
        import fake_ops
        from model_harness import build_pipeline
        from streamdiffusionv2_b200.pipeline_runner import PipelineStageRunner
        from streamdiffusionv2_b200.stage_transport import StageLink
        fake_ops.install(_Patch())
        case = cases.MODEL_CASES["m_stages"]
        fs, sched = cases.model_schedule(case)
        pipe, first, chunks = build_pipeline(case)
        role = "input" if rank == 0 else ("output" if rank == world - 1 else "middle")
        outs = []
        with torch.no_grad():
            torch.manual_seed(case["seed"] + 1)
            pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                         current_start=0, current_end=fs * (1 + case["frames"]), block_mode=role)
            torch.manual_seed(case["seed"] + 2)
            link = StageLink(rank, world, torch.device("cpu"), (len(case["levels"]), fs * case["frames"],
                             cases.MODEL_KW["dim"]), tuple(pipe.hidden_states.shape), dtype=torch.float32, timeout_s=60)
            runner = PipelineStageRunner(pipe, link, rank, world, ranges_a)
            for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
                if i == 4:
                    runner.rebalance(ranges_b)
                o = runner.step(i, noise, cs, ce, None, last=(i == 3))
                if o is not None:
                    outs.append(o.clone().numpy())
                if i == 3:
                    runner.quiesce()
            runner.finish()
            owned = [i for i in range(cases.MODEL_KW["num_layers"]) if pipe.kv_cache1[i]["k"].shape[1] > 0]
        q.put((rank, "ok", outs, (runner.block_range, owned)))
    except Exception:
        q.put((rank, "error", traceback.format_exc(), None))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run(target, world, *args, timeout=240):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    extra = args[-1] if args and isinstance(args[-1], dict) else None
    if extra is not None:
        args = args[:-1]
    procs = [ctx.Process(target=target, args=(r, world, port, *args, q), kwargs=extra or {}) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            r = q.get(timeout=timeout)
            results[r[0]] = r[1:]
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return results


@pytest.mark.parametrize("quiesce_every", [0, 3])
def test_two_rank_pipeline_matches_reference_fixture(quiesce_every):
    case = cases.MODEL_CASES["m_stages"]
    meta, z = cases.load_fixture("m_stages")
    nblk, split = cases.MODEL_KW["num_layers"], case["split"]
    res = _run(_worker_pipeline, 2, [[0, split], [split, nblk]], quiesce_every)
    for r, v in res.items():
        assert v[0] == "ok", v[1]
    outs = res[1][1]
    assert len(outs) == case["chunks"]
    for i, o in enumerate(outs):
        assert np.abs(o - z[f"out_{i}"]).max() < 5e-4, i
    for i in range(case["chunks"]):
        for key in ("global_end", "local_end", "evict_idx", "current_step"):
            assert res[0][2][i][key] == meta["steps"][i]["stageA_layer0"][key]
            assert res[1][2][i][key] == meta["steps"][i]["stageB_layerL"][key]


def test_parking_a_full_ring_at_a_barrier_changes_nothing():
    """Staggered ranks pause with one packet on every edge (park + barrier), twice, and go on:
    same outputs and index state as the uninterrupted stream."""
    case = cases.MODEL_CASES["m_stages"]
    meta, z = cases.load_fixture("m_stages")
    nblk, split = cases.MODEL_KW["num_layers"], case["split"]
    res = _run(_worker_pipeline, 2, [[0, split], [split, nblk]], 0, {"park_at": (1, 3, 4)})
    for r, v in res.items():
        assert v[0] == "ok", v[1]
    outs = res[1][1]
    assert len(outs) == case["chunks"]
    for i, o in enumerate(outs):
        assert np.abs(o - z[f"out_{i}"]).max() < 5e-4, i
    for i in range(case["chunks"]):
        assert res[0][2][i]["global_end"] == meta["steps"][i]["stageA_layer0"]["global_end"]
        assert res[1][2][i]["global_end"] == meta["steps"][i]["stageB_layerL"]["global_end"]


def test_three_rank_ring_parks_and_resumes():
    plain = _run(_worker_pipeline, 3, [[0, 1], [1, 2], [2, 3]], 0)
    parked = _run(_worker_pipeline, 3, [[0, 1], [1, 2], [2, 3]], 0, {"park_at": (2, 4)})
    for res in (plain, parked):
        for r, v in res.items():
            assert v[0] == "ok", v[1]
    assert len(parked[2][1]) == len(plain[2][1])
    for a, b in zip(parked[2][1], plain[2][1]):
        assert np.array_equal(a, b)


def test_prompt_restart_travels_the_ring_and_the_links_stay_usable():
    res = _run(_worker_restart, 3, [[0, 1], [1, 2], [2, 3]])
    for r, v in res.items():
        assert v[0] == "ok", v[1]
    assert res[0][1] == ["sent"]
    assert res[1][1] == ["prompt two \u2713"] and res[2][1] == ["prompt two \u2713"]
    assert res[2][2] == 6 and res[0][2] == 0


@pytest.mark.parametrize("a,b", [([[0, 2], [2, 3]], [[0, 1], [1, 3]]), ([[0, 1], [1, 3]], [[0, 2], [2, 3]])])
def test_blocks_move_between_stages_with_their_cache_state(a, b):
    """Rebalancing mid-stream must not change the stream: the moved block's K/V, index tensors and
    evict queue travel with it, so the outputs equal the reference fixture's."""
    case = cases.MODEL_CASES["m_stages"]
    _, z = cases.load_fixture("m_stages")
    res = _run(_worker_rebalance, 2, a, b)
    for r, v in res.items():
        assert v[0] == "ok", v[1]
    outs = res[1][1]
    assert len(outs) == case["chunks"]
    for i, o in enumerate(outs):
        assert np.abs(o - z[f"out_{i}"]).max() < 5e-4, i
    assert res[0][2][0] == b[0] and res[1][2][0] == b[1]
    moved = (set(range(*a[0])) ^ set(range(*b[0])))
    for r in (0, 1):     # the giver holds a placeholder for what it gave away
        gave = moved & set(range(*a[r]))
        assert not (gave & set(res[r][2][1]))


def test_three_rank_pipeline_runs_with_a_middle_stage():
    """input -> middle -> output over three ranks; index state must stay consistent on every stage
    (all stages see the same row starts) and the stream must complete."""
    res = _run(_worker_pipeline, 3, [[0, 1], [1, 2], [2, 3]], 4)
    for r, v in res.items():
        assert v[0] == "ok", v[1]
    n = cases.MODEL_CASES["m_stages"]["chunks"]
    assert len(res[2][1]) == n
    for i in range(n):
        assert res[0][2][i]["global_end"] == res[1][2][i]["global_end"] == res[2][2][i]["global_end"]
        assert np.isfinite(res[2][1][i]).all()


def _worker_fault(rank, world, port, mode, q):
    try:
        _init(rank, world, port)
        from streamdiffusionv2_b200.stage_transport import StageLink
        link = StageLink(rank, world, torch.device("cpu"), (2, 4, 8), (2, 1, 4, 2, 2), dtype=torch.float32,
                         timeout_s=3)
        if mode == "silent_peer":
            if rank == 1:
                try:
                    link.recv()                       # rank 0 never sends
                    q.put((rank, "no error", None, None))
                except Exception as e:                # the bounded wait surfaces as an exception
                    q.put((rank, "raised", type(e).__name__, None))
            else:
                import time
                time.sleep(6)
                q.put((rank, "idle", None, None))
        elif mode == "bad_shape":
            if rank == 0:
                try:
                    link.send(0, torch.zeros(2, 4, 9), torch.zeros(2, 1, 4, 2, 2), [1, 8, 1, 2, 2], [0, 0], [4, 4], 0)
                    q.put((rank, "no error", None, None))
                except ValueError:
                    q.put((rank, "raised", "ValueError", None))
            else:
                q.put((rank, "idle", None, None))
        elif mode == "roundtrip":
            if rank == 0:
                link.send(7, torch.arange(64.).view(2, 4, 8), torch.ones(2, 1, 4, 2, 2), [1, 8, 1, 2, 2], [6, 12],
                          [12, 18], 500)
                back = link.recv()
                q.put((rank, "ok", (back.chunk_idx, back.starts, float(back.latents.sum())), None))
            else:
                pkt = link.recv()
                ok = (pkt.chunk_idx == 7 and pkt.current_step == 500 and pkt.starts == [6, 12]
                      and pkt.ends == [12, 18] and pkt.patched_x_shape == [1, 8, 1, 2, 2]
                      and torch.equal(pkt.activations, torch.arange(64.).view(2, 4, 8)))
                link.send(pkt.chunk_idx, None, pkt.latents * 2, pkt.patched_x_shape, pkt.starts, pkt.ends,
                          pkt.current_step)
                q.put((rank, "ok" if ok else "mismatch", None, None))
            link.drain()
    except Exception:
        q.put((rank, "error", traceback.format_exc(), None))
    finally:
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:
            pass


def test_packet_roundtrip_two_ranks():
    res = _run(_worker_fault, 2, "roundtrip", timeout=60)
    assert res[1][0] == "ok", res[1]
    assert res[0][0] == "ok" and res[0][1] == (7, [6, 12], 64.0), res[0]


def test_silent_peer_times_out_instead_of_hanging():
    """Failure made on the host: the upstream rank never sends.  The receiver's wait is bounded by
    the link timeout and raises; nothing spins forever."""
    res = _run(_worker_fault, 2, "silent_peer", timeout=60)
    assert res[1][0] == "raised", res[1]


def test_wrong_shape_is_rejected_before_anything_is_sent():
    res = _run(_worker_fault, 2, "bad_shape", timeout=60)
    assert res[0][0] == "raised", res[0]


def test_balanced_block_ranges_cover_all_blocks_and_spare_the_end_stages():
    from streamdiffusionv2_b200.stage_transport import balanced_block_ranges, contiguous_block_ranges
    for total, world in ((30, 8), (30, 4), (30, 2), (40, 8), (30, 7), (3, 3), (31, 4)):
        r = balanced_block_ranges(total, world)
        assert r[0][0] == 0 and r[-1][1] == total and all(a[1] == b[0] for a, b in zip(r, r[1:]))
        sizes = [b - a for a, b in r]
        assert sorted(sizes) == sorted(b - a for a, b in contiguous_block_ranges(total, world)) or world == 2
        assert sizes[0] == min(sizes) and sizes[-1] <= sizes[len(sizes) // 2]
    assert [b - a for a, b in balanced_block_ranges(30, 8)] == [3, 4, 4, 4, 4, 4, 4, 3]


def test_block_ranges_follow_the_reference_split():
    from streamdiffusionv2_b200.stage_transport import contiguous_block_ranges as r
    assert r(30, 2) == [[0, 15], [15, 30]]
    assert [b - a for a, b in r(30, 4)] == [8, 8, 7, 7]
    assert [b - a for a, b in r(30, 8)] == [4, 4, 4, 4, 4, 4, 3, 3]
    assert [b - a for a, b in r(40, 8)] == [5] * 8
    for n, w in ((30, 4), (30, 8), (40, 4), (7, 3)):
        rr = r(n, w)
        assert rr[0][0] == 0 and rr[-1][1] == n and all(rr[i][1] == rr[i + 1][0] for i in range(w - 1))


# ---------------------------------------------------------------------------------------------
# stage boundaries inside a block, and ranges planned from measured costs
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("world,half_ranges", [
    (2, [[0, 3], [3, 6]]),            # stage A: block 0 and the self-attention of block 1
    (2, [[0, 1], [1, 6]]),            # stage A: only the self-attention of block 0
    (3, [[0, 3], [3, 4], [4, 6]]),    # a middle stage that runs only the second half of block 1
])
def test_half_block_stage_boundaries_reproduce_the_reference_fixture(world, half_ranges):
    """Stages may meet after a block's self-attention residual; the stream is the one the reference's
    whole-block pipeline produced."""
    case = cases.MODEL_CASES["m_stages"]
    _, z = cases.load_fixture("m_stages")
    res = _run(_worker_pipeline, world, half_ranges, 0, {"halves": True})
    for r, v in res.items():
        assert v[0] == "ok", v[1]
    outs = res[world - 1][1]
    assert len(outs) == case["chunks"]
    if world == 2:                      # the fixture is a two-stage run (ring depth 2)
        for i, o in enumerate(outs):
            assert np.abs(o - z[f"out_{i}"]).max() < 5e-4, i
    else:                               # three stages: the deeper ring delays the re-noised rows; compare with whole blocks
        plain = _run(_worker_pipeline, 3, [[0, 1], [1, 2], [2, 3]], 0)
        for a, b in zip(outs, plain[2][1]):
            assert np.abs(a - b).max() < 1e-5


def test_partition_by_cost_is_optimal_and_respects_block_boundaries():
    import itertools
    from streamdiffusionv2_b200.stage_transport import partition_by_cost
    g = torch.Generator().manual_seed(5)
    for n, w in ((6, 2), (8, 3), (10, 4), (12, 3)):
        costs = (0.2 + torch.rand(n, generator=g)).tolist()
        over = (0.5 * torch.rand(w, generator=g)).tolist()
        for step in (1, 2):
            got = partition_by_cost(costs, over, boundary_step=step)
            assert got[0][0] == 0 and got[-1][1] == n and all(a[1] == b[0] for a, b in zip(got, got[1:]))
            assert all(b > a and a % step == 0 and b % step == 0 for a, b in got)
            t_got = max(over[r] + sum(costs[a:b]) for r, (a, b) in enumerate(got))
            best = min(max(over[r] + sum(costs[a:b]) for r, (a, b) in enumerate(zip((0,) + cut, cut + (n,))))
                       for cut in itertools.combinations(range(step, n, step), w - 1))
            assert abs(t_got - best) < 1e-12, (n, w, step)
    # 30 equal blocks on 8 stages, extra work on the first and the last stage: the remainder moves off the
    # ends (3-4-4-4-4-4-4-3); half-block boundaries cannot beat that here (any 8 consecutive halves are 4 blocks'
    # worth and the average stage holds 7.5), but they do where the counts leave room
    t = lambda rs, c, o: max(o[r] + sum(c[a:b]) for r, (a, b) in enumerate(rs))
    halves, over = [1.4, 0.45] * 30, [0.45, 0, 0, 0, 0, 0, 0, 0.25]
    whole = partition_by_cost(halves, over, boundary_step=2)
    assert [(b - a) // 2 for a, b in whole] == [3, 4, 4, 4, 4, 4, 4, 3]
    assert t(whole, halves, over) == pytest.approx(4 * 1.85)
    assert t(partition_by_cost(halves, over), halves, over) <= t(whole, halves, over) + 1e-12
    three = [1.0, 1.0] * 3
    assert t(partition_by_cost(three, [0, 0], 2), three, [0, 0]) == pytest.approx(4.0)
    assert t(partition_by_cost(three, [0, 0], 1), three, [0, 0]) == pytest.approx(3.0)
    # stages of different speed (GPUs under a power cap differ by several per cent): the faster ones get more
    units, scales = [0.725, 0.275] * 30, [1.774, 1.772, 1.663, 1.629]
    plan = partition_by_cost(units, [0.27, 0, 0, 0.39], boundary_step=2, scales=scales)
    assert [(b - a) // 2 for a, b in plan] == [7, 7, 8, 8]
    brute = min(max(o + sc * sum(units[a:b]) for o, sc, (a, b) in zip([0.27, 0, 0, 0.39], scales, zip((0,) + cut, cut + (60,))))
                for cut in itertools.combinations(range(2, 60, 2), 3))
    assert abs(t(plan, units, [0, 0, 0, 0]) * 0 + max(o + sc * sum(units[a:b]) for o, sc, (a, b) in
                                                      zip([0.27, 0, 0, 0.39], scales, plan)) - brute) < 1e-12
    with pytest.raises(ValueError):
        partition_by_cost([1.0], [0.0, 0.0])


def test_plan_uses_measurements_as_proportions_only():
    """A stage that happened to run slowly while it was being measured (another clock, a busier host)
    must not be handed fewer blocks for it: all stages are the same part under the same power cap."""
    from streamdiffusionv2_b200.stage_transport import plan_from_measurements
    ranges = [[0, 16], [16, 32], [32, 46], [46, 60]]                 # 8, 8, 7, 7 blocks
    speed = [1.0, 1.4, 0.8, 1.1]                                      # how fast each stage ran during the measurement
    per_half, extra = [], []
    for r, (a, b) in enumerate(ranges):
        per_half += [1.30 * speed[r], 0.50 * speed[r]] * ((b - a) // 2)
        extra.append([0.25, 0.16, 0.16, 0.40][r] * speed[r])
    plan, info = plan_from_measurements(per_half, extra, ranges, "half")
    even, _ = plan_from_measurements([1.30, 0.50] * 30, [0.25, 0.16, 0.16, 0.40], ranges, "half")
    assert plan == even
    assert abs(info["attention_share_of_block"] - 1.30 / 1.80) < 1e-9
    # 30.5 blocks of work on 4 stages: boundaries inside blocks get closer to 7.63 each than whole blocks can
    whole, winfo = plan_from_measurements(per_half, extra, ranges, "block")
    assert max(info["planned_stage_load_blocks"]) < max(winfo["planned_stage_load_blocks"]) - 0.1
    assert all(a % 2 == 0 and b % 2 == 0 for a, b in whole)


def test_measured_costs_give_every_rank_the_same_plan_and_the_stream_survives_the_move():
    """Three measured steps, one all-gather, the exact partition on every rank, blocks (or halves of
    blocks) moved with their K/V state mid-stream: the outputs stay those of the fixture."""
    case = cases.MODEL_CASES["m_stages"]
    _, z = cases.load_fixture("m_stages")
    nblk, split = cases.MODEL_KW["num_layers"], case["split"]
    res = _run(_worker_pipeline, 2, [[0, split], [split, nblk]], 0, {"replan_at": (1, 4, "half")})
    for r, v in res.items():
        assert v[0] == "ok", v[1]
    info = [next(s for s in res[r][2] if "planned" in s) for r in (0, 1)]
    assert info[0]["planned"] == info[1]["planned"]                       # same plan everywhere
    assert info[0]["half_range"] == info[0]["planned"][0] and info[1]["half_range"] == info[1]["planned"][1]
    assert len(info[0]["costs"]["per_half_ms"]) == 2 * nblk and min(info[0]["costs"]["per_half_ms"]) > 0
    outs = res[1][1]
    assert len(outs) == case["chunks"]
    for i, o in enumerate(outs):
        assert np.abs(o - z[f"out_{i}"]).max() < 5e-4, i

#!/usr/bin/env python
"""Streaming-FPS benchmark of the causal Wan DiT with the sm_100a attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: random-init Wan-1.3B-shaped causal DiT (30 blocks, dim 1536, 12 heads x 128, FFN 8960),
bf16, 480x832 video (latent 16 x 60 x 104 per frame, 1560 tokens per latent frame), text context
512 x 4096 ~ N(0,1), 2 denoise levels batched as 2 cache rows, 2 latent frames per chunk, cache of
1 sink + 20 ring latent frames.  The stream is first advanced until the ring is full and wrapping;
every warm-up and timed step is then one chunk step (8 video frames) against the full cache.
N > 1: the same model split into N contiguous block ranges, one rank per GPU, stage activations
passed rank to rank over NCCL (one chunk in flight per stage).  The timed region is steady state:
the warm-up leaves rank r exactly r chunks behind rank 0, then every rank runs K chunk steps between
the two barriers, so K chunks enter the pipeline and K leave it inside the region.
One JSON line is printed by rank 0.  `--impl reference` times the CPU restatement of the
reference's attention path on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FRAME_TOKENS = 1560          # 30 x 52 tokens per latent frame at 480 x 832
LATENT_HW = (60, 104)
CACHE_FRAMES = 21            # 1 sink + 20 ring
# dram__bytes_read.sum + dram__bytes_write.sum of one launch at the N=1 workload's shape (ncu, B200)
ATTN_DRAM_BYTES_1P3B = 450.4e6 + 14.5e6
APPEND_DRAM_BYTES_1P3B = 57.56e6 + 11.5e6
FRAMES_PER_CHUNK = 2
VIDEO_FRAMES_PER_CHUNK = 4 * FRAMES_PER_CHUNK
LEVELS = [700, 500]
MODEL_1P3B = dict(model_type="t2v", patch_size=(1, 2, 2), text_len=512, in_dim=16, dim=1536, ffn_dim=8960,
                  freq_dim=256, text_dim=4096, out_dim=16, num_heads=12, num_layers=30, qk_norm=True,
                  cross_attn_norm=True, eps=1e-6)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference attention path on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_attention_path(samples: int, warmup: int, q_tokens: int, budget_s: float = 150.0):
    """Times rope + slot write + attention over the full 21-frame cache for one layer and the 2
    cache rows of the workload (bf16 tensors, fp32 math on CPU, as the reference does there), on
    `q_tokens` of the chunk's 3120 query tokens per row.  Returns seconds per full layer call
    (scaled to 3120 query tokens) per sample."""
    from oracle import causal_attention_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    H, D, B = MODEL_1P3B["num_heads"], 128, len(LEVELS)
    smax = CACHE_FRAMES * FRAME_TOKENS
    n_full = FRAMES_PER_CHUNK * FRAME_TOKENS
    g = torch.Generator().manual_seed(0)
    table = orc.rope_table(D)
    kc = torch.randn(B, smax, H, D, generator=g).to(torch.bfloat16)
    vc = torch.randn(B, smax, H, D, generator=g).to(torch.bfloat16)
    q, k, v = (torch.randn(B, n_full, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    times = []
    t_begin = time.time()
    for i in range(warmup + samples):
        t0 = time.time()
        sf = [30, 28]
        rq = orc.rope_apply(q, (FRAMES_PER_CHUNK, 30, 52), table, sf)
        rk = orc.rope_apply(k, (FRAMES_PER_CHUNK, 30, 52), table, sf)
        for b, dst in enumerate((3120, 6240)):
            kc[b, dst:dst + n_full] = rk[b]
            vc[b, dst:dst + n_full] = v[b]
        t_rope = time.time() - t0
        t1 = time.time()
        orc.attend_cache(rq[:, :q_tokens], kc, vc, [smax] * B)
        t_att = (time.time() - t1) * (n_full / q_tokens)
        if i >= warmup:
            times.append(t_rope + t_att)
        if time.time() - t_begin > budget_s and len(times) >= 1:
            break
    return times


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    q_tokens = 780 if args.steps > 8 else 3120
    times = cpu_attention_path(args.steps, min(args.warmup, 1), q_tokens)
    layer_s = statistics.mean(times)
    chunk_s = layer_s * MODEL_1P3B["num_layers"]
    fps = VIDEO_FRAMES_PER_CHUNK / chunk_s
    sample = (f"attention path only (rope + slot write + attention over the full 32760-token cache), 1 of 30 "
              f"layers, 2 cache rows, {q_tokens} of 3120 query tokens per row timed and scaled; chunk time = 30 x "
              f"layer time; linear layers, norms and FFN not included")
    line = {"impl": "reference", "metric": metric_name(), "value": fps, "unit": "video frames/s",
            "n_gpus": args.gpus, "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": chunk_s * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 storage, fp32 math",
            "data": "synthetic", "config": workload_config(args.gpus),
            "cpu_baseline": {"value": fps, "unit": "video frames/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": fps, "unit": "video frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    args.emit(line)


def metric_name():
    return "streaming_fps_480x832_wan1.3b" if MODEL_1P3B["dim"] == 1536 else "streaming_fps_480x832_wan14b"


def workload_config(n_gpus: int):
    name = "Wan-1.3B" if MODEL_1P3B["dim"] == 1536 else "Wan-14B"
    return {"workload": f"random-init causal {name} DiT, 480x832, {len(LEVELS)} denoise levels ({len(LEVELS)} cache "
                        "rows), 2 latent frames per chunk, 1 sink + 20 ring frame cache, full and wrapping",
            "tokens_per_chunk_row": FRAMES_PER_CHUNK * FRAME_TOKENS, "cache_tokens": CACHE_FRAMES * FRAME_TOKENS,
            "cache_rows": len(LEVELS), "blocks": MODEL_1P3B["num_layers"],
            "parallelism": "single GPU" if n_gpus == 1 else f"pipeline of {n_gpus} contiguous block ranges",
            "l2_policy": "per-step working set (2.8 GB weights + 12 GB K/V cache) far exceeds the 126 MB L2; "
                         "no explicit flush"}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def build_pipeline(device, n_layers_override=None):
    from streamdiffusionv2_b200.stream_pipeline import DiffusionWrapper, StreamPipeline
    from streamdiffusionv2_b200.wan_model import CausalWanModel
    torch.manual_seed(0)
    kw = dict(MODEL_1P3B)
    if n_layers_override:
        kw["num_layers"] = n_layers_override
    with torch.device(device):
        model = CausalWanModel(**kw)
    torch.nn.init.normal_(model.head.head.weight, std=0.02)   # the stock init zeroes the output projection
    model = model.to(dtype=torch.bfloat16).eval()
    g = torch.Generator(device="cpu").manual_seed(1)
    prompt = torch.randn(1, 512, kw["text_dim"], generator=g).to(device=device, dtype=torch.bfloat16)
    pipe = StreamPipeline(DiffusionWrapper(model), lambda text_prompts: {"prompt_embeds": prompt.clone()}, LEVELS,
                          kw["num_layers"], kw["num_heads"], FRAME_TOKENS, CACHE_FRAMES, 1, -1, FRAMES_PER_CHUNK,
                          device=device)
    return pipe


class ChunkSchedule:
    """Chunk starts as the reference's drivers advance them, with the refresh rule."""

    def __init__(self):
        self.start = FRAME_TOKENS * (1 + FRAMES_PER_CHUNK)
        self.end = self.start + FRAMES_PER_CHUNK * FRAME_TOKENS

    def next(self):
        if self.start // FRAME_TOKENS >= 50:
            self.start = CACHE_FRAMES * FRAME_TOKENS - FRAME_TOKENS
            self.end = self.start + FRAMES_PER_CHUNK * FRAME_TOKENS
        cur = (self.start, self.end)
        self.start = self.end
        self.end += FRAMES_PER_CHUNK * FRAME_TOKENS
        return cur


def use_library_ops():
    """Comparison arm (`--impl library`): the same model and stream, but the three cache kernels are
    replaced by the calls the reference makes on a GPU - the fp64 complex rope chain with slice
    writes into the cache (models/wan/causal_model.py:94-108, 321-322), flash_attn_with_kvcache
    (:353-358), flash_attn_func for the text cross-attention (wan/modules/attention.py) - and the
    block's norm / modulation / gate chains run as separate PyTorch ops.  The slot bookkeeping stays
    ours (host integers, no device read-backs), so this arm is an upper bound on what the
    reference's own loop would reach.  Library kernels only: `gpu_launches` is reported as 0."""
    import math
    from flash_attn import flash_attn_func, flash_attn_with_kvcache
    from streamdiffusionv2_b200 import ops, wan_model

    def rope_kv_append(q, k, v, k_cache, v_cache, table, grid, start_frames, dst_begin, *, q_out=None,
                       index_tensors=None, index_values=None):
        B, n, H, D = q.shape
        f, h, w = (int(x) for x in grid)
        tc = torch.view_as_complex(table)
        c = D // 2
        ct, ch = c - 2 * (c // 3), c // 3
        if q_out is None:
            q_out = torch.empty((B, n, H, D), dtype=q.dtype, device=q.device)
        with ops._Logged("rope_kv_append", 6.0 * B * n * H * D * q.element_size()):
            for b in range(B):
                sf = int(start_frames[b])
                mult = torch.cat([tc[sf:sf + f, :ct].view(f, 1, 1, -1).expand(f, h, w, -1),
                                  tc[:h, ct:ct + ch].view(1, h, 1, -1).expand(f, h, w, -1),
                                  tc[:w, ct + ch:].view(1, 1, w, -1).expand(f, h, w, -1)], dim=-1).reshape(n, 1, -1)
                rq = torch.view_as_complex(q[b].to(torch.float64).reshape(n, H, -1, 2)) * mult
                rk = torch.view_as_complex(k[b].to(torch.float64).reshape(n, H, -1, 2)) * mult
                q_out[b] = torch.view_as_real(rq).flatten(2).type_as(q)
                d = int(dst_begin[b])
                k_cache[b:b + 1, d:d + n] = torch.view_as_real(rk).flatten(2).type_as(k).unsqueeze(0)
                v_cache[b:b + 1, d:d + n] = v[b:b + 1]
                if index_tensors is not None:
                    index_tensors[0][b:b + 1].fill_(int(index_values[0][b]))
                    index_tensors[1][b:b + 1].fill_(int(index_values[1][b]))
        return q_out

    def attn_kvcache(q, k_cache, v_cache, seq_lens, *, out=None, softmax_scale=None):
        B, n, H, D = q.shape
        lens = torch.tensor([int(x) for x in seq_lens[:B]], dtype=torch.int32, device=q.device)
        with ops._Logged("attn_kvcache", 4.0 * n * D * H * float(sum(int(x) for x in seq_lens[:B]))):
            return flash_attn_with_kvcache(q, k_cache, v_cache, cache_seqlens=lens, softmax_scale=softmax_scale)

    def cross_attn(q, k, v, *, out=None, softmax_scale=None):
        B = q.shape[0]
        with ops._Logged("cross_attn", 4.0 * B * q.shape[1] * q.shape[3] * q.shape[2] * k.shape[1]):
            return flash_attn_func(q, k.expand(B, -1, -1, -1), v.expand(B, -1, -1, -1), softmax_scale=softmax_scale)

    ops.rope_kv_append, ops.attn_kvcache, ops.cross_attn = rope_kv_append, attn_kvcache, cross_attn
    wan_model._fusable = lambda x: False


def run_single_gpu(args):
    from streamdiffusionv2_b200 import ops
    if args.impl == "library":
        use_library_ops()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks = measured_peaks()
    pipe = build_pipeline(device)
    g = torch.Generator(device="cpu").manual_seed(2)
    h, w = LATENT_HW
    first = torch.randn(1, 1 + FRAMES_PER_CHUNK, 16, h, w, generator=g).to(device=device, dtype=torch.bfloat16)
    n_host = 8
    host_chunks = [torch.randn(1, FRAMES_PER_CHUNK, 16, h, w, generator=g).to(torch.bfloat16).pin_memory()
                   for _ in range(n_host)]
    dev_chunks = [c.to(device) for c in host_chunks]
    host_out = torch.empty(FRAMES_PER_CHUNK, 16, h, w, dtype=torch.bfloat16).pin_memory()
    sched = ChunkSchedule()

    with torch.no_grad():
        pipe.prepare(text_prompts=["synthetic"], device=device, dtype=torch.bfloat16, noise=first, current_start=0,
                     current_end=FRAME_TOKENS * (1 + FRAMES_PER_CHUNK))
        if args.graphs and args.impl == "ours":
            pipe.enable_step_graphs()      # steady-state steps replay the DiT forward from a CUDA graph
        fill = 0
        while min(pipe.kv_cache1[0]["_sdv2_host"].local_end) < CACHE_FRAMES * FRAME_TOKENS or fill < 11:
            cs, ce = sched.next()
            pipe.inference_stream(dev_chunks[fill % n_host], cs, ce)
            fill += 1
        for i in range(args.warmup):
            cs, ce = sched.next()
            pipe.inference_stream(dev_chunks[i % n_host], cs, ce)
        torch.cuda.synchronize()
        ops.read_status(device)

        # ---- timed region 1: inputs resident in HBM
        log = ops.LaunchLog(timed=not args.graphs)
        ops.set_launch_log(log)
        sampler = ClockSampler(0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_push("timed")        # lets a profiler select the launches of the timed region
        e0.record()
        for i in range(args.steps):
            cs, ce = sched.next()
            pipe.inference_stream(dev_chunks[i % n_host], cs, ce)
        e1.record()
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_pop()
        clocks = sampler.stop()
        ops.set_launch_log(None)
        ms = e0.elapsed_time(e1)
        ops.read_status(device)

        # ---- timed region 2: host buffers in, host result out, every step
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e2.record()
        for i in range(args.steps):
            cs, ce = sched.next()
            x = host_chunks[i % n_host].to(device, non_blocking=True)
            out = pipe.inference_stream(x, cs, ce)
            host_out.copy_(out[-1], non_blocking=True)
        e3.record()
        torch.cuda.synchronize()
        ms_e2e = e2.elapsed_time(e3)
        ops.read_status(device)

        # ---- per-kernel durations: launches inside a graph cannot be bracketed by events, so the
        # same steps are run once more from Python with every launch of ours timed
        tlog = log
        if args.graphs:
            graphs, pipe.step_graphs = pipe.step_graphs, None
            tlog = ops.LaunchLog(timed=True)
            ops.set_launch_log(tlog)
            for i in range(min(args.steps, 6)):
                cs, ce = sched.next()
                pipe.inference_stream(dev_chunks[i % n_host], cs, ce)
            torch.cuda.synchronize()
            ops.set_launch_log(None)
            pipe.step_graphs = graphs

    launches = sum(log.counts.values())
    att = tlog.durations_ms("attn_kvcache")
    app = tlog.durations_ms("rope_kv_append")
    att_ms = statistics.mean(att)
    att_flops = log.work["attn_kvcache"] / log.counts["attn_kvcache"]
    app_ms = statistics.mean(app)
    app_bytes = log.work["rope_kv_append"] / log.counts["rope_kv_append"]
    fps = VIDEO_FRAMES_PER_CHUNK * args.steps / (ms / 1e3)
    fps_e2e = VIDEO_FRAMES_PER_CHUNK * args.steps / (ms_e2e / 1e3)
    achieved = att_flops / (att_ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"]
    cpu = None
    if not args.no_cpu_baseline:
        times = cpu_attention_path(3, 1, 780, budget_s=40.0)
        layer_s = statistics.mean(times)
        cpu = {"value": VIDEO_FRAMES_PER_CHUNK / (layer_s * MODEL_1P3B["num_layers"]), "unit": "video frames/s",
               "cores": os.cpu_count() or 1, "kind": "port",
               "sample": f"attention path only, 1 of 30 layers, 2 cache rows, 780 of 3120 query tokens per row timed "
                         f"and scaled, {len(times)} samples; chunk time = 30 x layer time; linear layers not included"}
    line = {
        "metric": metric_name(), "value": fps, "unit": "video frames/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(1),
        "e2e": {"value": fps_e2e, "unit": "video frames/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": host_chunks[0].numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2},
        "gpu_launches": launches, "gpu_launches_by_kernel": log.counts,
        "roofline": {"kernel": "attn_kvcache (tcgen05)", "bound": "tensor", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peaks["source"] + " sustained bf16",
                     "traffic": ATTN_DRAM_BYTES_1P3B if MODEL_1P3B["dim"] == 1536 else None,
                     "traffic_note": "DRAM bytes read + written per launch, one ncu capture of this shape "
                                     "(2 rows x 12 heads x 3120 queries x 32760 keys); algorithmic K+V+Q+out = 441 MB",
                     "avg_launch_ms": att_ms, "flops_per_launch": att_flops,
                     "share_of_step": att_ms * log.counts["attn_kvcache"] / ms,
                     "timed_in": "launch-by-launch pass of the same steps after the timed region (graph replay "
                                 "hides single launches from events)" if args.graphs else "the timed region"},
        "roofline_append": {"kernel": "rope_kv_append", "bound": "hbm", "achieved": app_bytes / (app_ms * 1e-3) / 1e9,
                            "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": app_bytes / (app_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                            "avg_launch_ms": app_ms, "bytes_per_launch": app_bytes,
                            "traffic": APPEND_DRAM_BYTES_1P3B if MODEL_1P3B["dim"] == 1536 else None,
                            "traffic_note": "DRAM bytes per launch, one ncu capture of this shape from a flushed "
                                            "cache: all 57.5 MB of reads, 11.5 MB of the 57.5 MB of writes (the "
                                            "rest is still in L2 when the kernel ends)"},
        "cpu_baseline": cpu, "clocks": clocks,
        "step_graphs": None if pipe.step_graphs is None else {"replayed_steps": pipe.step_graphs.replays,
                                                              "eager_steps": pipe.step_graphs.eager_steps},
    }
    if args.impl == "library":
        line.update(impl="library", gpu_launches=0, gpu_launches_by_kernel={})
        line["roofline"]["kernel"] = "flash_attn_with_kvcache (library)"
        line["roofline_append"]["kernel"] = "fp64 complex rope chain + slice writes (PyTorch ops)"
    args.emit(line)


def run_pipeline(args):
    """N ranks = N pipeline stages over contiguous block ranges; every rank runs K chunk steps of
    its own stage, timed on the device between barriers; the slowest rank's time counts."""
    import torch.distributed as dist
    from streamdiffusionv2_b200 import ops
    from streamdiffusionv2_b200.pipeline_runner import PipelineStageRunner
    from streamdiffusionv2_b200.stage_transport import StageLink, balanced_block_ranges, contiguous_block_ranges

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl")   # lazy communicators: the stage links create theirs one edge at a time
    peaks = measured_peaks()
    pipe = build_pipeline(device)
    split = balanced_block_ranges if args.block_split == "balanced" else contiguous_block_ranges
    ranges = split(MODEL_1P3B["num_layers"], world)
    role = "input" if rank == 0 else ("output" if rank == world - 1 else "middle")
    g = torch.Generator(device="cpu").manual_seed(2)
    h, w = LATENT_HW
    first = torch.randn(1, 1 + FRAMES_PER_CHUNK, 16, h, w, generator=g).to(device=device, dtype=torch.bfloat16)
    n_host = 8
    host_chunks = [torch.randn(1, FRAMES_PER_CHUNK, 16, h, w, generator=g).to(torch.bfloat16).pin_memory()
                   for _ in range(n_host)]
    dev_chunks = [c.to(device) for c in host_chunks]
    host_out = torch.empty(FRAMES_PER_CHUNK, 16, h, w, dtype=torch.bfloat16).pin_memory()
    sched = ChunkSchedule()
    rows = len(LEVELS)
    n_tok = FRAMES_PER_CHUNK * FRAME_TOKENS

    def barrier():
        dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    with torch.no_grad():
        pipe.prepare(text_prompts=["synthetic"], device=device, dtype=torch.bfloat16, noise=first, current_start=0,
                     current_end=FRAME_TOKENS * (1 + FRAMES_PER_CHUNK), block_mode=role,
                     owned_blocks=range(ranges[rank][0], ranges[rank][1]), unowned="free")
        link = StageLink(rank, world, device, (rows, n_tok, MODEL_1P3B["dim"]),
                         (rows, FRAMES_PER_CHUNK, 16, h, w), dtype=torch.bfloat16, timeout_s=90)
        runner = PipelineStageRunner(pipe, link, rank, world, ranges, prefetch=bool(int(os.environ.get("SDV2_PREFETCH", "0"))))
        if args.graphs:
            pipe.enable_step_graphs()      # recorded at this rank's first steady step after the ring was emptied
        chunk = [0]

        def one_step(src, last=False):
            cs, ce = sched.next()
            i = chunk[0]
            chunk[0] += 1
            x = src(i) if rank == 0 else None
            return runner.step(i, x, cs, ce, None, last=last)

        def phase(n, src, sink=None, keep_full=True):
            """n chunk steps on this rank.  keep_full: the ring stays full across the barrier that
            follows - every rank pauses with the packet for its next step already received and its
            own send completed (`park`), so the device synchronise cannot wait on a peer and the
            next phase starts in steady state.  Otherwise the ring is emptied (`quiesce`)."""
            for j in range(n):
                out = one_step(src, last=(j == n - 1))
                if sink is not None and out is not None:
                    sink(out)
            runner.park() if keep_full else runner.quiesce()

        resident = lambda i: dev_chunks[i % n_host]
        phase(12 + world, resident, keep_full=False)      # fill the K/V caches until they wrap
        # warm-up, staggered: rank r stops r chunks behind rank 0, which is where a running stream
        # has it; from here on every rank runs the same number of steps per phase
        phase(max(args.warmup, 1) + (world - 1 - rank), resident)
        barrier()
        ops.read_status(device)

        log = ops.LaunchLog(timed=not args.graphs)
        ops.set_launch_log(log)
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        runner.stage_events = []
        e0.record()
        phase(args.steps, resident)                       # K steps on every rank; K chunks enter, K leave
        e1.record()
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        ops.set_launch_log(None)
        ms = e0.elapsed_time(e1)
        stage_ms = statistics.mean(a.elapsed_time(b) for a, b in runner.stage_events)
        runner.stage_events = None

        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e2.record()
        phase(args.steps, lambda i: host_chunks[i % n_host].to(device, non_blocking=True),
              sink=lambda out: host_out.copy_(out[-1], non_blocking=True))
        e3.record()
        barrier()
        ms_e2e = e2.elapsed_time(e3)
        ops.read_status(device)

        tlog = log
        if args.graphs:                    # per-kernel durations: a launch-by-launch pass of the same steps
            graphs, pipe.step_graphs = pipe.step_graphs, None
            tlog = ops.LaunchLog(timed=True)
            ops.set_launch_log(tlog)
            phase(4, resident)
            barrier()
            ops.set_launch_log(None)
            pipe.step_graphs = graphs

    att = tlog.durations_ms("attn_kvcache")
    stats = torch.tensor([ms, ms_e2e, float(sum(log.counts.values())), statistics.mean(att) if att else 0.0],
                         dtype=torch.float64, device=device)
    mx = stats.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    per_stage = [torch.zeros(1, dtype=torch.float64, device=device) for _ in range(world)]
    dist.all_gather(per_stage, torch.tensor([stage_ms], dtype=torch.float64, device=device))
    sm = stats.clone()
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    if rank == 0:
        ms_max, ms_e2e_max = mx[0].item(), mx[1].item()
        att_ms = sm[3].item() / world
        att_flops = tlog.work["attn_kvcache"] / tlog.counts["attn_kvcache"]
        achieved = att_flops / (att_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops_sustained"]
        line = {
            "metric": metric_name(), "value": VIDEO_FRAMES_PER_CHUNK * args.steps / (ms_max / 1e3),
            "unit": "video frames/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": VIDEO_FRAMES_PER_CHUNK * args.steps / (ms_e2e_max / 1e3), "unit": "video frames/s",
                    "ms_per_step": ms_e2e_max / args.steps, "h2d_bytes_per_step": host_chunks[0].numel() * 2,
                    "d2h_bytes_per_step": host_out.numel() * 2},
            "gpu_launches": int(sm[2].item()),
            "roofline": {"kernel": "attn_kvcache (tcgen05)", "bound": "tensor", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peaks["source"] + " sustained bf16",
                         "traffic": None, "avg_launch_ms": att_ms, "flops_per_launch": att_flops},
            "cpu_baseline": None, "clocks": clocks,
            "stage_blocks": ranges, "stage_compute_ms": [round(t.item(), 3) for t in per_stage], "stage_hop_bytes": rows * n_tok * MODEL_1P3B["dim"] * 2,
        }
        args.emit(line)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library"],
                    help="reference: the CPU restatement on the host cores; library: comparison arm, N=1 only, "
                         "the reference's GPU op chain (flash-attn, PyTorch ops) under the same model")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graphs", dest="graphs", action="store_false",
                    help="launch every op of every step from Python instead of replaying steady steps from a CUDA graph")
    ap.add_argument("--block-split", default="reference", choices=["reference", "balanced"],
                    help="N>1: the reference's default block ranges (remainder on the first stages) or the "
                         "remainder on the middle stages")
    ap.add_argument("--model", default="1.3b", choices=["1.3b", "14b"],
                    help="1.3b is the headline workload; 14b = 40 blocks, dim 5120, 40 heads, 4 denoise levels")
    args = ap.parse_args()
    if args.model == "14b":
        MODEL_1P3B.update(dim=5120, ffn_dim=13824, num_heads=40, num_layers=40)
        LEVELS[:] = [1000, 750, 500, 250]
    args.warmup = max(args.warmup, 0)
    # Libraries (NCCL's version banner, for one) write to stdout; the contract is ONE JSON line
    # there, so everything but that line goes to stderr.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    args.emit = lambda line: os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return run_single_gpu(args)
    if args.impl == "library":
        raise SystemExit("--impl library is a single-GPU comparison")
    return run_pipeline(args)


if __name__ == "__main__":
    main()

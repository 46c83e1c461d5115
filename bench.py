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
ATTN_DRAM_BYTES_1P3B = 448.0e6 + 14.7e6
APPEND_DRAM_BYTES_1P3B = 57.59e6 + 8.88e6
FRAMES_PER_CHUNK = 2
VIDEO_FRAMES_PER_CHUNK = 4 * FRAMES_PER_CHUNK
SINK_FRAMES = 1
ADAPT_SINK_THRESHOLD = -1    # > -1: sink frames are refreshed when the new frame drifts away from them
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
# CPU arm: the reference's attention path on the host cores
# ---------------------------------------------------------------------------------------------

def _cpu_layer(H, rows, dtype, total_steps):
    """(call, kind): one full-size call of the cached self-attention path on CPU tensors - rope,
    ring slot write, index update, attention over the whole cache.  The reference's own
    CausalWanSelfAttention module when the reference is installed beside the benchmark
    (baseline/_ref), else the oracle's restatement of it."""
    from oracle import causal_attention_oracle as orc
    from oracle.reference_shim import import_reference, reference_root
    D, smax = 128, CACHE_FRAMES * FRAME_TOKENS
    root = reference_root()
    if root is not None:
        ref = import_reference(root, flash_attn=False)      # flash-attn has no CPU kernels
        layer = ref.cm.CausalWanSelfAttention(dim=H * D, num_heads=H, qk_norm=False)

        class Feed(torch.nn.Module):                        # q/k/v arrive projected: the path starts after the GEMMs
            value = None

            def forward(self, x):
                return self.value

        layer.q, layer.k, layer.v, layer.o = Feed(), Feed(), Feed(), torch.nn.Identity()
        layer.sink_size, layer.adapt_sink_thr = 1, -1
        table = orc.rope_table(D)
        kv = {"k": torch.zeros(rows, smax, H, D, dtype=dtype), "v": torch.zeros(rows, smax, H, D, dtype=dtype),
              "global_end_index": torch.zeros(rows, dtype=torch.long),
              "local_end_index": torch.zeros(rows, dtype=torch.long),
              "total_steps": total_steps, "current_step": total_steps}

        def call(q, k, v, starts, frames):
            n = frames * FRAME_TOKENS
            layer.q.value, layer.k.value, layer.v.value = (t.flatten(2) for t in (q, k, v))
            grid = torch.tensor([[frames, 30, 52]] * len(starts), dtype=torch.long)
            cs = torch.tensor(starts, dtype=torch.long)
            with torch.no_grad():
                return layer(torch.zeros(len(starts), n, 1, dtype=dtype), None, grid, table, None, kv, cs, cs + n)

        return call, "reference", kv, layer
    cache = orc.OracleCache.zeros(rows, smax, H, D, dtype, total_steps=total_steps)
    table = orc.rope_table(D)

    def call(q, k, v, starts, frames):
        return orc.self_attention_step(q, k, v, cache, table, (frames, 30, 52), starts, 1)[0]

    return call, "port", cache, None


def cpu_hot_path(max_steps: int, budget_s: float, layers_per_step: int):
    """Whole chunk steps of the attention path on the host cores at the N=1 workload's shape: per
    step `layers_per_step` full-size layer calls (2 cache rows x 3120 new tokens x 12 heads against
    the full 32760-token cache, bf16 tensors, fp32 math as the reference does on CPU).  Nothing is
    sub-sampled or scaled.  Runs until `max_steps` steps are done or the budget is used (at least
    one step).  Returns (seconds per step list, kind, warm-up layer calls)."""
    torch.set_num_threads(os.cpu_count() or 1)
    H, B, n_full = MODEL_1P3B["num_heads"], len(LEVELS), FRAMES_PER_CHUNK * FRAME_TOKENS
    call, kind, state, layer = _cpu_layer(H, B, torch.bfloat16, len(LEVELS))
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(B, n_full, H, 128, generator=g).to(torch.bfloat16) for _ in range(3))
    # start from a full, wrapped cache (what 11 chunks of streaming leave behind): random contents,
    # local_end = cache length, the nine ring slots queued for eviction in order
    smax = CACHE_FRAMES * FRAME_TOKENS
    queue = list(range(2 * n_full, smax + 1, n_full))
    if kind == "reference":
        state.update(k=torch.randn(B, smax, H, 128, generator=g).to(torch.bfloat16),
                     v=torch.randn(B, smax, H, 128, generator=g).to(torch.bfloat16))
        state["local_end_index"].fill_(smax)
        state["global_end_index"].fill_(smax)
        layer.evict_idx = [list(queue) for _ in range(B)]
    else:
        state.k.copy_(torch.randn(B, smax, H, 128, generator=g))
        state.v.copy_(torch.randn(B, smax, H, 128, generator=g))
        state.state.local_end = [smax] * B
        state.state.global_end = [smax] * B
        state.state.evict_idx = [list(queue) for _ in range(B)]
    sched = ChunkSchedule(first_frames=CACHE_FRAMES)
    rows = [smax] * B

    def layer_calls(n):
        nonlocal rows
        cs, _ = sched.next()
        rows = [cs] + rows[:-1]
        for _ in range(n):
            call(q, k, v, rows, FRAMES_PER_CHUNK)

    warm = 1
    layer_calls(1)
    times, t_begin = [], time.time()
    while len(times) < max_steps:
        t0 = time.time()
        layer_calls(layers_per_step)
        times.append(time.time() - t0)
        if time.time() - t_begin + times[-1] > budget_s:
            break
    return times, kind, warm


def cpu_single_layer_config(budget_s: float = 60.0):
    """The single-layer configuration on the host cores as specified: 12 heads x 128, fp32, one
    cache row of 32760 tokens, 24 steps of 3120 tokens drawn from seed 0.  Returns the median
    seconds per step and the median over the full-cache steps (10 and later)."""
    torch.set_num_threads(os.cpu_count() or 1)
    H = 12
    call, kind, _, _ = _cpu_layer(H, 1, torch.float32, 1)
    g = torch.Generator().manual_seed(0)
    times, t_begin = [], time.time()
    for s in range(24):
        q, k, v = (torch.randn(1, 3120, H * 128, generator=g).view(1, 3120, H, 128) for _ in range(3))
        t0 = time.time()
        call(q, k, v, [3120 * s], 2)
        times.append(time.time() - t0)
        if time.time() - t_begin > budget_s:
            break
    steady = times[10:]
    return {"kind": kind, "steps_run": len(times), "median_step_s": statistics.median(times),
            "steady_state_median_s": statistics.median(steady) if steady else None, "cores": os.cpu_count() or 1,
            "config": "1 layer, 12 heads x 128, fp32, 1 row, 32760-token cache, 24 steps x 3120 tokens, seed 0"}


def cpu_baseline_leg(max_steps: int, budget_s: float):
    times, kind, warm = cpu_hot_path(max_steps, budget_s, MODEL_1P3B["num_layers"])
    step_s = statistics.median(times)
    return {"value": VIDEO_FRAMES_PER_CHUNK / step_s, "unit": "video frames/s", "cores": os.cpu_count() or 1,
            "kind": kind, "steps_run": len(times), "s_per_step": step_s,
            "sample": f"{len(times)} whole chunk step(s) of the attention path: {MODEL_1P3B['num_layers']} full-size "
                      f"layer calls each (rope + ring slot write + attention of 2 rows x 3120 queries over the full "
                      f"32760-token cache, full and wrapping), nothing sub-sampled or scaled; {warm} layer call of warm-up; "
                      "GEMMs, norms and FFN are outside the path and not included"}, times


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU implementation of the path on the host cores, all
    threads.  One step = one whole chunk step of the attention path (see cpu_hot_path); as many of
    the requested steps as fit in the time budget are run, and `steps` / `ms_per_step` say what
    was run and measured."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, times = cpu_baseline_leg(max(args.steps, 1), args.cpu_budget)
    fps = base["value"]
    base["single_layer_config"] = cpu_single_layer_config(40.0)
    line = {"impl": "reference", "metric": metric_name(), "value": fps, "unit": "video frames/s",
            "n_gpus": args.gpus, "steps": len(times), "warmup": 0, "ms_per_step": base["s_per_step"] * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 storage, fp32 math",
            "data": "synthetic", "config": workload_config(args.gpus), "cpu_baseline": base,
            "e2e": {"value": fps, "unit": "video frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "steps_requested": args.steps, "warmup_requested": args.warmup,
            "note": "warm-up is one full-size layer call, not whole steps; steps = whole steps actually run "
                    "inside the time budget"}
    args.emit(line)


def metric_name():
    return "streaming_fps_480x832_wan1.3b" if MODEL_1P3B["dim"] == 1536 else "streaming_fps_480x832_wan14b"


def workload_config(n_gpus: int):
    name = "Wan-1.3B" if MODEL_1P3B["dim"] == 1536 else "Wan-14B"
    adaptive = f", adaptive sink refresh below {ADAPT_SINK_THRESHOLD}" if ADAPT_SINK_THRESHOLD > -1 else ""
    return {"workload": f"random-init causal {name} DiT, 480x832, {len(LEVELS)} denoise levels ({len(LEVELS)} cache "
                        f"rows), {FRAMES_PER_CHUNK} latent frame(s) per chunk, {SINK_FRAMES} sink + "
                        f"{CACHE_FRAMES - SINK_FRAMES} ring frame cache, full and wrapping{adaptive}",
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
                          kw["num_layers"], kw["num_heads"], FRAME_TOKENS, CACHE_FRAMES, SINK_FRAMES, ADAPT_SINK_THRESHOLD,
                          FRAMES_PER_CHUNK, device=device)
    return pipe


class ChunkSchedule:
    """Chunk starts as the reference's drivers advance them, with the refresh rule
    (streamv2v/inference.py:234-252).  The first chunk (`first_frames`) was taken by prepare()."""

    def __init__(self, first_frames=None):
        first_frames = 1 + FRAMES_PER_CHUNK if first_frames is None else first_frames
        self.start = FRAME_TOKENS * first_frames
        self.end = self.start + FRAMES_PER_CHUNK * FRAME_TOKENS

    def next(self):
        if self.start // FRAME_TOKENS >= 50:
            self.start = CACHE_FRAMES * FRAME_TOKENS - FRAME_TOKENS
            self.end = self.start + FRAMES_PER_CHUNK * FRAME_TOKENS
        cur = (self.start, self.end)
        self.start = self.end
        self.end += FRAMES_PER_CHUNK * FRAME_TOKENS
        return cur


def use_library_ops(attention="flash_attn"):
    """Fallback comparison arm for boxes where the reference itself is not installed: this package's
    model and stream with the three cache kernels replaced by the calls the reference makes on a GPU
    - the fp64 complex rope chain with slice writes into the cache (models/wan/causal_model.py:94-108,
    321-322), flash_attn_with_kvcache (:353-358) or PyTorch SDPA (:111-157), flash_attn_func / SDPA for
    the text cross-attention - and the block's norm / modulation / gate chains as separate PyTorch
    ops.  The slot bookkeeping stays ours (host integers, no device read-backs), so this arm is an
    upper bound on the reference's own loop.  Library kernels only: `gpu_launches` is 0.
    Returns a function that restores the package's own ops."""
    import torch.nn.functional as F
    from streamdiffusionv2_b200 import ops, wan_model
    saved = (ops.rope_kv_append, ops.attn_kvcache, ops.cross_attn, wan_model._fusable)
    if attention == "flash_attn":
        from flash_attn import flash_attn_func, flash_attn_with_kvcache

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
        lens = [int(x) for x in seq_lens[:B]]
        with ops._Logged("attn_kvcache", 4.0 * n * D * H * float(sum(lens))):
            if attention == "flash_attn":
                lt = torch.tensor(lens, dtype=torch.int32, device=q.device)
                return flash_attn_with_kvcache(q, k_cache, v_cache, cache_seqlens=lt, softmax_scale=softmax_scale)
            if all(x == k_cache.shape[1] for x in lens):
                return F.scaled_dot_product_attention(q.transpose(1, 2), k_cache.transpose(1, 2),
                                                      v_cache.transpose(1, 2)).transpose(1, 2).contiguous()
            return torch.cat([F.scaled_dot_product_attention(
                q[b:b + 1].transpose(1, 2), k_cache[b:b + 1, :x].transpose(1, 2),
                v_cache[b:b + 1, :x].transpose(1, 2)).transpose(1, 2) for b, x in enumerate(lens)]).contiguous()

    def cross_attn(q, k, v, *, out=None, softmax_scale=None):
        B = q.shape[0]
        with ops._Logged("cross_attn", 4.0 * B * q.shape[1] * q.shape[3] * q.shape[2] * k.shape[1]):
            if attention == "flash_attn":
                return flash_attn_func(q, k.expand(B, -1, -1, -1), v.expand(B, -1, -1, -1), softmax_scale=softmax_scale)
            return F.scaled_dot_product_attention(q.transpose(1, 2), k.expand(B, -1, -1, -1).transpose(1, 2),
                                                  v.expand(B, -1, -1, -1).transpose(1, 2)).transpose(1, 2).contiguous()

    ops.rope_kv_append, ops.attn_kvcache, ops.cross_attn = rope_kv_append, attn_kvcache, cross_attn
    wan_model._fusable = lambda x: False

    def restore():
        ops.rope_kv_append, ops.attn_kvcache, ops.cross_attn, wan_model._fusable = saved
    return restore


def _stream_fps(pipe, device, steps, warmup, dev_chunks, first, fill_until_wrapped):
    """prepare + fill + warm-up + `steps` timed chunk steps of a streaming pipeline object (this
    package's or the reference's: same method names and arguments).  Returns ms per step."""
    sched = ChunkSchedule()
    with torch.no_grad():
        pipe.prepare(text_prompts=["synthetic"], device=device, dtype=torch.bfloat16, noise=first, current_start=0,
                     current_end=FRAME_TOKENS * (1 + FRAMES_PER_CHUNK))
        for i in range(fill_until_wrapped + warmup):
            cs, ce = sched.next()
            pipe.inference_stream(noise=dev_chunks[i % len(dev_chunks)], current_start=cs, current_end=ce,
                                  current_step=None)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(steps):
            cs, ce = sched.next()
            pipe.inference_stream(noise=dev_chunks[i % len(dev_chunks)], current_start=cs, current_end=ce,
                                  current_step=None)
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def reference_gpu_arms(device, steps, warmup, dev_chunks, first):
    """The reference's GPU path on the same workload, same box, same process, a few steps each.
    With the reference installed beside the benchmark (baseline/_ref = `pip install --no-deps
    --target`, unmodified): its own CausalWanModel under its own CausalStreamInferencePipeline,
    (1) stock, i.e. flash_attn_with_kvcache / flash_attention where flash-attn imports,
    (2) with flash-attn treated as absent, i.e. its PyTorch SDPA paths
    (models/wan/causal_model.py:111-157, 373-384), and (3) the same classes after `install()`.
    Without it: this package's model with the reference's op chain patched in (use_library_ops)."""
    import gc
    from oracle.reference_shim import build_reference_pipeline, import_reference, reference_root
    out = {"steps": steps, "warmup": warmup}
    root = reference_root()
    g = torch.Generator(device="cpu").manual_seed(1)
    prompt = torch.randn(1, 512, MODEL_1P3B["text_dim"], generator=g)

    def init(model):
        torch.nn.init.normal_(model.head.head.weight, std=0.02)

    def run(label, flash, patch):
        try:
            if root is not None:
                ref = import_reference(root, flash_attn=flash)
                if flash and not ref.cm.FLASH_ATTN_AVAILABLE:
                    out[label] = {"unavailable": "flash-attn does not import on this box"}
                    return
                torch.manual_seed(0)
                pipe = build_reference_pipeline(ref, MODEL_1P3B, LEVELS, FRAME_TOKENS, CACHE_FRAMES, SINK_FRAMES,
                                                FRAMES_PER_CHUNK, prompt, device=device, dtype=torch.bfloat16,
                                                init_parameters=init, construct_on_device=True)
                pipe.adapt_sink_threshold = ADAPT_SINK_THRESHOLD
                if patch:
                    from streamdiffusionv2_b200.causal_attention import install
                    install(pipe.generator.model)
                ms = _stream_fps(pipe, device, steps, warmup, dev_chunks, first, 12)
            else:
                restore = use_library_ops("flash_attn" if flash else "sdpa")
                try:
                    ms = _stream_fps(build_pipeline(device), device, steps, warmup, dev_chunks, first, 12)
                finally:
                    restore()
            out[label] = {"value": VIDEO_FRAMES_PER_CHUNK / (ms / 1e3), "unit": "video frames/s", "ms_per_step": ms}
        except Exception as e:                       # a comparison arm must not take the benchmark down
            out[label] = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}
        finally:
            pipe = None
            gc.collect()
            torch.cuda.empty_cache()

    out["source"] = ("unmodified reference installed under baseline/_ref, its own model and streaming pipeline"
                     if root is not None else
                     "reference not installed on this box: this package's model with the reference's GPU op chain")
    run("stock_flash_attn", True, False)
    run("sdpa_fallback", False, False)
    if root is not None:
        run("with_install", False, True)
    arms = {k: v["value"] for k, v in out.items() if isinstance(v, dict) and "value" in v and k != "with_install"}
    if arms:
        out["faster"] = max(arms, key=arms.get)
        out["faster_value"] = arms[out["faster"]]
    return out


class LatencyStamps:
    """Per-chunk latency under back-to-back load, on the device's own clock: an event when a
    chunk's input copy is enqueued, an event after the copy of a step's result to the host."""

    def __init__(self):
        self.t_in, self.t_out = [], []

    def enter(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.t_in.append(e)

    def leave(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.t_out.append(e)

    def latencies_ms(self, lag):
        """Chunk entering at step i is final (last denoise level, on the host) after step i + lag."""
        return [self.t_in[i].elapsed_time(self.t_out[i + lag]) for i in range(len(self.t_in) - lag)]


def _median(xs):
    return statistics.median(xs) if xs else None


def run_single_gpu(args):
    from streamdiffusionv2_b200 import ops
    restore = use_library_ops() if args.impl == "library" else None
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
    levels = len(LEVELS)

    def timed(n, body):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(n):
            body(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

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

        def resident_step(i):
            cs, ce = sched.next()
            pipe.inference_stream(dev_chunks[i % n_host], cs, ce)

        for i in range(args.warmup):
            resident_step(i)
        torch.cuda.synchronize()
        ops.read_status(device)

        # ---- timed region 1: inputs resident in HBM.  Exactly K steps per region; the region is
        # repeated until the regions together cover about two seconds, and the median counts.
        log = ops.LaunchLog(timed=not args.graphs)
        ops.set_launch_log(log)
        sampler = ClockSampler(0)
        sampler.start()
        torch.cuda.nvtx.range_push("timed")        # lets a profiler select the launches of the timed region
        regions = [timed(args.steps, resident_step)]
        ops.set_launch_log(None)
        # at least three regions, so that the median survives one disturbed region
        repeats = max(min(3, args.max_repeats),
                      min(args.max_repeats, -(-int(args.min_seconds * 1e3) // max(int(regions[0]), 1))))
        for _ in range(repeats - 1):
            regions.append(timed(args.steps, resident_step))
        torch.cuda.nvtx.range_pop()
        clocks = sampler.stop()
        ms = statistics.median(regions)
        ops.read_status(device)

        # ---- timed region 2: host buffers in, host result out, every step; per-chunk latency
        stamps = LatencyStamps()

        def host_step(i):
            cs, ce = sched.next()
            stamps.enter()
            x = host_chunks[i % n_host].to(device, non_blocking=True)
            out = pipe.inference_stream(x, cs, ce)
            host_out.copy_(out[-1], non_blocking=True)      # the row that just finished its last denoise level
            stamps.leave()

        regions_e2e = [timed(args.steps, host_step) for _ in range(repeats)]
        ms_e2e = statistics.median(regions_e2e)
        lat = stamps.latencies_ms(levels - 1)
        ops.read_status(device)

        # ---- per-kernel durations: launches inside a graph cannot be bracketed by events, so the
        # same steps are run once more from Python with every launch of ours timed
        tlog = log
        if args.graphs:
            graphs, pipe.step_graphs = pipe.step_graphs, None
            tlog = ops.LaunchLog(timed=True)
            ops.set_launch_log(tlog)
            for i in range(min(args.steps, 6)):
                resident_step(i)
            torch.cuda.synchronize()
            ops.set_launch_log(None)
            pipe.step_graphs = graphs

        ref_gpu = None
        if args.impl == "ours" and not args.no_reference_gpu:
            ref_gpu = reference_gpu_arms(device, args.reference_steps, 2, dev_chunks, first)

    launches = sum(log.counts.values())
    att = tlog.durations_ms("attn_kvcache")
    app = tlog.durations_ms("rope_kv_append")
    crs = tlog.durations_ms("cross_attn")
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
        cpu, _ = cpu_baseline_leg(1, 1.0)
        cpu["single_layer_config"] = cpu_single_layer_config(30.0)
    line = {
        "metric": metric_name(), "value": fps, "unit": "video frames/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(1),
        "repeats": repeats, "region_ms": [round(r, 3) for r in regions],
        "e2e": {"value": fps_e2e, "unit": "video frames/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": host_chunks[0].numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2,
                "region_ms": [round(r, 3) for r in regions_e2e]},
        "latency_ms": {"median": _median(lat), "max": max(lat) if lat else None, "chunks": len(lat),
                       "definition": "per chunk under back-to-back load, device clock: from the enqueue of the "
                                     "chunk's host->device copy to the completion of the device->host copy of its "
                                     f"last denoise level ({levels} levels = {levels} chunk steps in the stream batch)"},
        "gpu_launches": launches, "gpu_launches_by_kernel": log.counts,
        "roofline": {"kernel": "attn_kvcache (tcgen05)", "bound": "tensor", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peaks["source"] + " sustained bf16",
                     "traffic": ATTN_DRAM_BYTES_1P3B if MODEL_1P3B["dim"] == 1536 and CACHE_FRAMES == 21 else None,
                     "traffic_note": "DRAM bytes read + written per launch, one ncu capture of this shape "
                                     "(2 rows x 12 heads x 3120 queries x 32760 keys); algorithmic K+V+Q+out = 441 MB",
                     "avg_launch_ms": att_ms, "flops_per_launch": att_flops,
                     "share_of_step": att_ms * log.counts["attn_kvcache"] / regions[0],
                     "timed_in": "launch-by-launch pass of the same steps after the timed region (graph replay "
                                 "hides single launches from events)" if args.graphs else "the timed region"},
        "roofline_append": {"kernel": "rope_kv_append with the q/k RMS norm folded in (one launch where the unfused "
                                      "block ran the append and two norm launches: 192 MB of traffic instead of 115 MB)",
                            "bound": "hbm", "achieved": app_bytes / (app_ms * 1e-3) / 1e9,
                            "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": app_bytes / (app_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                            "avg_launch_ms": app_ms, "bytes_per_launch": app_bytes,
                            "traffic": APPEND_DRAM_BYTES_1P3B if MODEL_1P3B["dim"] == 1536 and FRAMES_PER_CHUNK == 2 else None,
                            "traffic_note": "DRAM bytes per launch, one ncu capture of this shape from a flushed "
                                            "cache: all 57.5 MB of reads, 8.9 MB of the 57.5 MB of writes (the "
                                            "rest is still in L2 when the kernel ends); with the norm the launch is "
                                            "bound by the f32<->f64 conversion unit (64 % busy), not by HBM; the "
                                            "plain append kernel reaches 0.59 of the HBM peak at this shape and 0.85 "
                                            "at 4 rows x 40 heads (kernel_bench.py)"},
        "cross_attn": {"avg_launch_ms": statistics.mean(crs) if crs else None,
                       "tflops": (tlog.work["cross_attn"] / tlog.counts["cross_attn"]) / (statistics.mean(crs) * 1e-3) / 1e12
                       if crs else None},
        "cpu_baseline": cpu, "clocks": clocks,
        "step_graphs": None if pipe.step_graphs is None else {"replayed_steps": pipe.step_graphs.replays,
                                                              "eager_steps": pipe.step_graphs.eager_steps},
    }
    if ref_gpu is not None:
        line["reference_gpu"] = ref_gpu
        if ref_gpu.get("faster_value"):
            line["speedup_vs_reference_gpu"] = fps / ref_gpu["faster_value"]
            if isinstance(ref_gpu.get("with_install"), dict) and "value" in ref_gpu["with_install"]:
                line["dropin_speedup_vs_reference_gpu"] = ref_gpu["with_install"]["value"] / ref_gpu["faster_value"]
    if args.impl == "library":
        restore()
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
    # "measured" starts on the reference's split and re-plans from measured costs once the caches are full
    split = balanced_block_ranges if args.block_split == "balanced" else contiguous_block_ranges
    ranges = split(MODEL_1P3B["num_layers"], world)
    measured = args.block_split.startswith("measured")
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

        def region(src, sink=None):
            """Exactly K chunk steps on every rank between two barriers; device time of this rank."""
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            phase(args.steps, src, sink)                  # K steps on every rank; K chunks enter, K leave
            e1.record()
            barrier()
            return e0.elapsed_time(e1)

        def max_over_ranks(values):
            t = torch.tensor(values, dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.tolist()

        reference_split = None
        if measured:
            # one region on the reference's split (kept in the record), then three launch-by-launch steps
            # with every half block timed, one all-gather, the exact partition, blocks moved with their K/V
            runner.stage_events = []
            ref_ms = max_over_ranks([region(resident)])[0]
            ref_stage = statistics.median(a.elapsed_time(b) for a, b in runner.stage_events)
            per_stage = [torch.zeros(1, dtype=torch.float64, device=device) for _ in range(world)]
            dist.all_gather(per_stage, torch.tensor([ref_stage], dtype=torch.float64, device=device))
            reference_split = {"stage_blocks": [list(r) for r in runner.block_ranges],
                               "value": VIDEO_FRAMES_PER_CHUNK * args.steps / (ref_ms / 1e3),
                               "ms_per_step": ref_ms / args.steps,
                               "stage_compute_ms": [round(t.item(), 3) for t in per_stage]}
            runner.stage_events = None
            runner.measure_costs(3)
            # rank r is r chunks behind rank 0 here; r extra steps bring every stage to the same chunk,
            # which is what moving K/V state between stages requires
            phase(3 + rank, resident, keep_full=False)
            planned = runner.plan_ranges("block" if args.block_split == "measured-blocks" else "half")
            runner.rebalance(planned, halves=True)
            phase(max(args.warmup, 1) + 2 + (world - 1 - rank), resident)     # re-record graphs, stagger again
            barrier()
            ops.read_status(device)

        log = ops.LaunchLog(timed=not args.graphs)
        ops.set_launch_log(log)
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        runner.stage_events = []
        first_ms = max_over_ranks([region(resident)])[0]
        ops.set_launch_log(None)
        # repeat the region until the regions cover about two seconds (same count on every rank)
        # (at least three, so that the median survives one disturbed region)
        repeats = max(min(3, args.max_repeats),
                      min(args.max_repeats, -(-int(args.min_seconds * 1e3) // max(int(first_ms), 1))))
        regions = [first_ms] + max_over_ranks([region(resident) for _ in range(repeats - 1)])
        clocks = sampler.stop() if rank == 0 else None
        ms = statistics.median(regions)
        stage_ms = statistics.median(a.elapsed_time(b) for a, b in runner.stage_events)  # a step that records its graph is an outlier
        runner.stage_events = None

        # host buffers in, host result out, every step; chunk latency from wall-clock-anchored device events:
        # rank 0 stamps a chunk's entry, the last rank the arrival of its final denoise level on the host
        stamps = LatencyStamps()
        anchor = torch.cuda.Event(enable_timing=True)

        def host_src(i):
            stamps.enter()
            return host_chunks[i % n_host].to(device, non_blocking=True)

        def host_sink(out):
            host_out.copy_(out[-1], non_blocking=True)
            stamps.leave()

        barrier()
        anchor.record()
        anchor.synchronize()
        anchor_wall = time.time()
        chunk_at_anchor = chunk[0]
        regions_e2e = max_over_ranks([region(host_src, host_sink) for _ in range(repeats)])
        ms_e2e = statistics.median(regions_e2e)
        ops.read_status(device)
        # wall-clock time (one node, one clock) of every stamp, indexed by this rank's chunk counter
        n_slots = repeats * args.steps
        mine = torch.full((2, n_slots), float("nan"), dtype=torch.float64, device=device)
        for row, evs in ((0, stamps.t_in), (1, stamps.t_out)):
            for j, ev in enumerate(evs[:n_slots]):
                mine[row, j] = anchor_wall + anchor.elapsed_time(ev) / 1e3
        first_chunk = torch.tensor([float(chunk_at_anchor)], dtype=torch.float64, device=device)
        all_stamps = [torch.zeros_like(mine) for _ in range(world)]
        all_first = [torch.zeros_like(first_chunk) for _ in range(world)]
        dist.all_gather(all_stamps, mine)
        dist.all_gather(all_first, first_chunk)
        lat = []
        if rank == 0:
            t_in, c_in = all_stamps[0][0].tolist(), int(all_first[0].item())
            t_out, c_out = all_stamps[world - 1][1].tolist(), int(all_first[world - 1].item())
            # a chunk that enters as chunk c leaves the last stage with its final level as the last row of the
            # stage batch of chunk c + (levels - 1) * world (it re-enters stage 0 `world` chunks later per level)
            lag = (rows - 1) * world
            for j, t0 in enumerate(t_in):
                k = (c_in + j + lag) - c_out
                same_region = 0 <= k < n_slots and (j // args.steps) == (k // args.steps)
                if same_region and t0 == t0 and t_out[k] == t_out[k]:
                    lat.append((t_out[k] - t0) * 1e3)

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
            "repeats": repeats, "region_ms": [round(r, 3) for r in regions],
            "e2e": {"value": VIDEO_FRAMES_PER_CHUNK * args.steps / (ms_e2e_max / 1e3), "unit": "video frames/s",
                    "ms_per_step": ms_e2e_max / args.steps, "h2d_bytes_per_step": host_chunks[0].numel() * 2,
                    "d2h_bytes_per_step": host_out.numel() * 2, "region_ms": [round(r, 3) for r in regions_e2e]},
            "latency_ms": {"median": _median(lat), "max": max(lat) if lat else None, "chunks": len(lat),
                           "definition": "per chunk under back-to-back load: from the enqueue of the chunk's "
                                         "host->device copy on stage 0 to the completion, on the last stage, of the "
                                         "device->host copy of its last denoise level; device events anchored to the "
                                         f"node's wall clock on each rank; the chunk crosses the {world} stages once "
                                         f"per denoise level ({rows} levels)"},
            "gpu_launches": int(sm[2].item()),
            "roofline": {"kernel": "attn_kvcache (tcgen05)", "bound": "tensor", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peaks["source"] + " sustained bf16",
                         "traffic": None, "avg_launch_ms": att_ms, "flops_per_launch": att_flops},
            "cpu_baseline": None, "clocks": clocks,
            "block_split": args.block_split,
            "stage_half_blocks": runner.half_ranges, "stage_blocks": [[a / 2, b / 2] for a, b in runner.half_ranges],
            "stage_compute_ms": [round(t.item(), 3) for t in per_stage],
            "stage_hop_bytes": rows * n_tok * MODEL_1P3B["dim"] * 2,
            "reference_split": reference_split,
            "measured_costs": getattr(runner, "last_costs", None),
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
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="N=1: skip the reference's GPU path (timed in the same process after this package's own)")
    ap.add_argument("--reference-steps", type=int, default=6, help="timed chunk steps per reference GPU arm")
    ap.add_argument("--cpu-budget", type=float, default=90.0, help="--impl reference: seconds of CPU work")
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="the timed region of K steps is repeated (at least three times) until the regions cover this long; "
                         "median counts")
    ap.add_argument("--max-repeats", type=int, default=8)
    ap.add_argument("--no-graphs", dest="graphs", action="store_false",
                    help="launch every op of every step from Python instead of replaying steady steps from a CUDA graph")
    ap.add_argument("--block-split", default="reference",
                    choices=["reference", "balanced", "measured", "measured-blocks"],
                    help="N>1: reference = the reference's default block ranges (remainder on the first stages); "
                         "balanced = remainder on the middle stages; measured = start on the reference's split, time "
                         "one region there, then re-plan the ranges from measured per-half-block costs (stage "
                         "boundaries may fall inside a block) and move the blocks; measured-blocks = the same with "
                         "boundaries at whole blocks")
    ap.add_argument("--workload", default="config2", choices=["config2", "v2v-default"],
                    help="config2: the headline workload (2 frames per chunk, 1 sink + 20 ring frames); v2v-default: the "
                         "reference's default video-to-video configuration (configs/wan_causal_dmd_v2v.yaml:53-56: 1 "
                         "frame per chunk, 6-frame cache, 3 sink frames refreshed adaptively below 0.2), N=1 only")
    ap.add_argument("--model", default="1.3b", choices=["1.3b", "14b"],
                    help="1.3b is the headline workload; 14b = 40 blocks, dim 5120, 40 heads, 4 denoise levels")
    args = ap.parse_args()
    if args.model == "14b":
        MODEL_1P3B.update(dim=5120, ffn_dim=13824, num_heads=40, num_layers=40)
        LEVELS[:] = [1000, 750, 500, 250]
    if args.workload == "v2v-default":
        global FRAMES_PER_CHUNK, VIDEO_FRAMES_PER_CHUNK, CACHE_FRAMES, SINK_FRAMES, ADAPT_SINK_THRESHOLD
        FRAMES_PER_CHUNK, VIDEO_FRAMES_PER_CHUNK, CACHE_FRAMES, SINK_FRAMES, ADAPT_SINK_THRESHOLD = 1, 4, 6, 3, 0.2
        args.no_cpu_baseline = True
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

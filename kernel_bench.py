"""Micro-benchmark of the cache kernels on synthetic bf16 q/k/v ~ N(0,1) (seed 0).

    python kernel_bench.py --kernel append --rows 2 --heads 12
    python kernel_bench.py --kernel attn --rows 1 --heads 12 --window-frames 21
    python kernel_bench.py --sweep            # window x heads x rows x chunk grid
    python kernel_bench.py --library-baselines   # what the reference executes on a GPU for the same steps

Prints one JSON line per configuration: time per launch (CUDA events on the launching stream,
L2 flushed between launches by writing a 256 MB buffer), append GB/s (6 x rows x tokens x heads x
128 x 2 bytes per launch) and attention TFLOP/s (4 x tokens x 128 x heads x sum of cache lengths).
A measurement script: it is not part of the package and the package never imports it.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

FRAME_TOKENS = 1560


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return statistics.median(out), min(out)


def run_config(kernel, rows, heads, window_frames, chunk_frames, iters, warmup, flush_l2=True):
    from streamdiffusionv2_b200 import ops
    from streamdiffusionv2_b200.wan_model import build_rope_table
    dev = torch.device("cuda")
    D = 128
    n = chunk_frames * FRAME_TOKENS
    s = window_frames * FRAME_TOKENS
    g = torch.Generator(device="cpu").manual_seed(0)
    mk = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16).to(dev)
    q, k, v = mk(rows, n, heads, D), mk(rows, n, heads, D), mk(rows, n, heads, D)
    kc = torch.randn(rows, s, heads, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(rows, s, heads, D, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush_l2 else None
    res = {"kernel": kernel, "rows": rows, "heads": heads, "window_frames": window_frames,
           "chunk_frames": chunk_frames}
    if kernel in ("append", "append_norm", "append_norm_sliced"):
        table = ops.rope_table_device(build_rope_table(D), dev)
        dst = [min(FRAME_TOKENS, s - n)] * rows
        extra = {}
        if kernel != "append":          # q/k RMS norm folded in; "_sliced": q, k, v are slices of one q|k|v projection
            wn = (1 + 0.1 * torch.randn(heads * D, generator=g)).to(torch.bfloat16).to(dev)
            extra["norm"] = (wn, wn.clone(), 1e-6)
            if kernel.endswith("sliced"):
                qkv = torch.stack([q, k, v], dim=2).contiguous()
                q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        fn = lambda: ops.rope_kv_append(q, k, v, kc, vc, table, (chunk_frames, 30, 52), [7] * rows, dst, q_out=out,
                                        **extra)
        med, best = _time(fn, iters, warmup, flush)
        nbytes = 6.0 * rows * n * heads * D * 2
        res.update(ms=med, ms_best=best, gbs=nbytes / med / 1e6, bytes_per_launch=nbytes)
    elif kernel == "attn":
        fn = lambda: ops.attn_kvcache(q, kc, vc, [s] * rows, out=out)
        med, best = _time(fn, iters, warmup, flush)
        fl = 4.0 * rows * n * s * D * heads
        res.update(ms=med, ms_best=best, tflops=fl / med / 1e9, flops_per_launch=fl)
    elif kernel == "cross":
        ck = mk(1, 512, heads, D).expand(rows, -1, -1, -1)
        cv = mk(1, 512, heads, D).expand(rows, -1, -1, -1)
        fn = lambda: ops.cross_attn(q, ck, cv, out=out)
        med, best = _time(fn, iters, warmup, flush)
        fl = 4.0 * rows * n * 512 * D * heads
        res.update(ms=med, ms_best=best, tflops=fl / med / 1e9, flops_per_launch=fl)
    else:
        raise ValueError(kernel)
    ops.read_status(dev)
    return res


def library_baselines(rows, heads, window_frames, chunk_frames, iters, warmup):
    """What the reference executes on a GPU for the same two steps, timed with the same protocol:
    the fp64 complex rope chain plus the K/V slice writes (models/wan/causal_model.py:94-108,
    321-322), and flash_attn_with_kvcache (:353-358) or, failing that, PyTorch SDPA (:111-157).
    Library calls only - nothing here is part of the product path."""
    import torch.nn.functional as F
    from streamdiffusionv2_b200.wan_model import build_rope_table
    dev = torch.device("cuda")
    D, n, s = 128, chunk_frames * FRAME_TOKENS, window_frames * FRAME_TOKENS
    q, k, v = (torch.randn(rows, n, heads, D, device=dev, dtype=torch.bfloat16) for _ in range(3))
    kc = torch.randn(rows, s, heads, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    table = build_rope_table(D).to(dev)
    ct, ch = 64 - 2 * (64 // 3), 64 // 3
    t, hh, ww = table.split([ct, ch, ch], dim=1)
    mult = torch.cat([t[7:7 + chunk_frames].repeat_interleave(1560, dim=0),
                      hh[:30].repeat_interleave(52, dim=0).repeat(chunk_frames, 1),
                      ww[:52].repeat(30, 1).repeat(chunk_frames, 1)], dim=-1).unsqueeze(1)

    def rope(x):
        out = x.clone()
        for i in range(rows):
            xi = torch.view_as_complex(x[i].to(torch.float64).reshape(n, heads, -1, 2))
            out[i] = torch.view_as_real(xi * mult).flatten(2).type_as(x)
        return out

    def chain():
        rq, rk = rope(q), rope(k)
        for i in range(rows):
            kc[i:i + 1, 1560:1560 + n] = rk[i:i + 1]
            vc[i:i + 1, 1560:1560 + n] = v[i:i + 1]
        return rq

    res = {"baseline": "library", "rows": rows, "heads": heads, "window_frames": window_frames,
           "chunk_frames": chunk_frames}
    med, _ = _time(chain, iters, warmup, flush)
    res["rope_append_torch_chain_ms"] = med
    res["rope_append_torch_chain_gbs"] = 6.0 * rows * n * heads * D * 2 / med / 1e6
    fl = 4.0 * rows * n * s * D * heads
    try:
        from flash_attn import flash_attn_with_kvcache
        lens = torch.full((rows,), s, dtype=torch.int32, device=dev)
        med, _ = _time(lambda: flash_attn_with_kvcache(q, kc, vc, cache_seqlens=lens), iters, warmup, flush)
        res["flash_attn_with_kvcache_ms"], res["flash_attn_with_kvcache_tflops"] = med, fl / med / 1e9
    except Exception as e:  # not installed, or no kernel for this GPU
        res["flash_attn_with_kvcache_error"] = repr(e)[:120]
    qq, kk, vv = q.transpose(1, 2), kc.transpose(1, 2), vc.transpose(1, 2)
    med, _ = _time(lambda: F.scaled_dot_product_attention(qq, kk, vv), iters, warmup, flush)
    res["torch_sdpa_ms"], res["torch_sdpa_tflops"] = med, fl / med / 1e9
    return res


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="attn", choices=["append", "append_norm", "append_norm_sliced", "attn", "cross"])
    ap.add_argument("--rows", type=int, default=2)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--window-frames", type=int, default=21)
    ap.add_argument("--chunk-frames", type=int, default=2)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--library-baselines", action="store_true")
    a = ap.parse_args(argv)
    if a.library_baselines:
        print(json.dumps(library_baselines(a.rows, a.heads, a.window_frames, a.chunk_frames, a.iters, a.warmup)))
        return
    if not a.sweep:
        print(json.dumps(run_config(a.kernel, a.rows, a.heads, a.window_frames, a.chunk_frames, a.iters, a.warmup,
                                    not a.no_flush)))
        return
    for heads in (12, 40):
        for window in (4, 8, 16, 32):
            for rows in (1, 4, 16):
                if rows * window * FRAME_TOKENS * heads * 128 * 2 * 2 > 60e9:
                    continue
                for chunk in (1, 2, 3):
                    for kernel in ("append", "attn"):
                        print(json.dumps(run_config(kernel, rows, heads, window, chunk, 5, 2)), flush=True)


if __name__ == "__main__":
    main()

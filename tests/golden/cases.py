"""Seeded inputs and call schedules shared by the fixture generator and the tests.

Nothing here touches the reference: the generator feeds these inputs to the reference and
stores its outputs; the tests feed the same inputs to the oracle and to the CUDA path.
"""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16}


def sha(t: torch.Tensor) -> str:
    """SHA-256 of a tensor's raw bytes in row-major order."""
    return hashlib.sha256(to_numpy_bits(t).tobytes()).hexdigest()


def to_numpy_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def from_numpy_bits(a: np.ndarray, dtype_name: str) -> torch.Tensor:
    if dtype_name == "torch.bfloat16":
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(a.copy())


class InputStream:
    """q, k, v ~ N(0,1) drawn in that order from one seeded CPU generator, cast to the case
    dtype.  `shared_mean` > 0 adds a per-channel offset that is redrawn every `mean_period`
    calls, so that consecutive chunks are (dis)similar on purpose for the adaptive sink test."""

    def __init__(self, case: dict):
        self.case = case
        self.g = torch.Generator().manual_seed(case["seed"])
        self.calls = 0
        self.mean = None

    def next(self, rows: int, tokens: int):
        c = self.case
        H, D = c["heads"], c["head_dim"]
        dt = DTYPES[c["dtype"]]
        out = []
        amp = c.get("shared_mean", 0.0)
        if amp and self.calls % c.get("mean_period", 4) == 0:
            self.mean = torch.randn(2, 1, 1, H, D, generator=self.g) * amp
        for j in range(3):
            t = torch.randn(rows, tokens, H, D, generator=self.g)
            if amp and j > 0:
                t = t + self.mean[j - 1]
            out.append(t.to(dt))
        self.calls += 1
        return out


def schedule(case: dict):
    """Yield the calls the reference's drivers would make.

    mode "single": one cache row; every chunk is presented `total_steps` times with the same
    start (streamv2v/inference_wo_batch-style driver and config-1 style driver).
    mode "stream": the first chunk (`first_frames`) is presented `total_steps` times to a
    one-row cache at start 0, the cache is replicated to `total_steps` rows, then every call
    shifts the rows' starts down by one and puts the new chunk in row 0
    (models/wan/causal_stream_inference.py:214-253, 265-272).
    The refresh rule of the drivers (streamv2v/inference.py:234-236) resets the start to
    (cache_frames-1)*fs once start//fs >= refresh_at."""
    h, w = case["grid_hw"]
    fs = h * w
    smax = case["cache_frames"] * fs
    ts = case["total_steps"]
    refresh = case.get("refresh_at")
    if case["mode"] == "single":
        start = 0
        for s in range(case["chunks"]):
            frames = case["first_frames"] if s == 0 else case["frames"]
            if refresh is not None and start // fs >= refresh:
                start = smax - fs
            for _ in range(ts):
                yield {"op": "call", "starts": [start], "frames": frames}
            start += frames * fs
    else:
        first = case["first_frames"]
        for _ in range(ts):
            yield {"op": "call", "starts": [0], "frames": first}
        yield {"op": "replicate", "rows": ts}
        start = first * fs
        rows = [start] * ts
        for s in range(case["chunks"]):
            if refresh is not None and start // fs >= refresh:
                start = smax - fs
            rows = [start] + rows[:-1]
            yield {"op": "call", "starts": list(rows), "frames": case["frames"]}
            start += case["frames"] * fs


def _k(**kw):
    base = dict(heads=2, head_dim=128, grid_hw=(2, 3), sink_size=1, adapt_sink_thr=-1, total_steps=1,
                mode="single", first_frames=2, frames=2, refresh_at=None, seed=0)
    base.update(kw)
    return base


# small layers whose K/V caches, index state and outputs are pinned bit-for-bit / in tolerance
KERNEL_CASES = {
    # config-1 shape in miniature: cache not a multiple of the chunk -> zero tail that is attended
    "k_fp32_single": _k(dtype="fp32", cache_frames=7, chunks=12),
    "k_bf16_single": _k(dtype="bf16", cache_frames=7, chunks=12, seed=1),
    # one row, two denoise levels per chunk: slot re-written, queue popped on the last level only
    "k_bf16_single_2level": _k(dtype="bf16", cache_frames=9, chunks=10, total_steps=2, seed=2),
    # stream-batch: 3-frame first chunk, rows lag by one chunk, overlapping slots, refresh rule
    "k_bf16_stream": _k(dtype="bf16", cache_frames=10, chunks=24, total_steps=2, mode="stream",
                        first_frames=3, refresh_at=22, seed=3),
    "k_fp32_stream3": _k(dtype="fp32", cache_frames=8, chunks=14, total_steps=3, mode="stream",
                         first_frames=3, seed=4, heads=1),
    # default video-to-video shape: one frame per chunk, 6-frame cache, 3 sink frames
    "k_bf16_1frame_sink3": _k(dtype="bf16", cache_frames=6, chunks=14, total_steps=2, mode="stream",
                              first_frames=2, frames=1, sink_size=3, seed=5),
    # no sink at all, three frames per chunk (text-to-video shape)
    "k_bf16_sink0_3frames": _k(dtype="bf16", cache_frames=9, chunks=9, first_frames=3, frames=3,
                               sink_size=0, seed=6),
    # adaptive sink refresh (data dependent queue pushes)
    "k_bf16_adaptive": _k(dtype="bf16", cache_frames=6, chunks=16, total_steps=2, mode="stream",
                          first_frames=2, frames=1, sink_size=3, adapt_sink_thr=0.2, shared_mean=1.5,
                          mean_period=5, seed=7),
    "k_fp32_adaptive_single": _k(dtype="fp32", cache_frames=6, chunks=16, first_frames=2, frames=1,
                                 sink_size=3, adapt_sink_thr=0.2, shared_mean=1.5, mean_period=3,
                                 seed=8, heads=1),
}

CROSS_CASES = {
    "x_bf16": dict(heads=2, head_dim=128, dtype="bf16", rows=2, n=24, lk=512, seed=11),
    "x_fp32": dict(heads=1, head_dim=128, dtype="fp32", rows=1, n=12, lk=512, seed=12),
}


def _t(**kw):
    base = dict(heads=1, head_dim=8, grid_hw=(30, 52), dtype="fp32", adapt_sink_thr=-1, seed=0,
                mode="single", total_steps=1, first_frames=2, frames=2, refresh_at=None)
    base.update(kw)
    return base


# index-state traces at production token counts (1560 tokens per latent frame)
TRACE_CASES = {
    "t_config1": _t(cache_frames=21, sink_size=1, chunks=24),
    "t_stream_1p3b": _t(cache_frames=21, sink_size=1, chunks=60, total_steps=2, mode="stream",
                        first_frames=3, refresh_at=50),
    "t_stream_14b_4level": _t(cache_frames=21, sink_size=1, chunks=40, total_steps=4, mode="stream",
                              first_frames=3, refresh_at=50),
    "t_v2v_default": _t(cache_frames=6, sink_size=3, chunks=60, total_steps=2, mode="stream",
                        first_frames=2, frames=1, refresh_at=50),
    "t_single_2level": _t(cache_frames=21, sink_size=1, chunks=30, total_steps=2, refresh_at=50),
    "t_t2v_3frames": _t(cache_frames=21, sink_size=0, chunks=20, first_frames=3, frames=3),
}


def load_fixture(name: str):
    z = np.load(os.path.join(HERE, f"{name}.npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    return meta, z


def load_traces():
    return json.load(open(os.path.join(HERE, "index_traces.json")))


# ---------------------------------------------------------------------------------------------
# model-level cases: a tiny causal DiT driven by the streaming scheduler
# ---------------------------------------------------------------------------------------------
import zlib  # noqa: E402

MODEL_KW = dict(model_type="t2v", patch_size=(1, 2, 2), text_len=512, in_dim=16, dim=256, ffn_dim=512,
                freq_dim=64, text_dim=64, out_dim=16, num_heads=2, num_layers=3, qk_norm=True,
                cross_attn_norm=True, eps=1e-6)

MODEL_CASES = {
    # stream batch, 2 frames per chunk, 3-frame first chunk, refresh rule kicks in
    "m_stream": dict(levels=[700, 500], frames=2, cache_frames=7, sink=1, chunks=10, latent_hw=(4, 6),
                     refresh_at=12, seed=100),
    # one frame per chunk with 3 sink frames, 3 levels
    "m_stream_1f": dict(levels=[800, 600, 400], frames=1, cache_frames=6, sink=3, chunks=9, latent_hw=(4, 6),
                        refresh_at=50, seed=101),
    # two pipeline stages (blocks [0,2) and [2,3)), one frame per chunk
    "m_stages": dict(levels=[700, 500], frames=1, cache_frames=6, sink=2, chunks=8, latent_hw=(4, 6),
                     refresh_at=50, seed=102, split=2),
}


def seed_parameters(model) -> None:
    """Deterministic weights keyed by parameter name, independent of construction order."""
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            g = torch.Generator().manual_seed(zlib.crc32(name.encode()) & 0x7FFFFFFF)
            r = torch.randn(p.shape, generator=g)
            if name.endswith("modulation"):
                p.copy_(0.2 * r)
            elif p.dim() >= 2:
                fan_in = p[0].numel()
                p.copy_(r * (0.7 / fan_in ** 0.5))
            elif "norm" in name and name.endswith("weight"):
                p.copy_(1.0 + 0.1 * r)
            else:
                p.copy_(0.02 * r)


def model_inputs(case: dict):
    """Prompt embedding, first-chunk latents and per-chunk latents for a model case."""
    g = torch.Generator().manual_seed(case["seed"])
    h, w = case["latent_hw"]
    prompt = torch.randn(1, 512, MODEL_KW["text_dim"], generator=g)
    first = torch.randn(1, 1 + case["frames"], 16, h, w, generator=g)
    chunks = [torch.randn(1, case["frames"], 16, h, w, generator=g) for _ in range(case["chunks"])]
    return prompt, first, chunks


def model_schedule(case: dict):
    """(current_start, current_end) per streamed chunk, with the drivers' refresh rule
    (streamv2v/inference.py:195-252)."""
    h, w = case["latent_hw"]
    fs = (h // 2) * (w // 2)
    smax = case["cache_frames"] * fs
    start = fs * (1 + case["frames"])
    end = start + case["frames"] * fs
    out = []
    for _ in range(case["chunks"]):
        if start // fs >= case["refresh_at"]:
            start = smax - fs
            end = start + case["frames"] * fs
        out.append((start, end))
        start = end
        end += case["frames"] * fs
    return fs, out

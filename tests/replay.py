"""Replays a golden case's call schedule through an arbitrary self-attention backend."""
from __future__ import annotations

import torch

import cases
from oracle import causal_attention_oracle as orc


def replay_oracle(case: dict):
    """Yield (step_index, q, k, v, out, cache, roped_q, seq_lens, dst) for every call."""
    H, D = case["heads"], case["head_dim"]
    dtype = cases.DTYPES[case["dtype"]]
    h, w = case["grid_hw"]
    fs = h * w
    smax = case["cache_frames"] * fs
    table = orc.rope_table(D)
    cache = orc.OracleCache.zeros(1, smax, H, D, dtype, total_steps=case["total_steps"])
    gen = cases.InputStream(case)
    i = 0
    for call in cases.schedule(case):
        if call["op"] == "replicate":
            b = call["rows"]
            cache.k = cache.k.repeat(b, 1, 1, 1)
            cache.v = cache.v.repeat(b, 1, 1, 1)
            st = cache.state
            st.rows = b
            st.global_end = st.global_end * b
            st.local_end = st.local_end * b
            continue
        starts, frames = call["starts"], call["frames"]
        q, k, v = gen.next(len(starts), frames * fs)
        out, rq, sl, dst = orc.self_attention_step(q, k, v, cache, table, (frames, h, w), starts,
                                                   case["sink_size"], case["adapt_sink_thr"])
        yield i, (q, k, v), out, cache, rq, sl, dst
        i += 1


class _AttnState:
    """The attributes of the reference attention module that the slot logic reads and writes."""

    def __init__(self, heads, head_dim, sink_size, adapt_sink_thr):
        self.num_heads, self.head_dim = heads, head_dim
        self.sink_size, self.adapt_sink_thr = sink_size, adapt_sink_thr
        self.evict_idx = None


def replay_cuda(case: dict, device="cuda"):
    """Same schedule through the CUDA path (streamdiffusionv2_b200.causal_attention).  Yields
    (step_index, out, kv_cache_dict, attn_state)."""
    from streamdiffusionv2_b200 import causal_attention as ca

    H, D = case["heads"], case["head_dim"]
    dtype = cases.DTYPES[case["dtype"]]
    h, w = case["grid_hw"]
    fs = h * w
    smax = case["cache_frames"] * fs
    freqs = orc.rope_table(D)
    mod = _AttnState(H, D, case["sink_size"], case["adapt_sink_thr"])
    kv = {"k": torch.zeros(1, smax, H, D, dtype=dtype, device=device),
          "v": torch.zeros(1, smax, H, D, dtype=dtype, device=device),
          "global_end_index": torch.tensor([0], dtype=torch.long, device=device),
          "local_end_index": torch.tensor([0], dtype=torch.long, device=device),
          "total_steps": case["total_steps"], "current_step": case["total_steps"]}
    gen = cases.InputStream(case)
    i = 0
    for call in cases.schedule(case):
        if call["op"] == "replicate":
            b = call["rows"]
            kv["k"] = kv["k"].repeat(b, 1, 1, 1)
            kv["v"] = kv["v"].repeat(b, 1, 1, 1)
            kv["global_end_index"] = kv["global_end_index"].repeat(b)
            kv["local_end_index"] = kv["local_end_index"].repeat(b)
            continue
        starts, frames = call["starts"], call["frames"]
        q, k, v = (t.to(device) for t in gen.next(len(starts), frames * fs))
        grid = torch.tensor([[frames, h, w]] * len(starts), dtype=torch.long)
        cs = torch.tensor(starts, dtype=torch.long, device=device)
        out = ca.cached_attention(mod, q, k, v, grid, freqs, kv, cs)
        ca.sync_evict_queue(mod)      # with the adaptive sink test the queue lives on the device
        yield i, out, kv, mod
        i += 1

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

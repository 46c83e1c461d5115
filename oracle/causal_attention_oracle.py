"""CPU oracle for the per-chunk causal self-attention path of the causal Wan DiT.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is
used by the tests, by the smoke check and by the benchmark's CPU-baseline leg as the
checker / the timed CPU arm, never as the product path.

It restates, in plain PyTorch-on-CPU and Python integers, what the reference computes
(paths are relative to the reference project root):

* rope table .................. models/wan/wan_base/modules/model.py:29-36 and
                                models/wan/causal_model.py:631-638
* per-chunk rope multiplier ... models/wan/causal_model.py:57-91
* rope application ............ models/wan/causal_model.py:94-108
* sink + ring slot state ...... models/wan/causal_model.py:268-342
* K/V slot write .............. models/wan/causal_model.py:321-322, 336-337
* attention over the cache .... models/wan/causal_model.py:111-157, 344-384
* cached text cross-attention . models/wan/wan_base/modules/model.py:161-194 and
                                models/wan/wan_base/modules/attention.py:80-135

Pinning: the reference ships no golden vectors for this path.  The oracle is pinned
against outputs of the reference itself (fixtures under tests/golden/, produced by
tests/golden/make_golden.py which imports the reference).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# rope table and multiplier
# --------------------------------------------------------------------------------------

def _rope_params(max_seq_len: int, dim: int, theta: float = 10000.0) -> torch.Tensor:
    """unit complex numbers exp(i * pos * theta^(-2j/dim)); model.py:29-36."""
    assert dim % 2 == 0
    inv = 1.0 / torch.pow(theta, torch.arange(0, dim, 2).to(torch.float64).div(dim))
    ang = torch.outer(torch.arange(max_seq_len), inv)
    return torch.polar(torch.ones_like(ang), ang)


def rope_table(head_dim: int = 128, max_seq_len: int = 1024) -> torch.Tensor:
    """complex128 [max_seq_len, head_dim/2]: temporal | height | width column groups.

    causal_model.py:631-638 (widths d-4*(d//6), 2*(d//6), 2*(d//6) real dims)."""
    d = head_dim
    return torch.cat([
        _rope_params(max_seq_len, d - 4 * (d // 6)),
        _rope_params(max_seq_len, 2 * (d // 6)),
        _rope_params(max_seq_len, 2 * (d // 6)),
    ], dim=1)


def rope_group_widths(half_dim: int):
    """number of complex columns in the (temporal, height, width) groups; causal_model.py:77-78."""
    c = half_dim
    return c - 2 * (c // 3), c // 3, c // 3


def rope_multiplier(table: torch.Tensor, f: int, h: int, w: int, start_frame: int) -> torch.Tensor:
    """complex128 [f*h*w, 1, D/2] for tokens ordered (frame, row, col); causal_model.py:57-73."""
    t, hh, ww = table.split(list(rope_group_widths(table.shape[1])), dim=1)
    tf = t[start_frame:start_frame + f].repeat_interleave(h * w, dim=0)
    hf = hh[:h].repeat_interleave(w, dim=0).repeat(f, 1)
    wf = ww[:w].repeat(h, 1).repeat(f, 1)
    return torch.cat([tf, hf, wf], dim=-1).unsqueeze(1)


def rope_apply(x: torch.Tensor, grid: Sequence[int], table: torch.Tensor,
               start_frames: Sequence[int]) -> torch.Tensor:
    """x [B, N, H, D] -> same shape/dtype; fp64 complex multiply then cast back.

    causal_model.py:94-108: pairs (2j, 2j+1) of the head dim form one complex number."""
    f, h, w = grid
    n_tok = f * h * w
    out = x.clone()
    for i, sf in enumerate(start_frames):
        mult = rope_multiplier(table, f, h, w, int(sf))
        xi = torch.view_as_complex(x[i, :n_tok].to(torch.float64).reshape(n_tok, x.shape[2], -1, 2))
        out[i, :n_tok] = torch.view_as_real(xi * mult).flatten(2).type_as(x)
    return out


def rope_apply_unfused_numpy(x: np.ndarray, grid: Sequence[int], table: np.ndarray,
                             start_frames: Sequence[int]) -> np.ndarray:
    """Independent restatement of rope_apply in float64 numpy with the multiply spelled out:
    re = rn(rn(a*c) - rn(b*d)), im = rn(rn(a*d) + rn(b*c)); result left in float64
    (the caller rounds to the storage type).  x is float64 [B, N, H, D]."""
    f, h, w = grid
    n_tok = f * h * w
    half = x.shape[-1] // 2
    ct, ch, cw = rope_group_widths(half)
    out = x.copy()
    tok = np.arange(n_tok)
    fi, yi, xi_ = tok // (h * w), (tok // w) % h, tok % w
    for i, sf in enumerate(start_frames):
        m = np.concatenate([table[int(sf) + fi, :ct], table[yi, ct:ct + ch], table[xi_, ct + ch:]], axis=1)
        c, d = m.real[:, None, :], m.imag[:, None, :]
        a, b = x[i, :n_tok, :, 0::2], x[i, :n_tok, :, 1::2]
        out[i, :n_tok, :, 0::2] = a * c - b * d
        out[i, :n_tok, :, 1::2] = a * d + b * c
    return out


# --------------------------------------------------------------------------------------
# sink + ring slot state machine
# --------------------------------------------------------------------------------------

@dataclass
class RingLayerState:
    """Mutable per-layer state: what the reference keeps in kv_cache[l] (index tensors and the
    two step counters, causal_stream_inference.py:98-105) and in self_attn.evict_idx
    (causal_model.py:179, 273-277)."""
    cache_tokens: int                       # Smax = kv_cache["k"].shape[1]
    rows: int                               # B = kv_cache["k"].shape[0]
    global_end: List[int] = field(default_factory=list)
    local_end: List[int] = field(default_factory=list)
    total_steps: int = 1
    current_step: int = 1
    evict_idx: Optional[List[List[int]]] = None

    def __post_init__(self):
        if not self.global_end:
            self.global_end = [0] * self.rows
        if not self.local_end:
            self.local_end = [0] * self.rows


def _ensure_queues(st: RingLayerState) -> None:
    """Queue creation and replication to all rows; causal_model.py:272-277."""
    if st.evict_idx is None:
        st.evict_idx = [[]]
    if len(st.evict_idx) < st.rows:
        st.evict_idx = [list(st.evict_idx[0]) for _ in range(st.rows)]


def ring_plan_row(st: RingLayerState, i: int, cs: int, n_new: int, frame_tokens: int, sink_size: int,
                  front: Optional[int] = None):
    """Slot logic for row i; causal_model.py:279-342.  Returns (dst_begin, seq_len) and mutates
    `st` exactly as the reference mutates the cache dict and the module's queue.  `front`, when
    not None, is the entry the adaptive sink test (causal_model.py:284-299) pushes at the front
    of the row's queue before the slot is chosen."""
    smax = st.cache_tokens
    sink_tokens = sink_size * frame_tokens
    q = st.evict_idx[i]
    ce = cs + n_new
    if front is not None:
        q.insert(0, int(front))
    if ce > smax or st.local_end[i] >= smax:                       # evict branch (:302-324)
        target_end = q[0]
        if st.rows == 1 and st.current_step > 1:
            st.current_step -= 1
        else:
            e = q.pop(0)
            if e > sink_tokens:
                q.append(e)
            st.current_step = st.total_steps
        begin, le = target_end - n_new, smax
        if begin < 0:
            raise RuntimeError("evicted slot starts before the cache (the reference raises a shape mismatch)")
    else:                                                          # append branch (:326-337)
        le = st.local_end[i] + ce - st.global_end[i]
        rolling_end = ce + n_new
        if rolling_end > sink_tokens and rolling_end <= smax and (not q or q[-1] != rolling_end):
            q.append(rolling_end)
        begin = le - n_new
        if begin < 0 or le > smax:
            raise RuntimeError("append slot outside the cache (the reference raises a shape mismatch)")
    st.global_end[i] = ce
    st.local_end[i] = le
    return begin, le


def ring_plan(st: RingLayerState, current_start: Sequence[int], n_new: int, frame_tokens: int,
              sink_size: int):
    """One call of the slot logic for all rows (no adaptive sink test).  Returns
    (dst_begin[B], seq_lens[B])."""
    _ensure_queues(st)
    dst_begin, seq_lens = [], []
    for i, cs in enumerate(current_start):
        b, le = ring_plan_row(st, i, int(cs), n_new, frame_tokens, sink_size)
        dst_begin.append(b)
        seq_lens.append(le)
    return dst_begin, seq_lens


def adaptive_sink_front(k_cache, v_cache, roped_k, v, row: int, sink_size: int, frame_tokens: int,
                        threshold: float) -> Optional[int]:
    """Adaptive sink refresh test for one row; causal_model.py:284-299.  Returns the queue
    entry to push at the front, or None."""
    sink_tokens = sink_size * frame_tokens
    if not (sink_tokens > 0 and threshold > -1 and v.shape[1] <= frame_tokens):
        return None
    i = row
    k_sink = k_cache[i:i + 1, :sink_tokens].reshape(sink_size, frame_tokens, -1).mean(1)
    k_new = roped_k[i:i + 1].reshape(1, frame_tokens, -1).mean(1)
    k_sim = torch.cosine_similarity(k_sink, k_new, dim=-1)
    v_sink = v_cache[i:i + 1, :sink_tokens].reshape(sink_size, frame_tokens, -1).mean(1)
    v_new = v[i:i + 1].reshape(1, frame_tokens, -1).mean(1)
    v_sim = torch.cosine_similarity(v_sink, v_new, dim=-1)
    avg = (k_sim + v_sim) / 2
    if avg.min() < threshold:
        return (int(torch.argmin(avg).item()) + 1) * frame_tokens
    return None


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------

def _upcast(t: torch.Tensor) -> torch.Tensor:
    return t.float() if t.dtype in (torch.float16, torch.bfloat16) else t


def attend_cache(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 seq_lens: Sequence[int]) -> torch.Tensor:
    """Non-causal softmax(q k^T / sqrt(D)) v of every query over cache[b, :seq_lens[b]];
    q [B,N,H,D], caches [B,S,H,D]; 16-bit inputs are up-cast to fp32 on CPU and the result is
    returned in q's dtype.  causal_model.py:111-157."""
    outs = []
    for b, sl in enumerate(seq_lens):
        qi = _upcast(q[b:b + 1].transpose(1, 2))
        ki = _upcast(k_cache[b:b + 1, :sl].transpose(1, 2))
        vi = _upcast(v_cache[b:b + 1, :sl].transpose(1, 2))
        o = F.scaled_dot_product_attention(qi, ki, vi, attn_mask=None, dropout_p=0.0, is_causal=False)
        outs.append(o.transpose(1, 2).to(q.dtype))
    return torch.cat(outs, dim=0).contiguous()


def attend_explicit(q, k_cache, v_cache, seq_lens, dtype=torch.float64) -> torch.Tensor:
    """Same contraction written out (scores, softmax, weighted sum) in `dtype`; used to
    cross-check attend_cache and as the high-precision yardstick for tolerances."""
    outs = []
    scale = 1.0 / math.sqrt(q.shape[-1])
    for b, sl in enumerate(seq_lens):
        qi = q[b].to(dtype).transpose(0, 1)               # [H,N,D]
        ki = k_cache[b, :sl].to(dtype).transpose(0, 1)    # [H,S,D]
        vi = v_cache[b, :sl].to(dtype).transpose(0, 1)
        p = torch.softmax(qi @ ki.transpose(1, 2) * scale, dim=-1)
        outs.append((p @ vi).transpose(0, 1))
    return torch.stack(outs, dim=0)


def cross_attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Text cross-attention core: every query attends all Lk context slots, no mask
    (context_lens is None on this path, causal_model.py:781); q [B,N,H,D], k/v [B,Lk,H,D]
    (batch may be a stride-0 expand).  model.py:189 -> attention.py:80-135."""
    qi, ki, vi = (_upcast(t.transpose(1, 2)) for t in (q, k, v))
    o = F.scaled_dot_product_attention(qi, ki, vi, attn_mask=None, dropout_p=0.0, is_causal=False)
    return o.transpose(1, 2).contiguous().to(q.dtype)


# --------------------------------------------------------------------------------------
# one full self-attention call on pre-projected q/k/v
# --------------------------------------------------------------------------------------

@dataclass
class OracleCache:
    """K/V tensors plus the slot state of one layer."""
    k: torch.Tensor
    v: torch.Tensor
    state: RingLayerState

    @classmethod
    def zeros(cls, rows, cache_tokens, heads, head_dim, dtype, total_steps=1):
        return cls(torch.zeros(rows, cache_tokens, heads, head_dim, dtype=dtype),
                   torch.zeros(rows, cache_tokens, heads, head_dim, dtype=dtype),
                   RingLayerState(cache_tokens, rows, total_steps=total_steps, current_step=total_steps))


def self_attention_step(q, k, v, cache: OracleCache, table, grid, current_start: Sequence[int],
                        sink_size: int, adapt_sink_thr: float = -1.0):
    """q,k,v [B,N,H,D] (already projected / normalised).  Ropes q and k, places k/v in their
    slots, updates the state and attends.  Returns (out [B,N,H,D], roped_q, seq_lens, dst_begin).
    causal_model.py:250-384 without the Linear layers."""
    f, h, w = grid
    fs = h * w
    n_new = q.shape[1]
    start_frames = [int(cs) // fs for cs in current_start]
    rq = rope_apply(q, grid, table, start_frames).type_as(v)
    rk = rope_apply(k, grid, table, start_frames).type_as(v)
    st = cache.state
    _ensure_queues(st)
    # the adaptive test of row i reads the cache after rows < i were written, as in the reference loop
    dst_all, sl_all = [], []
    for i, cs in enumerate(current_start):
        front = adaptive_sink_front(cache.k, cache.v, rk, v, i, sink_size, fs, adapt_sink_thr)
        dst, sl = ring_plan_row(st, i, int(cs), n_new, fs, sink_size, front)
        cache.k[i, dst:dst + n_new] = rk[i]
        cache.v[i, dst:dst + n_new] = v[i]
        dst_all.append(dst)
        sl_all.append(sl)
    out = attend_cache(rq, cache.k, cache.v, sl_all)
    return out, rq, sl_all, dst_all


# --------------------------------------------------------------------------------------
# storage rounding helpers (numpy has no bfloat16)
# --------------------------------------------------------------------------------------

def f64_to_bf16_bits_two_step(x: np.ndarray) -> np.ndarray:
    """float64 -> float32 (round-to-nearest-even) -> bfloat16 (round-to-nearest-even), returned as
    uint16 bit patterns.  This double rounding is what `.type_as(bf16)` does to a float64 tensor."""
    f32 = x.astype(np.float32)
    u = f32.view(np.uint32).astype(np.uint64)
    nan = np.isnan(f32)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    rounded[nan] = 0x7FC0
    return rounded

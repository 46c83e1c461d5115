"""Host-integer mirror of the sink + ring-buffer slot logic.

The reference decides, per cache row and per layer, where a chunk's K/V go and how long the valid
cache is, by reading the `global_end_index` / `local_end_index` device tensors back to the host
several times per row (models/wan/causal_model.py:279-342).  Here the same arithmetic runs on
Python integers kept beside the cache dict; the device tensors are still updated (by the append
kernel itself) so every other reader of the dict sees what the reference would have written.

State ownership is unchanged: the evict queue stays on the attention module (`evict_idx`,
causal_model.py:179), `current_step` / `total_steps` stay in the cache dict
(models/wan/causal_stream_inference.py:98-105).  The mirror lives under the private key
`_sdv2_host` of the cache dict and is re-read from the device tensors whenever they were replaced
or written through PyTorch ops that bump the tensors' version counter (`+=`, `fill_`, `copy_`,
index assignment: detected through the tensors' identity, data pointer and version).  Writers that
bypass the version counter are NOT detected: c10d collectives (`dist.broadcast` / `recv` into the
index tensors, as streamv2v/communication/kv_cache_manager.py:72-78 does), raw CUDA copies, other
libraries' kernels.  After such a write call `RingState.invalidate(kv_cache)`;
`causal_attention.watch_cache_manager` does that for the reference's `KVCacheManager`.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

_KEY = "_sdv2_host"


class RingState:
    """global_end / local_end of every row of one layer's cache, as Python ints."""

    __slots__ = ("global_end", "local_end", "_sig")

    def __init__(self, global_end: List[int], local_end: List[int], sig=None):
        self.global_end = global_end
        self.local_end = local_end
        self._sig = sig

    @staticmethod
    def _signature(kv_cache: dict):
        g, l = kv_cache["global_end_index"], kv_cache["local_end_index"]
        return (id(g), g.data_ptr(), g._version, id(l), l.data_ptr(), l._version, kv_cache["k"].shape[0])

    @classmethod
    def of(cls, kv_cache: dict) -> "RingState":
        """The mirror for this cache dict, re-synchronised (one device read) if stale."""
        sig = cls._signature(kv_cache)
        st: Optional[RingState] = kv_cache.get(_KEY)
        if st is None or st._sig != sig:
            rows = kv_cache["k"].shape[0]
            g = kv_cache["global_end_index"].reshape(-1).tolist()
            l = kv_cache["local_end_index"].reshape(-1).tolist()
            # the reference indexes element i of these tensors; shorter tensors would raise there
            if len(g) < rows or len(l) < rows:
                raise IndexError("global_end_index/local_end_index have fewer entries than cache rows")
            st = cls([int(x) for x in g], [int(x) for x in l], sig)
            kv_cache[_KEY] = st
        return st

    @staticmethod
    def invalidate(kv_cache: dict) -> None:
        """Forget the host mirror of this cache dict; the next call re-reads both index tensors from
        the device (one read-back).  Needed after anything wrote `global_end_index` /
        `local_end_index` without bumping their version counters (a collective, a raw copy)."""
        kv_cache.pop(_KEY, None)

    @staticmethod
    def _ensure_queues(kv_cache: dict, attn_module) -> None:
        """Queue creation and replication to all rows (causal_model.py:272-277)."""
        rows = kv_cache["k"].shape[0]
        if attn_module.evict_idx is None:
            attn_module.evict_idx = [[]]
        if len(attn_module.evict_idx) < rows:
            attn_module.evict_idx = [attn_module.evict_idx[0].copy() for _ in range(rows)]

    def plan_row(self, kv_cache: dict, attn_module, i: int, cs: int, n_new: int, frame_tokens: int,
                 front: Optional[int] = None) -> Tuple[int, int]:
        """Slot decision for row i (causal_model.py:279-342); mutates the queue on `attn_module`,
        the step counter in `kv_cache` and this mirror exactly as the reference loop body does.
        `front` is the entry the adaptive sink test pushes at the head of the queue, if any.
        Returns (dst_begin, seq_len)."""
        smax = kv_cache["k"].shape[1]
        rows = kv_cache["k"].shape[0]
        sink_tokens = attn_module.sink_size * frame_tokens
        ce = cs + n_new
        queue = attn_module.evict_idx[i]
        if front is not None:
            queue.insert(0, int(front))
        if ce > smax or self.local_end[i] >= smax:
            target_end = queue[0]
            if rows == 1 and kv_cache["current_step"] > 1:
                kv_cache["current_step"] -= 1
            else:
                head = queue.pop(0)
                if head > sink_tokens:
                    queue.append(head)
                kv_cache["current_step"] = kv_cache["total_steps"]
            begin, le = target_end - n_new, smax
        else:
            le = self.local_end[i] + ce - self.global_end[i]
            rolling_end = ce + n_new
            if rolling_end > sink_tokens and rolling_end <= smax and (not queue or queue[-1] != rolling_end):
                queue.append(rolling_end)
            begin = le - n_new
        if begin < 0 or begin + n_new > smax:
            raise RuntimeError(
                f"cache slot [{begin}, {begin + n_new}) of row {i} lies outside the {smax}-token cache")
        self.global_end[i] = ce
        self.local_end[i] = le
        return begin, le

    def plan(self, kv_cache: dict, attn_module, current_start: Sequence[int], n_new: int,
             frame_tokens: int) -> Tuple[List[int], List[int]]:
        """Slot decisions for all rows, in row order.  Returns (dst_begin, seq_lens)."""
        self._ensure_queues(kv_cache, attn_module)
        dst_begin, seq_lens = [], []
        for i, cs in enumerate(current_start):
            b, le = self.plan_row(kv_cache, attn_module, i, int(cs), n_new, frame_tokens)
            dst_begin.append(b)
            seq_lens.append(le)
        return dst_begin, seq_lens

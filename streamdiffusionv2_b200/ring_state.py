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

    # ------------------------------------------------------------------ queue kept on the device
    # With the adaptive sink test the evict queue depends on the data (causal_model.py:284-299), so a
    # host-side queue would need a read-back per row per layer.  In that mode the queue lives in a
    # device tensor [rows, 1 + QUEUE_CAP] (length, entries) that the plan kernel updates, kept on the
    # attention module as `_sdv2_queue`; the module's `evict_idx` lists are then a stale copy until
    # `sync_queue` refreshes them.  Everything else the slot logic decides does not depend on the
    # data and stays on the host (`plan_row_split`).
    QUEUE_CAP = 63

    @staticmethod
    def push_queue(kv_cache: dict, attn_module, device) -> torch.Tensor:
        """Device copy of the module's queues (created from the host lists when there is none, or
        when the number of cache rows changed); the device copy is authoritative afterwards."""
        rows = kv_cache["k"].shape[0]
        q = getattr(attn_module, "_sdv2_queue", None)
        if q is not None and attn_module.evict_idx is not getattr(attn_module, "_sdv2_queue_host", None):
            # somebody assigned a new `evict_idx` (the demo's cache resizer does, demo/vid2vid.py:146-148):
            # the host lists are what counts now
            attn_module._sdv2_queue = q = None
        if q is not None and (q.shape[0] != rows or q.device != torch.device(device)):
            RingState.pull_queue(attn_module)
            q = None
        if q is None:
            RingState._ensure_queues(kv_cache, attn_module)
            host = torch.zeros(rows, 1 + RingState.QUEUE_CAP, dtype=torch.int64)
            for i, lst in enumerate(attn_module.evict_idx[:rows]):
                if len(lst) > RingState.QUEUE_CAP:
                    raise RuntimeError("evict queue longer than the device record")
                host[i, 0] = len(lst)
                if lst:
                    host[i, 1:1 + len(lst)] = torch.tensor([int(x) for x in lst], dtype=torch.int64)
            q = host.to(device)
            attn_module._sdv2_queue = q
            attn_module._sdv2_queue_host = attn_module.evict_idx
        return q

    @staticmethod
    def sync_queue(attn_module) -> None:
        """Refresh `attn_module.evict_idx` from the device queue (one read-back); the device copy
        stays authoritative.  No-op when the queue lives on the host."""
        q = getattr(attn_module, "_sdv2_queue", None)
        if q is None:
            return
        host = q.cpu().tolist()
        attn_module.evict_idx = [[int(x) for x in row[1:1 + int(row[0])]] for row in host]
        attn_module._sdv2_queue_host = attn_module.evict_idx

    @staticmethod
    def pull_queue(attn_module) -> None:
        """Bring the queue back to the host lists and drop the device copy (the host-integer slot
        logic, block re-ownership and anything else that reads `evict_idx` call this first)."""
        if getattr(attn_module, "_sdv2_queue", None) is not None:
            RingState.sync_queue(attn_module)
            attn_module._sdv2_queue = None

    def plan_row_split(self, kv_cache: dict, attn_module, i: int, cs: int, n_new: int, frame_tokens: int):
        """The data-independent part of `plan_row` for row i: everything but the queue.  Updates the
        mirror and the step counter exactly as `plan_row` does and returns what the device-side queue
        logic needs: (evict, pop, push_value, append_begin, seq_len) where `evict` selects the branch
        (causal_model.py:302), `pop` says whether the head leaves the queue (:310-316), `push_value`
        is the rolling end the append branch registers unless it is already the tail (-1: none,
        :326-332) and `append_begin` the slot of the append branch."""
        smax = kv_cache["k"].shape[1]
        rows = kv_cache["k"].shape[0]
        sink_tokens = attn_module.sink_size * frame_tokens
        ce = cs + n_new
        if ce > smax or self.local_end[i] >= smax:
            evict, push_value, begin, le = True, -1, -1, smax
            if rows == 1 and kv_cache["current_step"] > 1:
                kv_cache["current_step"] -= 1
                pop = False
            else:
                kv_cache["current_step"] = kv_cache["total_steps"]
                pop = True
        else:
            evict, pop = False, False
            le = self.local_end[i] + ce - self.global_end[i]
            rolling_end = ce + n_new
            push_value = rolling_end if sink_tokens < rolling_end <= smax else -1
            begin = le - n_new
            if begin < 0 or begin + n_new > smax:
                raise RuntimeError(
                    f"cache slot [{begin}, {begin + n_new}) of row {i} lies outside the {smax}-token cache")
        self.global_end[i] = ce
        self.local_end[i] = le
        return evict, pop, push_value, begin, le

    @staticmethod
    def queue_step(queue: List[int], front: Optional[int], evict: bool, pop: bool, push_value: int,
                   append_begin: int, n_new: int, sink_tokens: int) -> int:
        """The queue half of the slot logic, as the device plan kernel runs it (this host version is
        the specification the kernel follows and what the CPU tests exercise).  Returns the slot."""
        if front is not None:
            queue.insert(0, int(front))
        if evict:
            target_end = queue[0]
            if pop:
                head = queue.pop(0)
                if head > sink_tokens:
                    queue.append(head)
            return target_end - n_new
        if push_value >= 0 and (not queue or queue[-1] != push_value):
            queue.append(push_value)
        return append_begin

    def plan(self, kv_cache: dict, attn_module, current_start: Sequence[int], n_new: int,
             frame_tokens: int) -> Tuple[List[int], List[int]]:
        """Slot decisions for all rows, in row order.  Returns (dst_begin, seq_lens)."""
        self.pull_queue(attn_module)
        self._ensure_queues(kv_cache, attn_module)
        dst_begin, seq_lens = [], []
        for i, cs in enumerate(current_start):
            b, le = self.plan_row(kv_cache, attn_module, i, int(cs), n_new, frame_tokens)
            dst_begin.append(b)
            seq_lens.append(le)
        return dst_begin, seq_lens

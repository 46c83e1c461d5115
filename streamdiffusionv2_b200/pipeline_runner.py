"""Per-rank driver of the pipeline-parallel stream: one rank per GPU, contiguous block ranges,
activations handed from stage to stage by `StageLink`.

Mirrors the data flow of the reference's rank loops (streamv2v/inference_pipe.py:511-800):

* stage 0 shifts the new chunk into the stage batch, runs its blocks and sends activations plus
  the stage-batch latents and row starts/ends downstream; once the ring is full it first adopts
  the latents and row indices that came back from the last stage `world_size` chunks earlier;
* middle stages receive, run their blocks on the received activations, forward;
* the last stage runs the remaining blocks, the head, the x0 conversion and the re-noising, and
  returns the new stage-batch latents to stage 0 (latents only; the reference also ships the
  activations back, which nobody reads).

`world_size` chunks are in flight around the ring, one per stage.
"""
from __future__ import annotations

from collections import deque
from typing import List, Optional, Sequence

import torch

from .ring_state import RingState
from .stage_transport import StageLink, StagePacket, contiguous_block_ranges, plan_from_measurements
from .stream_pipeline import StreamPipeline, assign_ints


class StreamRestart(Exception):
    """Raised by `step()` on a stage that received the restart packet; carries the new prompt."""

    def __init__(self, prompt: str):
        super().__init__("stream restart")
        self.prompt = prompt


class PipelineStageRunner:
    def __init__(self, pipe: StreamPipeline, link: StageLink, rank: int, world_size: int,
                 block_ranges: Optional[Sequence[Sequence[int]]] = None, prefetch: bool = False,
                 half_ranges: Optional[Sequence[Sequence[int]]] = None):
        # prefetch: post the next receive one chunk ahead.  Off by default: a posted NCCL receive is a
        # kernel that spins on a few SMs until its data arrives, and the attention CTAs (which need a
        # whole SM's shared memory) cannot run on those SMs meanwhile; a 20 MB hop takes ~30 us anyway.
        self.prefetch = prefetch
        self.pipe, self.link, self.rank, self.world = pipe, link, rank, world_size
        # Stage ranges are kept in half-block units (half 2i = self-attention part of block i, half
        # 2i + 1 = the rest of it): the reference splits at whole blocks (inference_pipe.py:59-74), which
        # is what `block_ranges` gives; `half_ranges` lets two stages meet inside a block.
        if half_ranges is None:
            ranges = block_ranges or contiguous_block_ranges(pipe.num_transformer_blocks, world_size)
            half_ranges = [[2 * int(a), 2 * int(b)] for a, b in ranges]
        self._set_ranges(half_ranges)
        self._measure_left = 0    # steps still to run with every half block timed (measure_costs)
        self._measured: List[list] = []
        self.role = "input" if rank == 0 else ("output" if rank == world_size - 1 else "middle")
        self.items = 0            # chunks processed (stage 0: sent)
        self.received = 0         # stage 0: packets taken from the closing edge
        self._returned = deque()  # stage 0: packets taken in by quiesce(), not yet adopted
        self.stage_events = None  # set to [] to record (start, end) CUDA events around each stage compute
        self._quiet = True        # nothing in flight on the links: a step may synchronise the device (graph recording)

    def _set_ranges(self, half_ranges: Sequence[Sequence[int]]) -> None:
        total = 2 * self.pipe.num_transformer_blocks
        hr = [[int(a), int(b)] for a, b in half_ranges]
        if (len(hr) != self.world or hr[0][0] != 0 or hr[-1][1] != total
                or any(a[1] != b[0] for a, b in zip(hr, hr[1:])) or any(b <= a for a, b in hr)):
            raise ValueError("stage ranges must be contiguous, non-empty and cover every block")
        self.half_ranges = hr
        self.half_range = list(hr[self.rank])
        # blocks whose self-attention (and therefore K/V cache) lives on each stage
        self.block_ranges = [[(a + 1) // 2, (b + 1) // 2] for a, b in hr]
        self.block_range = list(self.block_ranges[self.rank])
        self._whole_blocks = all(a % 2 == 0 and b % 2 == 0 for a, b in hr)

    @property
    def owned_blocks(self) -> range:
        return range(self.block_range[0], self.block_range[1])

    def _range_args(self) -> dict:
        """How this stage's range is handed to the pipeline: as whole blocks where it can be."""
        if self._whole_blocks:
            return {"block_num": [self.half_range[0] // 2, self.half_range[1] // 2]}
        return {"block_num": self.block_range, "half_blocks": self.half_range}

    # ------------------------------------------------------------------ measured stage costs
    def measure_costs(self, steps: int = 3) -> None:
        """Have the next `steps` chunk steps of this rank run launch by launch (no graph replay) with
        every half block and the whole stage timed; `plan_ranges` then uses the medians.  Call on every
        rank before the same chunk."""
        self._measure_left, self._measured = int(steps), []

    def _measured_step(self, run):
        """Run one stage computation, timed per half block when a measurement is in progress."""
        if self._measure_left <= 0:
            return run()
        from .wan_model import _stamp
        model, pipe = self.pipe.generator.model, self.pipe
        graphs, pipe.step_graphs = pipe.step_graphs, None
        model.half_stamps = []
        t0 = _stamp(pipe.hidden_states)
        try:
            out = run()
        finally:
            t1 = _stamp(pipe.hidden_states)
            self._measured.append((model.half_stamps, t0, t1))
            model.half_stamps = None
            pipe.step_graphs = graphs
            self._measure_left -= 1
        return out

    def plan_ranges(self, granularity: str = "half") -> List[List[int]]:
        """New stage ranges (half-block units) from the measured steps.  Every rank contributes the
        median launch-by-launch time of each half block it ran and of its stage's extra work
        (everything that is not a block: embedding, row shift, head, x0 conversion, re-noising); one
        all-gather on the default process group; then the same exact partition on every rank
        (`stage_transport.plan_from_measurements`, which uses the times as proportions only).
        granularity "block" keeps the boundaries at whole blocks.  Collective: call on every rank."""
        import statistics
        import torch.distributed as dist
        if not self._measured or self._measure_left > 0:
            raise RuntimeError("measure_costs() and the measured steps come first")
        n_half = 2 * self.pipe.num_transformer_blocks
        dev = self.pipe.device
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)

        def span(a, b):
            return a.elapsed_time(b) if hasattr(a, "elapsed_time") else (b - a) * 1e3

        per_half: dict = {}
        extras = []
        for stamps, t0, t1 in self._measured:
            inside = 0.0
            for h, a, b in stamps:
                d = span(a, b)
                per_half.setdefault(h, []).append(d)
                inside += d
            extras.append(span(t0, t1) - inside)
        mine = torch.zeros(n_half + 1, dtype=torch.float64)
        for h, v in per_half.items():
            mine[h] = statistics.median(v)
        mine[n_half] = max(statistics.median(extras), 0.0)
        mine = mine.to(dev)
        every = [torch.zeros_like(mine) for _ in range(self.world)]
        dist.all_gather(every, mine)
        every = [t.cpu() for t in every]
        costs = torch.stack([t[:n_half] for t in every]).max(dim=0).values.tolist()   # one rank measured each half
        overheads = [float(t[n_half]) for t in every]
        if min(costs) <= 0.0:
            raise RuntimeError("a half block was not measured on any rank")
        ranges, details = plan_from_measurements(costs, overheads, self.half_ranges, granularity)
        self.last_costs = {"per_half_ms": costs, "stage_extra_ms": overheads, **details}
        return ranges

    # ------------------------------------------------------------------ one chunk on this rank
    def step(self, chunk_idx: int = 0, noise: Optional[torch.Tensor] = None, current_start: Optional[int] = None,
             current_end: Optional[int] = None, current_step: Optional[int] = None,
             last: bool = False) -> Optional[torch.Tensor]:
        """Process one chunk on this rank.  Stage 0 needs `noise`, `current_start`, `current_end`
        (and optionally the adaptive `current_step`); the other stages take everything from the
        packet they receive.  The last stage returns the denoised stage batch, the others None.
        `last=True` marks the final chunk before `quiesce()`: no receive is posted ahead."""
        pipe, link = self.pipe, self.link
        if self.role == "input":
            if self.items >= self.world:
                if self._returned:
                    back = self._returned.popleft()     # taken in early by quiesce()
                else:
                    back = link.recv()                  # what the last stage made of chunk items-world
                    self.received += 1
                    if self.prefetch and not last:
                        link.post_recv()
                pipe.hidden_states.copy_(back.latents)
                assign_ints(pipe.kv_cache_starts, back.starts)
                assign_ints(pipe.kv_cache_ends, back.ends)
                pipe._starts_host = list(back.starts)
                pipe._ends_host = list(back.ends)
            elif self.prefetch and self.items == self.world - 1 and not last:
                link.post_recv()
            ev = self._mark()
            act, _ = self._measured_step(lambda: pipe.inference(
                noise=noise, current_start=current_start, current_end=current_end, current_step=current_step,
                block_mode="input", allow_record=self._quiet, **self._range_args()))
            self._quiet = False
            self._mark(ev)
            link.send(chunk_idx, act, pipe.hidden_states, pipe.generator.model.last_patched_x_shape,
                      pipe._starts_host, pipe._ends_host, -1 if current_step is None else int(current_step))
            self.items += 1
            return None

        pkt: StagePacket = link.recv()
        if pkt.chunk_idx == -1:
            # restart (inference_pipe.py:473-493): pass it on, forget the stream's position; the caller
            # prepares the pipeline again with the new prompt.  Nothing returns to stage 0 for it.
            if self.role == "middle":
                link.send_restart(pkt.prompt or "")
            link.drain()
            self.items = 0
            self._quiet = True
            raise StreamRestart(pkt.prompt or "")
        if self.prefetch and not last:
            link.post_recv()
        step = None if pkt.current_step < 0 else pkt.current_step
        ev = self._mark()
        out, pshape = self._measured_step(lambda: pipe.inference(
            noise=pkt.latents, current_start=pkt.starts, current_end=pkt.ends, current_step=step, block_mode=self.role,
            patched_x_shape=pkt.patched_x_shape, block_x=pkt.activations, starts_host=pkt.starts,
            allow_record=self._quiet, **self._range_args()))
        self._quiet = False
        self._mark(ev)
        if self.role == "middle":
            link.send(pkt.chunk_idx, out, pkt.latents, pkt.patched_x_shape, pkt.starts, pkt.ends, pkt.current_step)
            self.items += 1
            return None
        link.send(pkt.chunk_idx, None, out, pkt.patched_x_shape, pkt.starts, pkt.ends, pkt.current_step)
        self.items += 1
        return out

    def _mark(self, start=None):
        if self.stage_events is None:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        if start is not None:
            self.stage_events.append((start, e))
        return e

    def quiesce(self) -> None:
        """Empty the ring: stage 0 takes in every packet still travelling back to it (they are kept
        and adopted in order by the following steps), every stage waits for its sends.  Afterwards
        no transfer is posted or in flight, so a device-wide synchronise or a barrier cannot wait
        on a peer.  The step before it must have been run with `last=True` on every rank."""
        if self.role == "input":
            while self.received < self.items:          # one packet comes back per chunk sent
                pkt = self.link.recv()
                self.received += 1
                self._returned.append(StagePacket(pkt.chunk_idx, pkt.current_step, pkt.patched_x_shape, pkt.starts,
                                                  pkt.ends, None, pkt.latents.clone()))
        self.link.drain()
        self._quiet = True

    def restart(self, prompt: str) -> None:
        """Stage 0: start the stream over with a new prompt (inference_pipe.py:448-472).  Takes in and
        discards what is still travelling back, sends the restart packet down the ring and resets the
        chunk counters; every other stage's next `step()` raises `StreamRestart(prompt)`."""
        if self.role != "input":
            raise RuntimeError("only stage 0 starts a restart")
        while self.received < self.items:
            self.link.recv()
            self.received += 1
        self._returned.clear()
        self.link.send_restart(prompt)
        self.link.drain()
        self.items = self.received = 0
        self._quiet = True

    # ------------------------------------------------------------------ moving blocks between stages
    _QUEUE_SLOTS = 64   # evict-queue entries shipped per row (a queue holds at most one entry per cache frame)

    def rebalance(self, new_ranges: Sequence[Sequence[int]], halves: bool = False) -> None:
        """Switch to new contiguous stage ranges (whole blocks, or half-block units with `halves`)
        and move the K/V state of every block whose self-attention changes owner (streamv2v/inference_pipe.py:802-843, communication/kv_cache_manager.py:48-144).
        Call on every rank with the same ranges, directly after `quiesce()`: with the ring empty all
        stages have processed the same chunks, so the state moves as it is - K, V, both index
        tensors, the step counters and the block's evict queue (which the reference leaves behind).
        The old owner keeps an empty placeholder; recorded step graphs are dropped."""
        import torch.distributed as dist
        if not self._quiet:
            raise RuntimeError("rebalance() needs an empty ring: call quiesce() first")
        new_half = [[int(a) * (1 if halves else 2), int(b) * (1 if halves else 2)] for a, b in new_ranges]
        total = self.pipe.num_transformer_blocks
        if (len(new_half) != self.world or new_half[0][0] != 0 or new_half[-1][1] != 2 * total
                or any(a[1] != b[0] for a, b in zip(new_half, new_half[1:]))
                or any(b <= a for a, b in new_half)):
            raise ValueError("block ranges must be contiguous, non-empty and cover every block")
        new_ranges = [[(a + 1) // 2, (b + 1) // 2] for a, b in new_half]   # owners of the self-attention halves

        def owners(ranges):
            out = [0] * total
            for r, (a, b) in enumerate(ranges):
                out[a:b] = [r] * (b - a)
            return out

        old_owner, new_owner = owners(self.block_ranges), owners(new_ranges)
        pipe, dev = self.pipe, self.pipe.device
        for i in range(total):
            src, dst = old_owner[i], new_owner[i]
            if src == dst or self.rank not in (src, dst):
                continue
            kv = pipe.kv_cache1[i]
            module = pipe.generator.model.blocks[i].self_attn
            if self.rank == src:
                rows = kv["k"].shape[0]
                meta = torch.zeros(3 + rows * (1 + self._QUEUE_SLOTS), dtype=torch.int64)
                meta[0], meta[1], meta[2] = rows, int(kv["current_step"]), int(kv["total_steps"])
                queues = module.evict_idx if module.evict_idx is not None else []
                for r in range(rows):
                    q = [int(x) for x in (queues[r] if r < len(queues) else [])]
                    if len(q) > self._QUEUE_SLOTS:
                        raise RuntimeError("evict queue longer than the transfer record")
                    base = 3 + r * (1 + self._QUEUE_SLOTS)
                    meta[base] = len(q) if r < len(queues) else -1
                    meta[base + 1:base + 1 + len(q)] = torch.tensor(q, dtype=torch.int64)
                for t in (meta.to(dev), kv["global_end_index"], kv["local_end_index"], kv["k"].to(dev),
                          kv["v"].to(dev)):
                    dist.send(t.contiguous(), dst=dst)
                kv["k"], kv["v"] = kv["k"][:, :0], kv["v"][:, :0]         # placeholder, as for never-owned blocks
                RingState.invalidate(kv)
            else:
                rows = pipe.hidden_states.shape[0]
                meta = torch.zeros(3 + rows * (1 + self._QUEUE_SLOTS), dtype=torch.int64, device=dev)
                dist.recv(meta, src=src)
                m = meta.tolist()
                if m[0] != rows:
                    raise RuntimeError("the sender's cache has another number of rows")
                dtype = pipe.hidden_states.dtype
                shape = (rows, pipe.kv_cache_length, pipe.num_heads, pipe.head_dim)
                ge = torch.empty(rows, dtype=torch.int64, device=dev)
                le = torch.empty(rows, dtype=torch.int64, device=dev)
                k = torch.empty(shape, dtype=dtype, device=dev)
                v = torch.empty(shape, dtype=dtype, device=dev)
                for t in (ge, le, k, v):
                    dist.recv(t, src=src)
                kv.update(k=k, v=v, global_end_index=ge, local_end_index=le, current_step=m[1], total_steps=m[2])
                RingState.invalidate(kv)              # the host mirror is re-read from the received tensors
                queues = []
                for r in range(rows):
                    base = 3 + r * (1 + self._QUEUE_SLOTS)
                    if m[base] >= 0:
                        queues.append([int(x) for x in m[base + 1:base + 1 + m[base]]])
                module.evict_idx = queues if queues else None
        self._set_ranges(new_half)
        if pipe.step_graphs is not None:
            pipe.step_graphs.forget()

    def park(self) -> None:
        """Pause with the ring still full, for a barrier or a device-wide synchronise between two
        runs of steps.  Precondition: the ranks are staggered as in steady state, rank r having
        processed exactly r chunks fewer than rank 0, so that one packet is travelling on every
        edge.  Each rank takes that packet into its receive buffer (the next `step()` consumes it)
        and waits for its own send; afterwards nothing is in flight and nothing was dropped.  A
        rank whose upstream peer did not send raises on the host after the link's timeout instead
        of leaving a receive waiting on the GPU."""
        up = self.link.up
        if self.role == "input":
            due = self.items - (self.world - 1) - self.received - len(up.posted)
        else:
            due = 1 - len(up.posted)
        if due > 1:
            raise RuntimeError("park(): more than one packet outstanding; ranks are not staggered by one chunk")
        if due == 1:
            self.link.post_recv(confirm_sent=True)
        self.link.drain()
        self._quiet = True

    def finish(self) -> None:
        """End of stream: same as quiesce()."""
        self.quiesce()

"""Ring hand-off between pipeline-parallel stages of the DiT.

Replaces the reference's per-hop protocol (streamv2v/communication/distributed_communicator.py
:158-264: two shape headers, two payloads and two index vectors per hop, each header read back
to the host before its payload can be received) with

* one fixed-shape device payload per hop: stage activations [rows, tokens, dim] and the
  stage-batch latents [rows, frames, C, H, W] packed in one bf16 buffer, moved by a single
  NCCL point-to-point operation on the edge's own communicator (stages talk over NVLink);
* one small host-side metadata message (chunk index, denoise step of row 0, patched shape,
  per-row chunk starts/ends) on a CPU (gloo) group, so the receiver knows every integer it
  needs without reading device memory back.

Every ring edge r -> r+1 has its own two-rank process group, hence its own communicator and
stream, so a stage's send and its next receive do not serialise.  Receive buffers are
double-buffered.  A receive may be posted one chunk ahead (`post_recv`), but the runner does not
do so by default: a posted NCCL receive is a kernel that occupies a few SMs until its data
arrives, and measured on B200 that slowed each stage's attention by ~20 % (its CTAs need a whole
SM), while the 20 MB hop itself takes ~30 us.  The closing edge (last stage -> stage 0) carries
latents only.

`chunk_idx == -1` is the restart sentinel of the reference drivers (streamv2v/inference_pipe.py:
448-493): `send_restart(prompt)` sends a packet whose payload is ignored, followed by the new prompt
text on the host group; `recv()` returns it with `prompt` set.

Works on CPU tensors with the gloo backend too, which is how the host logic is tested.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass
class StagePacket:
    chunk_idx: int
    current_step: int
    patched_x_shape: List[int]
    starts: List[int]
    ends: List[int]
    activations: Optional[torch.Tensor]   # [rows, tokens, dim]; None on the closing edge
    latents: torch.Tensor                 # [rows, frames, C, H, W]
    prompt: Optional[str] = None          # set on a restart packet (chunk_idx == -1)


def contiguous_block_ranges(total_blocks: int, world_size: int) -> List[List[int]]:
    """Contiguous [start, end) block ranges per stage, as the reference driver splits them
    (streamv2v/inference_pipe.py:59-74): halves for two stages, otherwise the remainder goes to
    the first stages."""
    if world_size == 2:
        mid = total_blocks // 2
        return [[0, mid], [mid, total_blocks]]
    base, rem = divmod(total_blocks, world_size)
    out, start = [], 0
    for r in range(world_size):
        end = start + base + (1 if r < rem else 0)
        if r == world_size - 1:
            end = total_blocks
        out.append([start, end])
        start = end
    return out


def balanced_block_ranges(total_blocks: int, world_size: int) -> List[List[int]]:
    """Contiguous ranges with the remainder on the stages in the middle: the first stage also embeds
    the latents and shifts the stream batch, the last one runs the head, the x0 conversion and the
    re-noising, so giving them the extra blocks (as the default split does) makes them the slowest.
    Same block counts as `contiguous_block_ranges` up to which stages hold the remainder; this is the
    split the reference's run-time rebalancing (streamv2v/inference_pipe.py:802-843) moves towards."""
    base, rem = divmod(total_blocks, world_size)
    sizes = [base] * world_size
    # innermost stages first; of two equally far from the middle, the later one (the first stage's extra
    # work was measured larger than the last stage's)
    order = sorted(range(world_size), key=lambda r: (abs(r - (world_size - 1) / 2), -r))
    for r in order[:rem]:
        sizes[r] += 1
    out, start = [], 0
    for n in sizes:
        out.append([start, start + n])
        start += n
    return out


def partition_by_cost(costs: Sequence[float], overheads: Sequence[float], boundary_step: int = 1,
                      scales: Optional[Sequence[float]] = None) -> List[List[int]]:
    """Contiguous, non-empty ranges of `costs` (one per stage, in order) that minimise the slowest
    stage's time max_r(overheads[r] + scales[r] * sum of the costs in range r) - `scales` (default 1)
    lets stages differ in speed, which GPUs under a power cap do by several per cent: the run-time counterpart of the
    reference's compute_balanced_split (streamv2v/communication/utils.py:141-229), which moves
    whole blocks proportionally to the measured imbalance; this one takes the measured cost of
    every unit and the fixed extra time of every stage (patch embedding and row shift on the
    first, head and re-noising on the last) and solves the partition exactly.  `boundary_step` = 2
    with costs per half block restricts the boundaries to whole blocks.  Ties keep earlier stages
    shorter.  Returns [[start, end), ...] in units of `costs`."""
    n, w = len(costs), len(overheads)
    if w < 1 or n < w * boundary_step:
        raise ValueError("fewer units than stages")
    scales = [1.0] * w if scales is None else [float(x) for x in scales]
    if len(scales) != w or min(scales) <= 0:
        raise ValueError("one positive scale per stage")
    prefix = [0.0]
    for c in costs:
        prefix.append(prefix[-1] + float(c))
    cuts = list(range(0, n + 1, boundary_step))
    if cuts[-1] != n:
        raise ValueError("the number of units is not a multiple of boundary_step")
    inf = float("inf")
    # best[r][j]: smallest possible slowest-stage time for stages 0..r covering units [0, cuts[j])
    best = [[inf] * len(cuts) for _ in range(w)]
    back = [[-1] * len(cuts) for _ in range(w)]
    for j in range(1, len(cuts)):
        best[0][j] = overheads[0] + scales[0] * prefix[cuts[j]]
    for r in range(1, w):
        for j in range(r + 1, len(cuts)):
            for i in range(r, j):
                t = max(best[r - 1][i], overheads[r] + scales[r] * (prefix[cuts[j]] - prefix[cuts[i]]))
                if t < best[r][j]:
                    best[r][j], back[r][j] = t, i
    out, j = [], len(cuts) - 1
    for r in range(w - 1, -1, -1):
        i = back[r][j] if r > 0 else 0
        out.append([cuts[i], cuts[j]])
        j = i
    return out[::-1]


def plan_from_measurements(per_half_ms: Sequence[float], stage_extra_ms: Sequence[float],
                           half_ranges: Sequence[Sequence[int]], granularity: str = "half"):
    """Stage ranges (half-block units) from one launch-by-launch measurement per half block and per
    stage.  The measurements are used as proportions only: every block is the same layer, so a block
    is one unit of work, split between its two halves in the ratio measured on average, and a stage's
    extra work (embedding, head, re-noising ...) is expressed in units of the blocks measured on that
    same stage, which cancels how fast or slow that stage happened to run while it was being measured.
    All stages are then taken to be equally fast per unit: the GPUs of a node are the same part under
    the same power cap, and a stage that looks faster in normal operation merely idles part of each
    step and clocks higher while it works (measured on B200: a stage of 7 blocks ran at 1.66 ms per
    block beside stages of 8 at 1.81, and the other way round after the blocks were moved).
    Returns (ranges, details)."""
    n_half = len(per_half_ms)
    block_ms = [per_half_ms[2 * i] + per_half_ms[2 * i + 1] for i in range(n_half // 2)]
    attn_share = sum(per_half_ms[2 * i] / block_ms[i] for i in range(n_half // 2)) / (n_half // 2)
    units = [attn_share, 1.0 - attn_share] * (n_half // 2)
    extra_units = []
    for r, (a, b) in enumerate(half_ranges):
        first, last = a // 2, max((b + 1) // 2, a // 2 + 1)          # blocks this stage ran at least half of
        mean_block = sum(block_ms[first:last]) / (last - first)
        extra_units.append(max(float(stage_extra_ms[r]), 0.0) / mean_block)
    ranges = partition_by_cost(units, extra_units, boundary_step=2 if granularity == "block" else 1)
    load = [extra_units[r] + sum(units[a:b]) for r, (a, b) in enumerate(ranges)]
    return ranges, {"attention_share_of_block": attn_share, "stage_extra_blocks": extra_units,
                    "planned_stage_load_blocks": load}


class _Edge:
    """One direction of one ring edge as seen from this rank."""

    def __init__(self, group, meta_group, peer: int, numel: int, meta_len: int, dtype, device, depth: int = 2):
        self.group, self.meta_group, self.peer = group, meta_group, peer
        self.bufs = [torch.empty(numel, dtype=dtype, device=device) for _ in range(depth)]
        self.meta = [torch.zeros(meta_len, dtype=torch.int64) for _ in range(depth)]
        self.works: List[Optional[object]] = [None] * depth
        self.meta_works: List[Optional[object]] = [None] * depth
        self.next = 0
        self.posted: Deque[int] = deque()


class StageLink:
    """Point-to-point links of one stage: `up` (from the previous stage) and `down` (to the next)."""

    META_FIXED = 7  # chunk_idx, current_step, patched_x_shape[5]

    def __init__(self, rank: int, world_size: int, device: torch.device, act_shape: Sequence[int],
                 latent_shape: Sequence[int], dtype=torch.bfloat16, timeout_s: float = 120.0):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        if world_size < 2:
            raise ValueError("a pipeline needs at least two stages")
        self.rank, self.world, self.device = rank, world_size, torch.device(device)
        self.act_shape, self.latent_shape = tuple(act_shape), tuple(latent_shape)
        self.rows = self.latent_shape[0]
        self.act_numel = int(torch.Size(self.act_shape).numel())
        self.lat_numel = int(torch.Size(self.latent_shape).numel())
        self.meta_len = self.META_FIXED + 2 * self.rows
        import datetime
        to = datetime.timedelta(seconds=timeout_s)
        # every rank creates every group, in the same order
        self._edge_groups = [dist.new_group([i, (i + 1) % world_size], timeout=to) for i in range(world_size)]
        self._meta_groups = [dist.new_group([i, (i + 1) % world_size], backend="gloo", timeout=to)
                             for i in range(world_size)]
        prev_rank, next_rank = (rank - 1) % world_size, (rank + 1) % world_size
        up_edge, down_edge = prev_rank, rank          # edge i connects i -> i+1
        closing_up = rank == 0                         # stage 0 receives the closing edge
        closing_down = rank == world_size - 1
        self.up = _Edge(self._edge_groups[up_edge], self._meta_groups[up_edge], prev_rank,
                        self.lat_numel + (0 if closing_up else self.act_numel), self.meta_len, dtype, self.device)
        self.down = _Edge(self._edge_groups[down_edge], self._meta_groups[down_edge], next_rank,
                          self.lat_numel + (0 if closing_down else self.act_numel), self.meta_len, dtype,
                          self.device)
        self._up_has_act, self._down_has_act = not closing_up, not closing_down
        self._side = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self._warm_edges(dtype)

    def _warm_edges(self, dtype) -> None:
        """Create every edge's communicator now, one edge at a time, with nothing else in flight.
        A communicator that is created lazily by its first transfer blocks the host (and may
        synchronise the device) while another edge's receive is already waiting on the GPU for a
        send this host has not issued yet; two stages doing that to each other never finish."""
        for i in range(self.world):
            src, dst = i, (i + 1) % self.world
            if self.rank in (src, dst):
                t = torch.zeros(8, dtype=dtype, device=self.device)
                m = torch.zeros(2, dtype=torch.int64)
                if self.rank == src:
                    dist.send(m, dst=dst, group=self._meta_groups[i])
                    dist.send(t, dst=dst, group=self._edge_groups[i])
                else:
                    dist.recv(m, src=src, group=self._meta_groups[i])
                    dist.recv(t, src=src, group=self._edge_groups[i])
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
                dist.barrier(device_ids=[self.device.index])
            else:
                dist.barrier()

    # ------------------------------------------------------------------ receive side
    def post_recv(self, confirm_sent: bool = False) -> None:
        """Post the receive of the next packet from the previous stage.  Call it right after
        `recv()` returned and before enqueuing the compute that consumes that packet, so that the
        transfer only waits for work that is already ahead of it.

        `confirm_sent=True` first waits on the host for the packet's metadata message, which the
        sender issues together with the payload: if the peer never sent, that wait runs into the
        group's timeout and raises, and no device-side receive is left waiting on the GPU."""
        e = self.up
        i = e.next
        e.next = (i + 1) % len(e.bufs)
        if confirm_sent:
            e.meta_works[i] = dist.irecv(e.meta[i], src=e.peer, group=e.meta_group)
            e.meta_works[i].wait()
            e.meta_works[i] = None
        if self._side is not None:
            # order after everything already enqueued on the compute stream (the previous user of
            # this buffer), but not after what the caller enqueues next
            self._side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._side):
                e.works[i] = dist.irecv(e.bufs[i], src=e.peer, group=e.group)
        else:
            e.works[i] = dist.irecv(e.bufs[i], src=e.peer, group=e.group)
        if not confirm_sent:
            e.meta_works[i] = dist.irecv(e.meta[i], src=e.peer, group=e.meta_group)
        e.posted.append(i)

    def recv(self) -> StagePacket:
        """Next packet from the previous stage.  Blocks the host only for the metadata message;
        the payload is ordered on the current CUDA stream."""
        e = self.up
        if not e.posted:
            self.post_recv()
        i = e.posted.popleft()
        if e.meta_works[i] is not None:    # None: already taken in by post_recv(confirm_sent=True)
            e.meta_works[i].wait()
            e.meta_works[i] = None
        e.works[i].wait()          # NCCL: makes the current stream wait; gloo: blocks
        e.works[i] = None
        m = e.meta[i].tolist()
        prompt = None
        if int(m[0]) == -1:                # restart: the prompt text follows on the host group
            raw = torch.empty(int(m[1]), dtype=torch.uint8)
            if raw.numel():
                dist.recv(raw, src=e.peer, group=e.meta_group)
            prompt = bytes(raw.tolist()).decode("utf-8")
        buf = e.bufs[i]
        act = buf[:self.act_numel].view(self.act_shape) if self._up_has_act else None
        lat = buf[(self.act_numel if self._up_has_act else 0):].view(self.latent_shape)
        r = self.rows
        return StagePacket(int(m[0]), int(m[1]), [int(x) for x in m[2:7]], [int(x) for x in m[7:7 + r]],
                           [int(x) for x in m[7 + r:7 + 2 * r]], act, lat, prompt)

    # ------------------------------------------------------------------ send side
    def send(self, chunk_idx: int, activations: Optional[torch.Tensor], latents: torch.Tensor,
             patched_x_shape: Sequence[int], starts: Sequence[int], ends: Sequence[int], current_step: int) -> None:
        """Hand a packet to the next stage; returns immediately (the copy into the send buffer and
        the transfer are ordered after the work already enqueued on the current stream)."""
        e = self.down
        i = e.next
        e.next = (i + 1) % len(e.bufs)
        if e.works[i] is not None:
            e.works[i].wait()          # the transfer that last used this buffer
            e.meta_works[i].wait()
        buf = e.bufs[i]
        off = 0
        if self._down_has_act:
            if activations is None or activations.numel() != self.act_numel:
                raise ValueError("activations do not match the link's fixed shape")
            buf[:self.act_numel].view(self.act_shape).copy_(activations)
            off = self.act_numel
        if latents.numel() != self.lat_numel:
            raise ValueError("latents do not match the link's fixed shape")
        buf[off:].view(self.latent_shape).copy_(latents)
        if len(starts) != self.rows or len(ends) != self.rows or len(patched_x_shape) != 5:
            raise ValueError("metadata does not match the link's row count")
        e.meta[i].copy_(torch.tensor([chunk_idx, current_step, *patched_x_shape, *starts, *ends], dtype=torch.int64))
        e.meta_works[i] = dist.isend(e.meta[i], dst=e.peer, group=e.meta_group)
        e.works[i] = dist.isend(buf, dst=e.peer, group=e.group)

    def send_restart(self, prompt: str) -> None:
        """Tell the next stage that the stream starts over with `prompt`.  The packet has the usual
        fixed-size payload (whatever the send buffer holds; receivers ignore it), `chunk_idx = -1`
        and the prompt's byte length in the `current_step` field; the text follows."""
        e = self.down
        i = e.next
        e.next = (i + 1) % len(e.bufs)
        if e.works[i] is not None:
            e.works[i].wait()
            e.meta_works[i].wait()
        data = prompt.encode("utf-8")
        e.meta[i].zero_()
        e.meta[i][0] = -1
        e.meta[i][1] = len(data)
        e.meta_works[i] = dist.isend(e.meta[i], dst=e.peer, group=e.meta_group)
        e.works[i] = dist.isend(e.bufs[i], dst=e.peer, group=e.group)
        if data:
            dist.send(torch.tensor(list(data), dtype=torch.uint8), dst=e.peer, group=e.meta_group)

    def drain(self) -> None:
        """Wait for every outstanding send (call before tearing the process group down)."""
        e = self.down
        for i in range(len(e.bufs)):           # a finished work must not be waited on twice
            if e.works[i] is not None:
                e.works[i].wait()
                e.works[i] = None
            if e.meta_works[i] is not None:
                e.meta_works[i].wait()
                e.meta_works[i] = None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

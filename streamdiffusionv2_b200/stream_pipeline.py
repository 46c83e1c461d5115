"""Host-side mirror of the reference's streaming scheduler around the causal DiT.

`FlowSchedule`      sigma/timestep tables and the forward-noising rule (models/wan/flow_match.py).
`DiffusionWrapper`  flow prediction -> x0 and the three entry points the drivers call
                    (models/wan/wan_wrapper.py:174-340): forward, forward_input, forward_output.
`StreamPipeline`    owner of the cache dicts and of the stream-batch state
                    (models/wan/causal_stream_inference.py:87-420): prepare, inference_stream,
                    inference_wo_batch, inference (pipeline-parallel stages).

The cache dicts have the reference's keys and layouts, so the reference's own tools that touch them
(cache re-ownership, session reset) keep working.  Unlike the reference, the per-row chunk starts
are also kept as Python ints, which lets a whole chunk step run without a device read-back.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.nn as nn

from .causal_attention import HostStarts


def assign_ints(t: torch.Tensor, values) -> None:
    """t[j] = values[j] with device-side fills.  A copy from pageable host memory would make the
    stream wait for all earlier work before it starts, i.e. synchronise the host with the GPU."""
    for j, v in enumerate(values):
        t[j:j + 1].fill_(int(v))       # `t[j] = v` goes through a host scalar tensor and synchronises


class FlowSchedule:
    """Shifted linear sigma table; timesteps = sigma * 1000 (flow_match.py:7-45, with
    extra_one_step=True, sigma_min=0, as the wrapper configures it, wan_wrapper.py:164-167)."""

    def __init__(self, shift: float = 8.0, num_steps: int = 1000, sigma_min: float = 0.0, sigma_max: float = 1.0):
        s = torch.linspace(sigma_max, sigma_min, num_steps + 1)[:-1]
        self.sigmas = shift * s / (1 + (shift - 1) * s)
        self.timesteps = self.sigmas * num_steps

    def to(self, device):
        self.sigmas = self.sigmas.to(device)
        self.timesteps = self.timesteps.to(device)
        return self

    def sigma_of(self, timestep: torch.Tensor, dtype=None) -> torch.Tensor:
        """sigma of the table entry nearest to each timestep; [n] -> [n, 1, 1, 1]."""
        self.to(timestep.device)
        ts, sg = (self.timesteps, self.sigmas) if dtype is None else (self.timesteps.to(dtype), self.sigmas.to(dtype))
        idx = torch.argmin((ts.unsqueeze(0) - timestep.unsqueeze(1)).abs(), dim=1)
        return sg[idx].reshape(-1, 1, 1, 1)

    def add_noise(self, clean: torch.Tensor, noise: torch.Tensor, timestep: torch.Tensor) -> torch.Tensor:
        """(1 - sigma) * clean + sigma * noise for [n, C, H, W] tensors (flow_match.py:62-78)."""
        sigma = self.sigma_of(timestep)
        return ((1 - sigma) * clean + sigma * noise).type_as(noise)


class DiffusionWrapper(nn.Module):
    """Wraps the DiT: latents are [B, F, C, H, W] outside, [B, C, F, H, W] inside; the model's flow
    prediction is turned into an x0 prediction in float64 (wan_wrapper.py:174-199)."""

    def __init__(self, model: nn.Module, seq_len: int = 32760, shift: float = 8.0):
        super().__init__()
        self.model = model
        self.scheduler = FlowSchedule(shift=shift)
        self.seq_len = seq_len
        self.uniform_timestep = False

    def get_scheduler(self) -> FlowSchedule:
        return self.scheduler

    def _x0(self, flow: torch.Tensor, xt: torch.Tensor, timestep: torch.Tensor) -> torch.Tensor:
        sigma = self.scheduler.sigma_of(timestep.double(), dtype=torch.float64)
        return (xt.double() - sigma * flow.double()).to(flow.dtype)

    def forward(self, noisy_image_or_video, conditional_dict, timestep, kv_cache=None, crossattn_cache=None,
                current_start=None, current_end=None):
        flow = self.model(noisy_image_or_video.permute(0, 2, 1, 3, 4), t=timestep,
                          context=conditional_dict["prompt_embeds"], seq_len=self.seq_len, kv_cache=kv_cache,
                          crossattn_cache=crossattn_cache, current_start=current_start,
                          current_end=current_end).permute(0, 2, 1, 3, 4)
        return self._x0(flow.flatten(0, 1), noisy_image_or_video.flatten(0, 1),
                        timestep.flatten(0, 1)).unflatten(0, flow.shape[:2])

    def forward_input(self, noisy_image_or_video, conditional_dict, timestep, block_mode="input", block_num=None,
                      kv_cache=None, crossattn_cache=None, current_start=None, current_end=None,
                      patched_x_shape=None, block_x=None, half_blocks=None):
        """First or middle pipeline stage: returns (activations [B, L, dim], patched_x_shape)."""
        assert kv_cache is not None, "kv_cache must be provided"
        x = block_x if (block_x is not None and block_mode == "middle") else noisy_image_or_video.permute(0, 2, 1, 3, 4)
        return self.model(x, t=timestep, context=conditional_dict["prompt_embeds"], seq_len=self.seq_len,
                          kv_cache=kv_cache, crossattn_cache=crossattn_cache, current_start=current_start,
                          current_end=current_end, block_mode=block_mode, block_num=block_num,
                          patched_x_shape=patched_x_shape, **({} if half_blocks is None else {"half_blocks": half_blocks}))

    def forward_output(self, noisy_image_or_video, conditional_dict, timestep, block_mode="output", block_num=None,
                       kv_cache=None, crossattn_cache=None, current_start=None, current_end=None,
                       patched_x_shape=None, block_x=None, half_blocks=None):
        """Last pipeline stage: remaining blocks, head, x0 of the stage's latents."""
        assert kv_cache is not None, "kv_cache must be provided"
        flow = self.model(block_x, t=timestep, context=conditional_dict["prompt_embeds"], seq_len=self.seq_len,
                          kv_cache=kv_cache, crossattn_cache=crossattn_cache, current_start=current_start,
                          current_end=current_end, block_mode=block_mode, block_num=block_num,
                          patched_x_shape=patched_x_shape,
                          **({} if half_blocks is None else {"half_blocks": half_blocks})).permute(0, 2, 1, 3, 4)
        return self._x0(flow.flatten(0, 1), noisy_image_or_video.flatten(0, 1),
                        timestep.flatten(0, 1)).unflatten(0, flow.shape[:2])


class StreamPipeline(nn.Module):
    """Stream-batch scheduler: batch row i holds the chunk that entered i calls ago, at denoise
    level i, with its own copy of every layer's K/V cache."""

    def __init__(self, generator: DiffusionWrapper, text_encoder: Callable, denoising_step_list: Sequence[int],
                 num_transformer_blocks: int, num_heads: int, frame_seq_length: int, num_kv_cache: int,
                 num_sink_tokens: int, adapt_sink_threshold: float = -1, num_frame_per_block: int = 1,
                 device="cuda", head_dim: int = 128, warp_denoising_step: bool = False, drop_final_zero: bool = True):
        super().__init__()
        self.generator = generator
        self.text_encoder = text_encoder
        self.device = torch.device(device)
        self.scheduler = generator.get_scheduler()
        steps = torch.tensor(list(denoising_step_list), dtype=torch.long, device=self.device)
        if drop_final_zero and steps[-1].item() == 0:
            steps = steps[:-1]                                    # causal_stream_inference.py:75-78
        if warp_denoising_step:                                    # :80-85
            table = torch.cat((self.scheduler.timesteps.cpu(), torch.tensor([0], dtype=torch.float32))).to(self.device)
            steps = table[1000 - steps]
        self.denoising_step_list = steps
        self.num_transformer_blocks, self.num_heads, self.head_dim = num_transformer_blocks, num_heads, head_dim
        self.frame_seq_length = frame_seq_length
        self.num_kv_cache = num_kv_cache
        self.kv_cache_length = frame_seq_length * num_kv_cache
        self.num_sink_tokens = num_sink_tokens
        self.adapt_sink_threshold = adapt_sink_threshold
        self.num_frame_per_block = num_frame_per_block
        self.generator.model.num_frame_per_block = num_frame_per_block
        self.kv_cache1 = None
        self.crossattn_cache = None
        self.hidden_states = None
        self.block_x = None
        self.conditional_dict = None
        self._starts_host: List[int] = []
        self._ends_host: List[int] = []
        self.step_graphs = None      # StepGraphs once enable_step_graphs() was called
        self._graph_in = None

    # ------------------------------------------------------------------ CUDA-graph replay of steady steps
    def enable_step_graphs(self, enabled: bool = True) -> None:
        """Replay the DiT forward of steady-state chunk steps from a CUDA graph (step_graph.py).
        Call after `prepare`, and again after every later `prepare` (a new prompt or stream replaces
        the tensors a recorded step points at, so `prepare` drops the recordings).  Results, cache
        contents and index state are those of the eager path; steps that are not in steady state
        still run eagerly."""
        if not enabled:
            self.step_graphs = None
            return
        if self.kv_cache1 is None or self.hidden_states is None:
            raise RuntimeError("call prepare() first")
        if self.device.type != "cuda":
            raise RuntimeError("step graphs need a CUDA device")
        from .step_graph import StepGraphs
        self.step_graphs = StepGraphs(self.device, self.num_transformer_blocks, self.hidden_states.shape[0])
        self._graph_in = torch.empty_like(self.hidden_states)

    def _forward(self, key, fn, blocks: range, allow_record: bool = True, cross_blocks: Optional[range] = None):
        """fn() eagerly, or through the step graphs when they are enabled.  `blocks`: the blocks whose
        self-attention (K/V cache) runs in fn; `cross_blocks`: those whose cross-attention does (the
        same unless a stage boundary lies inside a block)."""
        if self.step_graphs is None:
            return fn(), False
        cross = blocks if cross_blocks is None else cross_blocks
        layers = [(self.generator.model.blocks[i].self_attn, self.kv_cache1[i],
                   self.crossattn_cache[i] if i in cross else None) for i in blocks]
        layers += [(None, None, self.crossattn_cache[i]) for i in cross if i not in blocks]
        n_new = self.hidden_states.shape[1] * self.frame_seq_length
        before = self.step_graphs.replays
        out = self.step_graphs.run(key, fn, layers, self._starts_host, n_new, allow_record=allow_record)
        return out, self.step_graphs.replays != before

    # ------------------------------------------------------------------ cache allocation
    def _initialize_kv_cache(self, batch_size, dtype, device):
        steps = len(self.denoising_step_list)
        self.kv_cache1 = []
        for blk in self.generator.model.blocks:
            blk.self_attn.sink_size = self.num_sink_tokens
            blk.self_attn.adapt_sink_thr = self.adapt_sink_threshold
            shape = [batch_size, self.kv_cache_length, self.num_heads, self.head_dim]
            self.kv_cache1.append({
                "k": torch.zeros(shape, dtype=dtype, device=device),
                "v": torch.zeros(shape, dtype=dtype, device=device),
                "global_end_index": torch.tensor([0], dtype=torch.long, device=device),
                "local_end_index": torch.tensor([0], dtype=torch.long, device=device),
                "total_steps": steps,
                "current_step": steps,
            })

    def _initialize_crossattn_cache(self, batch_size, dtype, device):
        shape = [batch_size, 512, self.num_heads, self.head_dim]
        self.crossattn_cache = [{"k": torch.zeros(shape, dtype=dtype, device=device),
                                 "v": torch.zeros(shape, dtype=dtype, device=device), "is_init": False}
                                for _ in range(self.num_transformer_blocks)]

    # ------------------------------------------------------------------ first chunk
    def prepare(self, text_prompts, device, dtype, block_mode="input", noise=None, current_start=0,
                current_end=None, block_num=None, batch_denoise=True, owned_blocks: Optional[range] = None,
                unowned: str = "cpu"):
        """Runs the first chunk through every denoise level with one cache row, then replicates the
        caches to one row per level (causal_stream_inference.py:124-255).  `owned_blocks`, when
        given, keeps only that range of K/V caches on the device (pipeline-parallel stage); the
        others are moved to host memory as the reference does (`unowned="cpu"`) or released
        (`unowned="free"`)."""
        self.device = torch.device(device)
        # recorded steps hold the addresses of the caches and of the text K/V that this call replaces
        self.step_graphs, self._graph_in = None, None
        batch_size = noise.shape[0]
        self.conditional_dict = self.text_encoder(text_prompts=text_prompts)
        if self.kv_cache1 is None:
            self._initialize_kv_cache(batch_size, dtype, device)
            self._initialize_crossattn_cache(batch_size, dtype, device)
        else:
            for c in self.crossattn_cache:
                c["is_init"] = False
        start_t = torch.tensor([current_start], dtype=torch.long, device=device)
        end_t = torch.tensor([current_end], dtype=torch.long, device=device)
        starts = HostStarts(start_t, [current_start])
        levels = len(self.denoising_step_list)
        denoised = None
        for index, level in enumerate(self.denoising_step_list):
            timestep = torch.ones([batch_size, noise.shape[1]], device=noise.device, dtype=torch.int64) * level
            denoised = self.generator(noisy_image_or_video=noise, conditional_dict=self.conditional_dict,
                                      timestep=timestep, kv_cache=self.kv_cache1,
                                      crossattn_cache=self.crossattn_cache, current_start=starts, current_end=end_t)
            if index < levels - 1:
                nxt = self.denoising_step_list[index + 1]
                noise = self.scheduler.add_noise(
                    denoised.flatten(0, 1), torch.randn_like(denoised.flatten(0, 1)),
                    nxt * torch.ones([batch_size], device=noise.device, dtype=torch.long)
                ).unflatten(0, denoised.shape[:2])
        if not batch_denoise:
            return denoised

        self.batch_size = levels
        if owned_blocks is None and block_num is not None:
            b = [int(i) for i in (block_num.tolist() if isinstance(block_num, torch.Tensor) else block_num)]
            owned_blocks = range(b[0], b[1])
        for i in range(self.num_transformer_blocks):
            kv, cc = self.kv_cache1[i], self.crossattn_cache[i]
            if torch.distributed.is_available() and torch.distributed.is_initialized():
                for t in (cc["k"], cc["v"], kv["k"], kv["v"]):
                    torch.distributed.broadcast(t, src=0)
            if owned_blocks is not None and i not in owned_blocks and unowned == "free":
                kv["k"], kv["v"] = kv["k"][:, :0], kv["v"][:, :0]
            kv["k"] = kv["k"].repeat(levels, 1, 1, 1)
            kv["v"] = kv["v"].repeat(levels, 1, 1, 1)
            kv["global_end_index"] = kv["global_end_index"].repeat(levels)
            kv["local_end_index"] = kv["local_end_index"].repeat(levels)
            cc["k"] = cc["k"].expand(levels, -1, -1, -1)
            cc["v"] = cc["v"].expand(levels, -1, -1, -1)
            if owned_blocks is not None and i not in owned_blocks and unowned == "cpu":
                kv["k"], kv["v"] = kv["k"].cpu(), kv["v"].cpu()

        self.hidden_states = torch.zeros((levels, self.num_frame_per_block, *noise.shape[2:]), dtype=noise.dtype,
                                         device=device)
        if block_mode in ("output", "middle"):
            # sized for the whole chunk; the reference sizes it for a single frame, which only
            # fits one-frame chunks (causal_stream_inference.py:241-244)
            self.block_x = torch.zeros((levels, self.frame_seq_length * self.num_frame_per_block,
                                        self.num_heads * self.head_dim), dtype=noise.dtype, device=device)
        else:
            self.block_x = None
        self.kv_cache_starts = torch.ones(levels, dtype=torch.long, device=device) * current_end
        self.kv_cache_ends = torch.ones(levels, dtype=torch.long, device=device) * current_end + self.frame_seq_length
        self._starts_host = [int(current_end)] * levels
        self._ends_host = [int(current_end) + self.frame_seq_length] * levels
        self.timestep = self.denoising_step_list
        self.conditional_dict["prompt_embeds"] = self.conditional_dict["prompt_embeds"].repeat(levels, 1, 1)
        return denoised

    # ------------------------------------------------------------------ per-chunk steps
    def _shift_in(self, noise, current_start, current_end):
        self.hidden_states[1:] = self.hidden_states[:-1].clone()
        self.hidden_states[0] = noise[0]
        self.kv_cache_starts[1:] = self.kv_cache_starts[:-1].clone()
        self.kv_cache_starts[0:1].fill_(int(current_start))
        self.kv_cache_ends[1:] = self.kv_cache_ends[:-1].clone()
        self.kv_cache_ends[0:1].fill_(int(current_end))
        self._starts_host = [int(current_start)] + self._starts_host[:-1]
        self._ends_host = [int(current_end)] + self._ends_host[:-1]

    def _renoise(self, x):
        for i in range(len(self.denoising_step_list) - 1):
            row = x[i:i + 1]          # slices, not list indices: an index list is copied host->device
            x[i:i + 1] = self.scheduler.add_noise(
                row, torch.randn_like(row),
                self.denoising_step_list[i + 1] * torch.ones([1], device=x.device, dtype=torch.long))
        return x

    def inference_stream(self, noise, current_start, current_end, current_step=None):
        """One chunk step of the stream batch (causal_stream_inference.py:257-296): shift rows
        down, run all levels in one batched forward, re-noise rows 0..levels-2."""
        self._shift_in(noise, current_start, current_end)
        if current_step is not None:
            self.timestep[0] = current_step
        x_in = self.hidden_states
        if self.step_graphs is not None:             # a recorded forward reads its input at a fixed address
            self._graph_in.copy_(self.hidden_states)
            x_in = self._graph_in
        fn = lambda: self.generator(
            noisy_image_or_video=x_in, conditional_dict=self.conditional_dict,
            timestep=self.timestep.unsqueeze(1).expand(-1, x_in.shape[1]),
            kv_cache=self.kv_cache1, crossattn_cache=self.crossattn_cache,
            current_start=HostStarts(self.kv_cache_starts, self._starts_host), current_end=self.kv_cache_ends)
        out, replayed = self._forward(("stream", tuple(x_in.shape)), fn, range(self.num_transformer_blocks))
        self.hidden_states = out.clone() if replayed else out    # a graph's output is overwritten by its next replay
        return self._renoise(self.hidden_states)

    def inference_wo_batch(self, noise, current_start, current_end, current_step=None):
        """All denoise levels of one chunk in sequence against a one-row cache
        (causal_stream_inference.py:298-348)."""
        batch_size = noise.shape[0]
        start_t = torch.ones(batch_size, dtype=torch.long, device=self.device) * current_start
        end_t = torch.ones(batch_size, dtype=torch.long, device=self.device) * current_end
        starts = HostStarts(start_t, [int(current_start)] * batch_size)
        if current_step is not None:
            self.denoising_step_list[0] = current_step
        levels = len(self.denoising_step_list)
        denoised = None
        for index, level in enumerate(self.denoising_step_list):
            timestep = torch.ones([batch_size, noise.shape[1]], device=noise.device, dtype=torch.int64) * level
            denoised = self.generator(noisy_image_or_video=noise, conditional_dict=self.conditional_dict,
                                      timestep=timestep, kv_cache=self.kv_cache1,
                                      crossattn_cache=self.crossattn_cache, current_start=starts, current_end=end_t)
            if index < levels - 1:
                nxt = self.denoising_step_list[index + 1]
                noise = self.scheduler.add_noise(
                    denoised.flatten(0, 1), torch.randn_like(denoised.flatten(0, 1)),
                    nxt * torch.ones([batch_size], device=noise.device, dtype=torch.long)
                ).unflatten(0, denoised.shape[:2])
        return denoised

    def inference(self, noise, current_start, current_end, current_step, block_mode="input", block_num=None,
                  patched_x_shape=None, block_x=None, starts_host: Optional[Sequence[int]] = None,
                  allow_record: bool = True, half_blocks: Optional[Sequence[int]] = None):
        """One chunk step of one pipeline stage (causal_stream_inference.py:350-420).  'input':
        shift the new chunk in and run the first block range; 'middle'/'output': adopt the
        previous stage's activations, latents and row starts, run this stage's range.  `half_blocks`
        = (a, b) gives the range in half-block units instead of `block_num` (see the model)."""
        if block_mode == "input":
            self._shift_in(noise, current_start, current_end)
        else:
            self.block_x.copy_(block_x)
            self.hidden_states.copy_(noise)
            if isinstance(current_start, torch.Tensor):
                self.kv_cache_starts.copy_(current_start)
                self._starts_host = [int(v) for v in (starts_host if starts_host is not None
                                                      else current_start.tolist())]
            else:                                             # host lists: no read-back, no host->device copy
                self._starts_host = [int(v) for v in current_start]
                assign_ints(self.kv_cache_starts, self._starts_host)
            if isinstance(current_end, torch.Tensor):
                self.kv_cache_ends.copy_(current_end)
                self._ends_host = [int(v) for v in current_end.tolist()]
            else:
                self._ends_host = [int(v) for v in current_end]
                assign_ints(self.kv_cache_ends, self._ends_host)
        if current_step is not None:
            self.timestep[0] = current_step
        common = dict(conditional_dict=self.conditional_dict,
                      timestep=self.timestep.unsqueeze(1).expand(-1, self.hidden_states.shape[1]),
                      kv_cache=self.kv_cache1, crossattn_cache=self.crossattn_cache,
                      current_start=HostStarts(self.kv_cache_starts, self._starts_host),
                      current_end=self.kv_cache_ends, block_mode=block_mode, block_num=block_num,
                      patched_x_shape=patched_x_shape, block_x=self.block_x)
        rng = [int(i) for i in (block_num.tolist() if isinstance(block_num, torch.Tensor) else block_num)]
        owned, cross = range(rng[0], rng[-1]), None
        if half_blocks is not None:
            lo, hi = int(half_blocks[0]), int(half_blocks[1])
            common["half_blocks"] = (lo, hi)
            owned, cross = range((lo + 1) // 2, (hi + 1) // 2), range(lo // 2, hi // 2)
            rng = [lo / 2, hi / 2]
        key = (block_mode, rng[0], rng[-1], tuple(self.hidden_states.shape),
               tuple(int(i) for i in patched_x_shape) if isinstance(patched_x_shape, (list, tuple)) else None)
        if block_mode == "output":
            fn = lambda: self.generator.forward_output(noisy_image_or_video=self.hidden_states, **common)
            denoised, replayed = self._forward(key, fn, owned, allow_record, cross)
            return self._renoise(denoised.clone() if replayed else denoised), None
        fn = lambda: self.generator.forward_input(noisy_image_or_video=self.hidden_states, **common)
        return self._forward(key, fn, owned, allow_record, cross)[0]

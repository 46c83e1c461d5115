"""Host-side mirror of the causal Wan DiT interface, built on the sm_100a attention kernels.

`CausalWanModel` takes the same constructor arguments, exposes the same parameter names and the
same kv-cache forward signature as the reference model (models/wan/causal_model.py:523-651,
700-840), so a checkpoint written for one loads into the other with strict=True and the reference
drivers can call either.  Only the inference (kv-cache) path exists here; everything that is not
attention is ordinary PyTorch (library GEMMs, norms), the attention modules call the kernels
through `causal_attention`.

Layout of one block (models/wan/causal_model.py:432-487): adaptive-LayerNorm modulated
self-attention over the ring cache, text cross-attention from the persistent cache, gated FFN;
six modulation vectors per frame come from the timestep embedding.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Union

import torch
import torch.nn as nn

from . import causal_attention as CA
from . import ops


# Residual addition + the LayerNorm of its result as one launch (ops.residual_layernorm); False runs them apart.
FUSE_RESIDUAL_LN = True


def _fusable(x: torch.Tensor) -> bool:
    """The fused element-wise kernels serve bf16 CUDA tensors; anything else (the fp32 CPU runs
    of the tests) takes the PyTorch op chain they reproduce."""
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192


def timestep_features(dim: int, t: torch.Tensor) -> torch.Tensor:
    """[cos | sin] of t * 10000^(-i/half) in float64 (models/wan/wan_base/modules/model.py:15-26)."""
    half = dim // 2
    t = t.to(torch.float64)
    freq = torch.pow(10000, -torch.arange(half, device=t.device, dtype=torch.float64) / half)
    ang = torch.outer(t, freq)
    return torch.cat([ang.cos(), ang.sin()], dim=1)


def build_rope_table(head_dim: int, positions: int = 1024, theta: float = 10000.0) -> torch.Tensor:
    """complex128 [positions, head_dim/2]: temporal, height and width column groups
    (models/wan/causal_model.py:631-638; models/wan/wan_base/modules/model.py:29-36)."""
    def unit(dim):
        inv = 1.0 / torch.pow(theta, torch.arange(0, dim, 2, dtype=torch.float64) / dim)
        ang = torch.outer(torch.arange(positions), inv)
        return torch.polar(torch.ones_like(ang), ang)
    d = head_dim
    return torch.cat([unit(d - 4 * (d // 6)), unit(2 * (d // 6)), unit(2 * (d // 6))], dim=1)


class RMSNorm(nn.Module):
    """x / rms(x) * weight with the statistics in fp32 (model.py:70-86)."""

    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.dim, self.eps = dim, eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        if _fusable(x) and self.weight.dtype == torch.bfloat16:
            return ops.rmsnorm(x, self.weight, self.eps)       # one launch, same roundings
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.eps)).type_as(x) * self.weight


class PlainLayerNorm(nn.LayerNorm):
    """LayerNorm that returns its input's dtype (model.py:89-100)."""

    def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = False):
        super().__init__(dim, eps=eps, elementwise_affine=elementwise_affine)

    def forward(self, x):
        return super().forward(x).type_as(x)


class _AttentionBase(nn.Module):
    def __init__(self, dim: int, num_heads: int, qk_norm: bool = True, eps: float = 1e-6):
        super().__init__()
        assert dim % num_heads == 0
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.qk_norm, self.eps = qk_norm, eps
        self.q = nn.Linear(dim, dim)
        self.k = nn.Linear(dim, dim)
        self.v = nn.Linear(dim, dim)
        self.o = nn.Linear(dim, dim)
        self.norm_q = RMSNorm(dim, eps=eps) if qk_norm else nn.Identity()
        self.norm_k = RMSNorm(dim, eps=eps) if qk_norm else nn.Identity()


class CausalSelfAttention(_AttentionBase):
    """Self-attention over the sink + ring K/V cache.  Carries the same mutable attributes as the
    reference module: `sink_size`, `adapt_sink_thr`, `evict_idx` (causal_model.py:177-179)."""

    def __init__(self, dim, num_heads, qk_norm=True, eps=1e-6):
        super().__init__(dim, num_heads, qk_norm, eps)
        self.sink_size = 3
        self.adapt_sink_thr = -1
        self.evict_idx = None

    forward = CA.self_attention_forward


class TextCrossAttention(_AttentionBase):
    """Cross-attention to the text context with K/V served from `crossattn_cache`."""

    forward = CA.cross_attention_forward


class DiTBlock(nn.Module):
    def __init__(self, dim, ffn_dim, num_heads, qk_norm=True, cross_attn_norm=False, eps=1e-6):
        super().__init__()
        self.norm1 = PlainLayerNorm(dim, eps)
        self.self_attn = CausalSelfAttention(dim, num_heads, qk_norm, eps)
        self.norm3 = PlainLayerNorm(dim, eps, elementwise_affine=True) if cross_attn_norm else nn.Identity()
        self.cross_attn = TextCrossAttention(dim, num_heads, qk_norm, eps)
        self.norm2 = PlainLayerNorm(dim, eps)
        self.ffn = nn.Sequential(nn.Linear(dim, ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(ffn_dim, dim))
        self.modulation = nn.Parameter(torch.randn(1, 6, dim) / dim ** 0.5)

    def forward(self, x, e, grid_sizes, freqs, context, kv_cache, crossattn_cache, current_start, part="all",
                modulated=None):
        """x [B, L, C]; e [B, F, 6, C] (per-frame modulation from the timestep embedding); `modulated`, when
        given, is `self.modulation.unsqueeze(1) + e` computed by the caller (for all its blocks in one launch).
        `part` runs the block in two halves for pipeline stages that meet inside a block: "attn" ends
        after the self-attention residual (causal_model.py:463-471), "rest" resumes there (cross-
        attention and FFN, :473-483); "attn" then "rest" computes exactly what "all" does."""
        frames = e.shape[1]
        per_frame = x.shape[1] // frames
        if modulated is None:
            modulated = self.modulation.unsqueeze(1) + e
        shift_a, scale_a, gate_a, shift_f, scale_f, gate_f = modulated.chunk(6, dim=2)

        fused = _fusable(x) and shift_a.dtype == torch.bfloat16

        def norm_modulate(norm, y, scale, shift):
            if fused:
                return ops.ln_modulate(y, scale, shift, frames, norm.eps)
            return (norm(y).unflatten(1, (frames, per_frame)) * (1 + scale) + shift).flatten(1, 2)

        def add_gated(x, y, gate):
            if fused:
                return ops.gate_residual(x, y, gate, frames)
            return x + (y.unflatten(1, (frames, per_frame)) * gate).flatten(1, 2)

        # where a residual addition is followed by a LayerNorm of its result, both run as one launch
        fuse3 = fused and ops.can_fuse_layernorm(x, self.norm3)
        fuse2 = fused and FUSE_RESIDUAL_LN and x.shape[-1] <= 5120
        xn = None
        if part != "rest":
            y = self.self_attn(norm_modulate(self.norm1, x, scale_a, shift_a), None, grid_sizes, freqs, None,
                               kv_cache, current_start, None)
            if fuse3 and FUSE_RESIDUAL_LN and part == "all":
                x, xn = ops.residual_layernorm(x, y, gate_a, frames, self.norm3.eps, weight=self.norm3.weight,
                                               bias=self.norm3.bias)
            else:
                x = add_gated(x, y, gate_a)
            if part == "attn":
                return x
        if xn is None:
            xn = ops.layernorm_affine(x, self.norm3.weight, self.norm3.bias, self.norm3.eps) if fuse3 \
                else self.norm3(x)
        c = self.cross_attn(xn, context, None, crossattn_cache=crossattn_cache)
        if fuse2:
            x, h = ops.residual_layernorm(x, c, None, frames, self.norm2.eps, scale=scale_f, shift=shift_f)
        else:
            x = x + c
            h = norm_modulate(self.norm2, x, scale_f, shift_f)
        y = ops.ffn(self.ffn, h) if fused else self.ffn(h)
        return add_gated(x, y, gate_f)


class OutputHead(nn.Module):
    def __init__(self, dim, out_dim, patch_size, eps=1e-6):
        super().__init__()
        self.norm = PlainLayerNorm(dim, eps)
        self.head = nn.Linear(dim, math.prod(patch_size) * out_dim)
        self.modulation = nn.Parameter(torch.randn(1, 2, dim) / dim ** 0.5)

    def forward(self, x, e):
        """x [B, L, C]; e [B, F, 1, C] -> [B, F, L/F, prod(patch)*out_dim]."""
        frames = e.shape[1]
        shift, scale = (self.modulation.unsqueeze(1) + e).chunk(2, dim=2)
        return self.head(self.norm(x).unflatten(1, (frames, x.shape[1] // frames)) * (1 + scale) + shift)


def _stamp(x: torch.Tensor):
    """A point in time on x's device: a recorded CUDA event, or host seconds for CPU tensors."""
    if x.is_cuda:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e
    import time
    return time.perf_counter()


def _as_ints(v) -> List[int]:
    if isinstance(v, torch.Tensor):
        return [int(i) for i in v.reshape(-1).tolist()]
    if isinstance(v, (list, tuple)):
        return [int(i) for i in v]
    return [int(v)]


class CausalWanModel(nn.Module):
    """Causal Wan DiT, inference path.  `forward` keeps the reference's calling convention:
    positional (x, t, context, seq_len) plus kv_cache / crossattn_cache / current_start /
    current_end / block_mode / block_num / patched_x_shape keywords."""

    def __init__(self, model_type="t2v", patch_size=(1, 2, 2), text_len=512, in_dim=16, dim=2048, ffn_dim=8192,
                 freq_dim=256, text_dim=4096, out_dim=16, num_heads=16, num_layers=32, window_size=(-1, -1),
                 qk_norm=True, cross_attn_norm=True, eps=1e-6):
        super().__init__()
        if model_type != "t2v":
            raise NotImplementedError("only the text-to-video variant is used by the streaming pipelines")
        self.model_type, self.patch_size, self.text_len = model_type, tuple(patch_size), text_len
        self.in_dim, self.dim, self.ffn_dim, self.freq_dim = in_dim, dim, ffn_dim, freq_dim
        self.text_dim, self.out_dim, self.num_heads, self.num_layers = text_dim, out_dim, num_heads, num_layers
        self.eps = eps
        self.patch_embedding = nn.Conv3d(in_dim, dim, kernel_size=self.patch_size, stride=self.patch_size)
        self.text_embedding = nn.Sequential(nn.Linear(text_dim, dim), nn.GELU(approximate="tanh"), nn.Linear(dim, dim))
        self.time_embedding = nn.Sequential(nn.Linear(freq_dim, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(dim, dim * 6))
        self.blocks = nn.ModuleList(
            [DiTBlock(dim, ffn_dim, num_heads, qk_norm, cross_attn_norm, eps) for _ in range(num_layers)])
        self.head = OutputHead(dim, out_dim, self.patch_size, eps)
        head_dim = dim // num_heads
        assert head_dim % 2 == 0
        # plain attribute, not a buffer: .to(dtype) must not touch it (causal_model.py:630-638)
        self.freqs = build_rope_table(head_dim)
        self.num_frame_per_block = 1
        # set to a list to have every half block of a forward timed on its own: (half index, start, end)
        # stamps (CUDA events on a GPU, seconds on the host) are appended; None = off
        self.half_stamps = None
        self.last_patched_x_shape = None
        self._shape_tensors = {}
        self.reset_parameters()

    def reset_parameters(self):
        """Xavier for every Linear, N(0, 0.02) for the two embedding MLPs, zero output projection
        (causal_model.py:991-1013)."""
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.xavier_uniform_(m.weight)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
        nn.init.xavier_uniform_(self.patch_embedding.weight.flatten(1))
        for seq in (self.text_embedding, self.time_embedding):
            for m in seq.modules():
                if isinstance(m, nn.Linear):
                    nn.init.normal_(m.weight, std=0.02)
        nn.init.zeros_(self.head.head.weight)

    # ------------------------------------------------------------------ forward
    def forward(self, *args, **kwargs):
        if kwargs.get("kv_cache") is None:
            raise NotImplementedError("this model serves the kv-cache inference path only")
        return self._forward_inference(*args, **kwargs)

    def _forward_inference(self, x, t, context, seq_len, clip_fea=None, y=None, kv_cache=None, crossattn_cache=None,
                           current_start=0, current_end=0, block_mode="input", block_num=(-1,),
                           patched_x_shape=None, half_blocks=None):
        """x: [B, C, F, H, W] latents ('input' mode) or [B, L, dim] activations of the previous
        pipeline stage ('middle' / 'output'); t: [B, F] timesteps; context: [B, Lt, text_dim].
        Returns [B, C, F, H, W], or (activations, patched_x_shape) when the stage ends before the
        last block.  block_num = (first_block, end_block) of this stage.  `half_blocks` = (a, b), when
        given, replaces it with a range in half-block units (half 2i = self-attention part of block i,
        half 2i + 1 = its cross-attention + FFN part), so that stages may meet inside a block; the
        reference knows whole blocks only (causal_model.py:794-833)."""
        device = self.patch_embedding.weight.device
        if self.freqs.device != device:
            self.freqs = self.freqs.to(device)
        rng = _as_ints(block_num)
        first, last = rng[0], rng[-1]

        if block_mode == "input":
            x = self.patch_embedding(x if isinstance(x, torch.Tensor) else torch.stack(list(x)))
            bsz, cch, frames, gh, gw = x.shape
            self.last_patched_x_shape = [1, int(cch), int(frames), int(gh), int(gw)]   # host copy for stage links
            key = (tuple(self.last_patched_x_shape), str(device))
            patched_x_shape = self._shape_tensors.get(key)       # built once: a host->device copy synchronises
            if patched_x_shape is None:
                patched_x_shape = torch.tensor(self.last_patched_x_shape, dtype=torch.int64, device=device)
                self._shape_tensors[key] = patched_x_shape
            x = x.flatten(2).transpose(1, 2)
        else:
            _, cch, frames, gh, gw = _as_ints(patched_x_shape)
            if x.shape[1] != frames * gh * gw:
                raise ValueError("stage activations do not match patched_x_shape")
            bsz = x.shape[0]
        grid_sizes = torch.tensor([[frames, gh, gw]] * bsz, dtype=torch.long)
        assert x.shape[1] <= seq_len

        e = self.time_embedding(timestep_features(self.freq_dim, t.flatten()).type_as(x))
        e0 = self.time_projection(e).unflatten(1, (6, self.dim)).unflatten(0, t.shape)

        n_blocks = len(self.blocks)
        if half_blocks is not None:
            lo, hi = int(half_blocks[0]), int(half_blocks[1])
            if not 0 <= lo <= hi <= 2 * n_blocks:
                raise ValueError("half_blocks outside the model")
            bounded = True
        else:
            lo = 2 * first if block_mode in ("output", "middle") else 0
            bounded = block_mode in ("input", "middle") and 0 <= last <= n_blocks
            hi = 2 * last if bounded else 2 * n_blocks
        if block_mode == "output":
            hi = 2 * n_blocks
        # a first or middle stage hands activations on; a range that reaches the end of the model does so
        # only in 'input' mode (the reference's convention, causal_model.py:819-833)
        hands_on = block_mode in ("input", "middle") and bounded and (hi < 2 * n_blocks or block_mode == "input")

        # the text embedding only feeds the cross-attention K/V projections, which are skipped once a
        # block's crossattn_cache is initialised: do not recompute it for blocks that will not read it
        # (a block reads it in its second half)
        need_ctx = crossattn_cache is None or any(
            c is None or not c.get("is_init", False) for c in crossattn_cache[lo // 2:hi // 2])
        ctx = None
        if need_ctx:
            ctx = context if isinstance(context, torch.Tensor) else torch.stack(
                [torch.cat([u, u.new_zeros(self.text_len - u.size(0), u.size(1))]) for u in context])
            if ctx.shape[1] < self.text_len:
                ctx = torch.cat([ctx, ctx.new_zeros(ctx.shape[0], self.text_len - ctx.shape[1], ctx.shape[2])], dim=1)
            ctx = self.text_embedding(ctx)

        starts = CA.HostStarts(current_start, CA.host_starts(current_start, bsz)) \
            if isinstance(current_start, torch.Tensor) else current_start

        # modulation + timestep embedding of every block of this range in one launch (the same element-wise
        # sums the blocks would form one by one)
        first_block, end_block = lo // 2, (hi + 1) // 2
        mods = None
        if end_block - first_block > 1:
            mods = self._stacked_modulation(first_block, end_block) + e0.unsqueeze(0)

        stamps = self.half_stamps
        h = lo
        while h < hi:
            idx, second = divmod(h, 2)
            if second:
                part, step = "rest", 1
            elif h + 1 < hi and stamps is None:
                part, step = "all", 2
            else:
                part, step = "attn", 1
            t0 = _stamp(x) if stamps is not None else None
            block = self.blocks[idx]
            x = block(x, e0, grid_sizes, self.freqs, ctx, kv_cache[idx], crossattn_cache[idx], starts, part=part,
                      modulated=None if mods is None else mods[idx - first_block])
            if stamps is not None:
                stamps.append((h, t0, _stamp(x)))
            h += step
        if hands_on:
            return x, patched_x_shape

        x = self.head(x, e.unflatten(0, t.shape).unsqueeze(2))
        return self.unpatchify(x, (frames, gh, gw))

    def _stacked_modulation(self, first: int, end: int) -> torch.Tensor:
        """[end - first, 1, 1, 6, C]: the blocks' modulation parameters side by side, rebuilt when one of
        them was written or replaced."""
        params = [self.blocks[i].modulation for i in range(first, end)]
        key = (first, end) + tuple((p.data_ptr(), p._version) for p in params)
        cached = getattr(self, "_mod_stack", None)
        if cached is None or cached[0] != key:
            with torch.no_grad():
                cached = (key, torch.stack([p.detach() for p in params]).unsqueeze(1))
            self._mod_stack = cached
        return cached[1]

    def unpatchify(self, x, grid):
        """[B, F, gh*gw, p0*p1*p2*C] -> [B, C, F*p0, gh*p1, gw*p2]."""
        f, gh, gw = grid
        p0, p1, p2 = self.patch_size
        b = x.shape[0]
        x = x.reshape(b, f, gh, gw, p0, p1, p2, self.out_dim)
        x = x.permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(b, self.out_dim, f * p0, gh * p1, gw * p2)

"""Kernel-backed forwards for the two attention modules of the causal Wan DiT.

`self_attention_forward` has the signature and the side effects of the reference
`CausalWanSelfAttention.forward` (models/wan/causal_model.py:189-389) on its kv-cache branch:
same `kv_cache` dict keys, same `evict_idx` / `sink_size` / `adapt_sink_thr` module attributes,
same cache contents and index tensors after the call.  `cross_attention_forward` mirrors
`WanT2VCrossAttention.forward` (models/wan/wan_base/modules/model.py:161-194) including the
`crossattn_cache` protocol.  `install(model)` binds them onto every block of a model that has the
reference's module layout, without touching parameters or their names.

Differences from the reference are in mechanism only: one fused launch ropes q/k and writes the
K/V slots for all rows, the slot arithmetic runs on host integers (no device read-backs), and
attention runs in the sm_100a kernels.  There is no fallback to PyTorch attention.
"""
from __future__ import annotations

import inspect
import math
import types
from typing import List, Optional, Sequence

import torch

from . import ops
from .ring_state import RingState

_start_cache = {}
_step_recorder = None
_POLL_EVERY = 32          # attention calls between two looks at the device status word
_calls_since_poll = 0


def set_step_recorder(recorder) -> None:
    """While set (a step is being recorded into a CUDA graph, see step_graph.py), the append kernel
    of every layer reads its per-row slot parameters from the recorder's device array instead of
    receiving them as launch arguments."""
    global _step_recorder
    _step_recorder = recorder


def host_starts(current_start, rows: int) -> List[int]:
    """`current_start` as Python ints.  The drivers pass a device int64 tensor that they update in
    place once per chunk; it is read back once per version and shared by all layers of a forward.
    A sequence of ints (or a `HostStarts`) skips the read-back entirely."""
    if isinstance(current_start, HostStarts):
        return current_start.values
    if isinstance(current_start, torch.Tensor):
        key = id(current_start)
        sig = (current_start.data_ptr(), current_start._version)
        hit = _start_cache.get(key)
        if hit is not None and hit[0] == sig and hit[2] is current_start:
            return hit[1]
        vals = [int(x) for x in current_start.reshape(-1).tolist()]
        if len(_start_cache) > 64:
            _start_cache.clear()
        _start_cache[key] = (sig, vals, current_start)
        return vals
    if isinstance(current_start, (list, tuple)):
        return [int(x) for x in current_start]
    return [int(current_start)] * rows


class HostStarts:
    """A device tensor of chunk starts together with its host copy, for callers that already know
    the values (avoids the one read-back per chunk)."""

    def __init__(self, tensor: torch.Tensor, values: Sequence[int]):
        self.tensor = tensor
        self.values = [int(v) for v in values]

    def __floordiv__(self, other):  # the model computes start_frame = current_start // frame_tokens
        return HostStarts(self.tensor // other, [v // int(other) for v in self.values])

    def tolist(self):
        return list(self.values)


def adaptive_similarities(kv_cache, roped_k, v, sink_size: int, frame_tokens: int) -> torch.Tensor:
    """[rows, sink] similarity of the new frame to every sink frame, for all rows at once, with the
    reference's own operations (causal_model.py:286-296): cosine similarity of the per-frame mean K,
    the same for V, averaged.  Rows are independent (row i reads cache row i only).  Stays on the
    device: the threshold test and everything that follows from it run in the plan kernel."""
    rows = roped_k.shape[0]
    if roped_k.is_cuda:
        # the four means in two launches, straight from the cache (no reshaped copies)
        means = ops.frame_means(kv_cache["k"][:rows], kv_cache["v"][:rows], roped_k, v, sink_size, frame_tokens)
        k_sink, k_new = means[:, :sink_size, 0], means[:, sink_size:, 0]
        v_sink, v_new = means[:, :sink_size, 1], means[:, sink_size:, 1]
    else:                                      # host tensors: only the tests of the host logic come here
        sink_tokens = sink_size * frame_tokens
        k_sink = kv_cache["k"][:rows, :sink_tokens].reshape(rows, sink_size, frame_tokens, -1).mean(2)
        k_new = roped_k.reshape(rows, 1, frame_tokens, -1).mean(2)
        v_sink = kv_cache["v"][:rows, :sink_tokens].reshape(rows, sink_size, frame_tokens, -1).mean(2)
        v_new = v.reshape(rows, 1, frame_tokens, -1).mean(2)
    k_sim = torch.cosine_similarity(k_sink, k_new, dim=-1)
    v_sim = torch.cosine_similarity(v_sink, v_new, dim=-1)
    return ((k_sim + v_sim) / 2).contiguous()


def sync_evict_queue(attn_module) -> None:
    """Refresh `attn_module.evict_idx` (the reference's attribute) from the device-resident queue that
    the adaptive sink path keeps (one read-back); no-op for modules whose queue lives on the host."""
    RingState.sync_queue(attn_module)


def cached_attention(attn_module, q, k, v, grid_sizes, freqs, kv_cache, current_start, norm=None):
    """Rope, slot write, index update and attention for already projected q/k/v [B, N, H, D].
    Returns the attention output [B, N, H, D].  This is the part of the reference forward between
    the qkv projection and the output projection (causal_model.py:250-384).  With `norm` =
    (weight_q, weight_k, eps) q and k are the raw projections and their RMS norm
    (causal_model.py:212-214) runs inside the append launch."""
    B, n_new, H, D = q.shape
    f, gh, gw = (int(x) for x in grid_sizes[0].tolist())
    frame_tokens = gh * gw
    starts = host_starts(current_start, B)
    if len(starts) < B:
        raise ValueError("current_start has fewer entries than batch rows")
    starts = starts[:B]
    start_frames = [s // frame_tokens for s in starts]
    table = ops.rope_table_device(freqs, q.device)
    state = RingState.of(kv_cache)
    index_tensors = (kv_cache["global_end_index"], kv_cache["local_end_index"])
    sink_tokens = attn_module.sink_size * frame_tokens
    adaptive = sink_tokens > 0 and attn_module.adapt_sink_thr > -1 and n_new <= frame_tokens

    extra = {} if norm is None else {"norm": norm}
    if not adaptive:
        dst, seq_lens = state.plan(kv_cache, attn_module, starts, n_new, frame_tokens)
        if _step_recorder is not None:
            extra["step_params"] = _step_recorder.layer_params(attn_module, kv_cache, start_frames, dst, state,
                                                               seq_lens, n_new, frame_tokens)
        roped_q = ops.rope_kv_append(q, k, v, kv_cache["k"], kv_cache["v"], table, (f, gh, gw), start_frames,
                                     dst, index_tensors=index_tensors,
                                     index_values=(state.global_end, state.local_end), **extra)
    else:
        # The slot of a row depends on the data (roped k against the sink frames already in the cache), so the
        # queue lives on the device: rope into a staging chunk, compute the similarities there, let the plan
        # kernel decide the slots, then run the append itself with the slots read from device memory.  Nothing
        # is read back.  Everything that does not depend on the data is still decided here, on host integers.
        if n_new != frame_tokens:
            raise RuntimeError("the adaptive sink test compares whole frames: one latent frame per chunk")
        queue = RingState.push_queue(kv_cache, attn_module, q.device)
        inputs = [[], [], [], [], [], [], []]
        seq_lens = []
        for i in range(B):
            evict, pop, push_value, begin, le = state.plan_row_split(kv_cache, attn_module, i, starts[i], n_new,
                                                                     frame_tokens)
            for lst, val in zip(inputs, (start_frames[i], state.global_end[i], le, int(evict), int(pop), push_value,
                                         begin)):
                lst.append(val)
            seq_lens.append(le)
        stage_kw = dict(extra)
        if _step_recorder is not None:      # a recorded step must not carry this step's start frames by value
            step_params, plan_kw, stage_kw["step_params"] = _step_recorder.adaptive_layer_params(
                attn_module, kv_cache, inputs, seq_lens, n_new, frame_tokens)
        else:
            step_params = torch.empty((4, B), dtype=torch.int64, device=q.device)
            plan_kw = {"host_inputs": inputs}
        stage_k = torch.empty((B, n_new, H, D), dtype=k.dtype, device=k.device)
        stage_v = torch.empty((B, n_new, H, D), dtype=v.dtype, device=v.device)
        ops.rope_kv_append(q, k, v, stage_k, stage_v, table, (f, gh, gw), start_frames, [0] * B, **stage_kw)
        sim = adaptive_similarities(kv_cache, stage_k, stage_v, attn_module.sink_size, frame_tokens)
        ops.ring_plan_adaptive(sim, attn_module.adapt_sink_thr, queue, frame_tokens, n_new, step_params, **plan_kw)
        roped_q = ops.rope_kv_append(q, k, v, kv_cache["k"], kv_cache["v"], table, (f, gh, gw), start_frames,
                                     [0] * B, index_tensors=index_tensors, step_params=step_params, **extra)

    if q.dtype == torch.bfloat16:
        out = ops.attn_kvcache(roped_q, kv_cache["k"], kv_cache["v"], seq_lens)
    else:
        out = ops.attn_kvcache_simt(roped_q, kv_cache["k"], kv_cache["v"], seq_lens)
    # a kernel that gave up a bounded wait wrote nothing: surface that instead of streaming garbage
    global _calls_since_poll
    _calls_since_poll += 1
    if _calls_since_poll >= _POLL_EVERY and _step_recorder is None:
        _calls_since_poll = 0
        ops.poll_status(q.device)
    return out


def _fusable(x: torch.Tensor) -> bool:
    """The fused element-wise kernels serve bf16 CUDA tensors with rows of at most 8192 elements."""
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192


def _qk_norm(norm, x: torch.Tensor) -> torch.Tensor:
    """norm(x) for the q / k norms.  An RMS norm with a bf16 weight (the reference's WanRMSNorm,
    models/wan/wan_base/modules/model.py:69-84, or this package's own) runs as one launch that
    reproduces its roundings; anything else (Identity when qk_norm is off, fp32 runs) is called as is."""
    w = getattr(norm, "weight", None)
    if (w is not None and type(norm).__name__.endswith("RMSNorm") and _fusable(x) and w.dtype == torch.bfloat16
            and hasattr(norm, "eps")):
        return ops.rmsnorm(x, w, norm.eps)
    return norm(x)


def _is_rms(norm) -> bool:
    w = getattr(norm, "weight", None)
    return w is not None and type(norm).__name__.endswith("RMSNorm") and hasattr(norm, "eps")


def _fused_qkv_weights(attn):
    """[3 * dim, dim] weight and [3 * dim] bias of the q | k | v projections of an attention module,
    concatenated once and kept on the module (`_sdv2_qkv`); rebuilt when any of the six parameters was
    replaced or written (identity, address, version counter).  The parameters themselves stay as
    they are, so checkpoints load and save unchanged."""
    lins = (attn.q, attn.k, attn.v)
    ps = [p for l in lins for p in (l.weight, l.bias)]
    key = tuple((id(p), p.data_ptr(), p._version) if p is not None else None for p in ps)
    hit = getattr(attn, "_sdv2_qkv", None)
    if hit is not None and hit[0] == key:
        return hit[1], hit[2]
    with torch.no_grad():
        w = torch.cat([l.weight for l in lins], dim=0).contiguous()
        b = None if any(l.bias is None for l in lins) else torch.cat([l.bias for l in lins], dim=0).contiguous()
    attn._sdv2_qkv = (key, w, b)
    return w, b


def project_qkv(attn, x):
    """q, k, v [b, s, n, d] of a self-attention module plus the norm still to be applied.
    On CUDA in bf16: one GEMM over the concatenated q | k | v weight, q / k / v are slices of its
    output, and when the q and k norms are RMS norms that the append kernel can fold in, they are
    returned as (weight_q, weight_k, eps) instead of being run.  Elsewhere: the module's own three
    projections and norms, as the reference runs them (causal_model.py:212-218)."""
    b, s, n, d = *x.shape[:2], attn.num_heads, attn.head_dim
    plain = all(type(l) is torch.nn.Linear for l in (attn.q, attn.k, attn.v))
    if _fusable(x) and plain and attn.q.weight.dtype == torch.bfloat16:
        w, bias = _fused_qkv_weights(attn)
        qkv = torch.nn.functional.linear(x, w, bias).view(b, s, 3, n, d)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if (_is_rms(attn.norm_q) and _is_rms(attn.norm_k) and attn.norm_q.eps == attn.norm_k.eps
                and ops.can_fuse_norm(q, k, v, attn.norm_q.weight, attn.norm_k.weight)):
            return q, k, v, (attn.norm_q.weight, attn.norm_k.weight, attn.norm_q.eps)
        q = _qk_norm(attn.norm_q, q.reshape(b, s, n * d)).view(b, s, n, d)
        k = _qk_norm(attn.norm_k, k.reshape(b, s, n * d)).view(b, s, n, d)
        return q, k, v, None
    q = _qk_norm(attn.norm_q, attn.q(x)).view(b, s, n, d)
    k = _qk_norm(attn.norm_k, attn.k(x)).view(b, s, n, d)
    v = attn.v(x).view(b, s, n, d)
    return q, k, v, None


def self_attention_forward(self, x, seq_lens, grid_sizes, freqs, block_mask, kv_cache=None, current_start=0,
                           current_end=0, causal_rope_cache=None):
    """Drop-in for CausalWanSelfAttention.forward on the kv-cache path (the training branch, which
    the streaming pipelines never take, is delegated to the original forward)."""
    if kv_cache is None:
        original = getattr(self, "_sdv2_original_forward", None)
        if original is None:
            raise RuntimeError("the kernel-backed self-attention serves the kv-cache path only")
        return original(x, seq_lens, grid_sizes, freqs, block_mask)
    q, k, v, norm = project_qkv(self, x)
    out = cached_attention(self, q, k, v, grid_sizes, freqs, kv_cache, current_start, norm=norm)
    return self.o(out.flatten(2))


def cross_attention_forward(self, x, context, context_lens, crossattn_cache=None):
    """Drop-in for WanT2VCrossAttention.forward: K/V of the text context are computed on the
    first call after `is_init` was cleared and read from the cache afterwards."""
    b, n, d = x.size(0), self.num_heads, self.head_dim
    q = _qk_norm(self.norm_q, self.q(x)).view(b, -1, n, d)
    if crossattn_cache is not None:
        if not crossattn_cache["is_init"]:
            crossattn_cache["is_init"] = True
            k = _qk_norm(self.norm_k, self.k(context)).view(b, -1, n, d)
            v = self.v(context).view(b, -1, n, d)
            crossattn_cache["k"] = k
            crossattn_cache["v"] = v
        else:
            k = crossattn_cache["k"]
            v = crossattn_cache["v"]
    else:
        k = self.norm_k(self.k(context)).view(b, -1, n, d)
        v = self.v(context).view(b, -1, n, d)
    if context_lens is not None:
        raise NotImplementedError("per-sample context lengths are not used on the streaming path")
    if q.dtype == torch.bfloat16:
        out = ops.cross_attn(q, k, v)
    else:
        out = ops.attn_kvcache_simt(q, k, v, [k.shape[1]] * b)
    return self.o(out.flatten(2))


def block_forward(self, x, e, seq_lens, grid_sizes, freqs, context, context_lens, block_mask, kv_cache=None,
                  crossattn_cache=None, current_start=0, current_end=0, causal_rope_cache=None):
    """Drop-in for CausalWanAttentionBlock.forward (models/wan/causal_model.py:432-483): same
    arguments, same arithmetic.  On bf16 CUDA tensors the two norm -> modulate chains and the two
    gated residual additions run as one launch each (they reproduce the op chain's bf16 roundings);
    otherwise the op chain itself runs.  x [B, L, C]; e [B, F, 6, C]."""
    frames = e.shape[1]
    per_frame = x.shape[1] // frames
    shift_a, scale_a, gate_a, shift_f, scale_f, gate_f = (self.modulation.unsqueeze(1) + e).chunk(6, dim=2)
    fused = _fusable(x) and shift_a.dtype == torch.bfloat16

    def norm_modulate(norm, y, scale, shift):
        if fused and getattr(norm, "weight", None) is None:
            return ops.ln_modulate(y, scale, shift, frames, norm.eps)
        return (norm(y).unflatten(1, (frames, per_frame)) * (1 + scale) + shift).flatten(1, 2)

    def add_gated(x, y, gate):
        if fused:
            return ops.gate_residual(x, y, gate, frames)
        return x + (y.unflatten(1, (frames, per_frame)) * gate).flatten(1, 2)

    y = self.self_attn(norm_modulate(self.norm1, x, scale_a, shift_a), seq_lens, grid_sizes, freqs, block_mask,
                       kv_cache, current_start, current_end, causal_rope_cache)
    # where a residual addition is followed by a LayerNorm of its result, both run as one launch
    if fused and ops.can_fuse_layernorm(x, self.norm3):
        x, xn = ops.residual_layernorm(x, y, gate_a, frames, self.norm3.eps, weight=self.norm3.weight,
                                       bias=self.norm3.bias)
    else:
        x = add_gated(x, y, gate_a)
        xn = self.norm3(x)
    c = self.cross_attn(xn, context, context_lens, crossattn_cache=crossattn_cache)
    if fused and getattr(self.norm2, "weight", None) is None and x.shape[-1] <= 5120:
        x, h = ops.residual_layernorm(x, c, None, frames, self.norm2.eps, scale=scale_f, shift=shift_f)
    else:
        x = x + c
        h = norm_modulate(self.norm2, x, scale_f, shift_f)
    y = ops.ffn(self.ffn, h) if fused else self.ffn(h)
    return add_gated(x, y, gate_f)


def watch_cache_manager(manager) -> None:
    """Make the reference's `KVCacheManager` (streamv2v/communication/kv_cache_manager.py:48-86)
    safe to use with the host-integer slot mirror: its `broadcast_kv_blocks` writes the index tensors
    of the moved blocks with collectives, which do not bump the tensors' version counters, so the
    mirror would keep the old integers (and, when the donor's rank is lower than the receiver's, no
    `+=` follows to reveal the change).  After this call every `broadcast_kv_blocks` ends by
    invalidating the mirrors of the blocks it moved.  Idempotent."""
    if getattr(manager, "_sdv2_watched", False):
        return
    original = manager.broadcast_kv_blocks

    def broadcast_kv_blocks(block_indices, donor_rank):
        try:
            return original(block_indices, donor_rank)
        finally:
            for bi in block_indices:
                RingState.invalidate(manager.pipeline.kv_cache1[bi])

    manager.broadcast_kv_blocks = broadcast_kv_blocks
    manager._sdv2_watched = True


def install(model, fuse_block: bool = True) -> int:
    """Bind the kernel-backed forwards onto every block of `model` (anything with a `.blocks`
    list whose items have `.self_attn` and `.cross_attn`, as the reference CausalWanModel has).
    Parameters, buffers and attribute names are left untouched, so checkpoints keep loading.
    With `fuse_block`, blocks that have the reference block's layout (norm1, norm2, norm3, ffn,
    modulation) also get `block_forward`, whose element-wise chains are single launches on bf16
    CUDA tensors.  Returns the number of blocks patched."""
    n = 0
    for block in model.blocks:
        sa, ca = block.self_attn, block.cross_attn
        takes_reference_args = "context_lens" in inspect.signature(
            getattr(block, "_sdv2_original_forward", block.forward)).parameters
        if (fuse_block and takes_reference_args
                and all(hasattr(block, a) for a in ("norm1", "norm2", "norm3", "ffn", "modulation"))):
            if not hasattr(block, "_sdv2_original_forward"):
                block._sdv2_original_forward = block.forward
            block.forward = types.MethodType(block_forward, block)
        if not hasattr(sa, "_sdv2_original_forward"):
            sa._sdv2_original_forward = sa.forward
        sa.forward = types.MethodType(self_attention_forward, sa)
        if not hasattr(sa, "evict_idx"):
            sa.evict_idx = None
        ca.forward = types.MethodType(cross_attention_forward, ca)
        n += 1
    return n

"""Tensor-level wrappers over the C ABI of libsdv2.so.

Every function takes CUDA tensors, launches on the current stream of the tensors' device and does
not synchronise.  There is no CPU or PyTorch fallback: a missing library or a failing call raises.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _native as N

_workspaces: Dict[int, torch.Tensor] = {}
_tables: Dict[Tuple[int, int, int], Tuple[torch.Tensor, torch.Tensor]] = {}


class LaunchLog:
    """Optional per-launch record for measurements: counts launches per entry point and, when
    `timed` is set, brackets each launch with CUDA events on the launching stream.  Off unless a
    caller installs one with `set_launch_log`."""

    def __init__(self, timed: bool = False):
        self.timed = timed
        self.counts: Dict[str, int] = {}
        self.events: Dict[str, list] = {}
        self.work: Dict[str, float] = {}

    def durations_ms(self, name: str):
        return [a.elapsed_time(b) for a, b in self.events.get(name, [])]


_log: Optional[LaunchLog] = None


def set_launch_log(log: Optional[LaunchLog]) -> None:
    global _log
    _log = log


def current_launch_log() -> Optional[LaunchLog]:
    return _log


class _Logged:
    __slots__ = ("name", "work", "ev")

    def __init__(self, name: str, work: float = 0.0):
        self.name, self.work, self.ev = name, work, None

    def __enter__(self):
        if _log is not None:
            _log.counts[self.name] = _log.counts.get(self.name, 0) + 1
            _log.work[self.name] = _log.work.get(self.name, 0.0) + self.work
            if _log.timed:
                self.ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                self.ev[0].record()
        return self

    def __exit__(self, *exc):
        if self.ev is not None:
            self.ev[1].record()
            _log.events.setdefault(self.name, []).append(self.ev)
        return False


def workspace(device: torch.device) -> torch.Tensor:
    """Per-device scratch for the attention kernels (status word first), zeroed on creation."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        nbytes = int(N.lib().sdv2_attn_workspace_bytes(N.MAX_ROWS, 1 << 20, 64, 128))
        ws = torch.zeros(nbytes + 256, dtype=torch.uint8, device=torch.device("cuda", idx))
        off = (-ws.data_ptr()) % 256
        ws = ws[off:off + nbytes]
        _workspaces[idx] = ws
    return ws


def rope_table_device(freqs: torch.Tensor, device: torch.device) -> torch.Tensor:
    """complex128 [rows, head_dim/2] table (the model's `freqs`) -> float64 [rows, head_dim/2, 2]
    on `device`, cached per source tensor."""
    key = (id(freqs), freqs.data_ptr(), device.index if device.index is not None else -1)
    hit = _tables.get(key)
    if hit is not None and hit[0] is freqs:
        return hit[1]
    if freqs.dtype != torch.complex128:
        raise ValueError("rope table must be complex128")
    t = torch.view_as_real(freqs.to(device)).contiguous()
    if len(_tables) > 16:
        _tables.clear()
    _tables[key] = (freqs, t)
    return t


def rope_kv_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, table: torch.Tensor, grid: Sequence[int],
                   start_frames: Sequence[int], dst_begin: Sequence[int], *,
                   q_out: Optional[torch.Tensor] = None,
                   index_tensors: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                   index_values: Optional[Tuple[Sequence[int], Sequence[int]]] = None,
                   step_params: Optional[torch.Tensor] = None,
                   norm: Optional[Tuple[torch.Tensor, torch.Tensor, float]] = None) -> torch.Tensor:
    """Rope q and k, write k/v of every row into cache slot [dst_begin[b], dst_begin[b]+N).
    q, k, v: [B, N, H, D]; caches [B, Smax, H, D]; table: float64 [rows, D/2, 2] on the device.
    Optionally stores index_values into the (global_end, local_end) int64 device tensors.
    With `step_params` (device int64 [4, B], contiguous: start frames | slots | global ends |
    local ends) the kernel reads those values from that tensor when it runs and the host-side
    start_frames / dst_begin / index_values arguments are ignored: the launch then carries nothing
    that changes from step to step and can be replayed from a CUDA graph.
    With `norm` = (weight_q, weight_k, eps), q and k are the raw projection outputs and are RMS
    normalised over the token row in the same launch (see `can_fuse_norm`); the result equals
    `rmsnorm` followed by this function bit for bit.
    Returns the roped q ([B, N, H, D], contiguous)."""
    B, n_new, H, D = q.shape
    if q_out is None:
        q_out = torch.empty((B, n_new, H, D), dtype=q.dtype, device=q.device)
    f, h, w = (int(x) for x in grid)
    ge_dev = le_dev = None
    ge_val = le_val = None
    if index_tensors is not None:
        g, l = index_tensors
        if g.dtype != torch.int64 or l.dtype != torch.int64 or g.numel() < B or l.numel() < B:
            raise ValueError("index tensors must be int64 with one entry per row")
        if not (g.is_contiguous() and l.is_contiguous()):
            raise ValueError("index tensors must be contiguous")
        ge_dev, le_dev = g.data_ptr(), l.data_ptr()
        if step_params is None:
            ge_val, le_val = N.i64_array(index_values[0]), N.i64_array(index_values[1])
    views = [N.view(t) for t in (q, k, v, q_out, k_cache, v_cache)]
    if step_params is not None and (step_params.dtype != torch.int64 or not step_params.is_contiguous()
                                    or step_params.numel() != 4 * B or step_params.device != q.device):
        raise ValueError("step_params must be a contiguous int64 [4, rows] tensor on the same device")
    if norm is not None:
        wq, wk, eps = norm
        if not can_fuse_norm(q, k, v, wq, wk):
            raise ValueError("this layout cannot take the fused norm: apply rmsnorm first")
        host = step_params is None
        # everything is marshalled before the (optionally timed) launch bracket opens
        args = [*[C.byref(x) for x in views], B, n_new, H, D, k_cache.shape[1], table.data_ptr(), table.shape[0],
                f, h, w, N.i64_array(start_frames) if host else None, N.i64_array(dst_begin) if host else None,
                None if host else step_params.data_ptr(), ge_dev, le_dev, ge_val, le_val,
                wq.data_ptr(), wk.data_ptr(), float(eps), workspace(q.device).data_ptr(), N.stream_ptr(q.device)]
        fn = N.lib().sdv2_norm_rope_kv_append
        with _Logged("rope_kv_append", 6.0 * B * n_new * H * D * q.element_size()):
            rc = fn(*args)
        N.check(rc, "sdv2_norm_rope_kv_append")
        return q_out
    if step_params is not None:
        if (step_params.dtype != torch.int64 or not step_params.is_contiguous() or step_params.numel() != 4 * B
                or step_params.device != q.device):
            raise ValueError("step_params must be a contiguous int64 [4, rows] tensor on the same device")
        args = [*[C.byref(x) for x in views], B, n_new, H, D, k_cache.shape[1], table.data_ptr(), table.shape[0],
                f, h, w, step_params.data_ptr(), ge_dev, le_dev, N.dtype_code(q.dtype),
                workspace(q.device).data_ptr(), N.stream_ptr(q.device)]
        fn = N.lib().sdv2_rope_kv_append_indirect
        with _Logged("rope_kv_append", 6.0 * B * n_new * H * D * q.element_size()):
            rc = fn(*args)
        N.check(rc, "sdv2_rope_kv_append_indirect")
        return q_out
    args = [*[C.byref(x) for x in views], B, n_new, H, D, k_cache.shape[1], table.data_ptr(), table.shape[0],
            f, h, w, N.i64_array(start_frames), N.i64_array(dst_begin), ge_dev, le_dev, ge_val, le_val,
            N.dtype_code(q.dtype), workspace(q.device).data_ptr(), N.stream_ptr(q.device)]
    fn = N.lib().sdv2_rope_kv_append
    with _Logged("rope_kv_append", 6.0 * B * n_new * H * D * q.element_size()):
        rc = fn(*args)
    N.check(rc, "sdv2_rope_kv_append")
    return q_out


_mean_scratch: Dict[Tuple[int, int], torch.Tensor] = {}


def frame_means(k_cache: torch.Tensor, v_cache: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                sink_frames: int, frame_tokens: int) -> torch.Tensor:
    """[rows, sink_frames + 1, 2, H * D] per-frame means (K, V) of the cache's sink frames and of the new
    frame (last entry), in the tensors' dtype, for the adaptive sink test."""
    rows, _, H, D = k_new.shape
    means = torch.empty((rows, sink_frames + 1, 2, H * D), dtype=k_new.dtype, device=k_new.device)
    need = int(N.lib().sdv2_frame_means_scratch_bytes(rows, sink_frames, H, D))
    idx = k_new.device.index if k_new.device.index is not None else torch.cuda.current_device()
    scratch = _mean_scratch.get((idx, need))
    if scratch is None:
        scratch = _mean_scratch[(idx, need)] = torch.empty(need, dtype=torch.uint8, device=k_new.device)
    views = [N.view(t) for t in (k_cache, v_cache, k_new, v_new)]
    with _Logged("frame_means", 2.0 * rows * (sink_frames + 1) * frame_tokens * H * D * k_new.element_size()):
        rc = N.lib().sdv2_frame_means(*[C.byref(x) for x in views], rows, sink_frames, frame_tokens, H, D,
                                      k_cache.shape[1], N.dtype_code(k_new.dtype), means.data_ptr(),
                                      scratch.data_ptr(), scratch.numel(), N.stream_ptr(k_new.device))
    N.check(rc, "sdv2_frame_means")
    return means


def ring_plan_adaptive(sim: Optional[torch.Tensor], threshold: float, queue: torch.Tensor, frame_tokens: int,
                       n_new: int, step_params: torch.Tensor, *, host_inputs: Optional[Sequence[Sequence[int]]] = None,
                       host_inputs_dev: Optional[torch.Tensor] = None) -> None:
    """One launch of the device-side slot logic for all rows of a layer (adaptive sink refresh).
    sim: [rows, sink_frames] similarities on the device (bf16 / fp32) or None; queue: int64
    [rows, 1 + cap] on the device, updated in place; host_inputs: 7 lists of `rows` ints (start frame,
    global end, local end, evict, pop, push value, append slot) or, for a launch that is recorded in a
    graph, the same as a device int64 [7, rows] tensor; step_params: device int64 [4, rows], written
    for `rope_kv_append(step_params=...)`."""
    rows = queue.shape[0]
    if queue.dtype != torch.int64 or not queue.is_contiguous() or step_params.dtype != torch.int64 \
            or not step_params.is_contiguous() or step_params.numel() != 4 * rows:
        raise ValueError("queue / step_params must be contiguous int64 tensors")
    sink = 0
    sim_ptr, code = None, 0
    if sim is not None:
        if sim.shape[0] != rows or not sim.is_contiguous():
            raise ValueError("sim must be a contiguous [rows, sink_frames] tensor")
        sink, sim_ptr, code = sim.shape[1], sim.data_ptr(), N.dtype_code(sim.dtype)
    hv = dev = None
    if host_inputs_dev is not None:
        if host_inputs_dev.dtype != torch.int64 or not host_inputs_dev.is_contiguous() \
                or host_inputs_dev.numel() != 7 * rows:
            raise ValueError("host_inputs_dev must be a contiguous int64 [7, rows] tensor")
        dev = host_inputs_dev.data_ptr()
    else:
        hv = N.i64_array([int(x) for lst in host_inputs for x in lst])
    with _Logged("ring_plan"):
        rc = N.lib().sdv2_ring_plan_adaptive(sim_ptr, code, rows, sink, float(threshold), queue.data_ptr(),
                                             queue.shape[1] - 1, int(frame_tokens), int(n_new), hv, dev,
                                             step_params.data_ptr(), workspace(queue.device).data_ptr(),
                                             N.stream_ptr(queue.device))
    N.check(rc, "sdv2_ring_plan_adaptive")


def can_fuse_norm(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, weight_q: torch.Tensor,
                  weight_k: torch.Tensor) -> bool:
    """Whether `rope_kv_append(norm=...)` serves these tensors: bf16 on CUDA, the heads of a token back
    to back (slices of a fused q|k|v projection qualify), a token row of at most 8192 elements that
    still fits the kernel's staging buffers, bf16 weights of the row's length."""
    B, n_new, H, D = q.shape
    dim = H * D
    if not (q.is_cuda and q.dtype == torch.bfloat16 and weight_q.dtype == torch.bfloat16
            and weight_k.dtype == torch.bfloat16 and weight_q.numel() == dim and weight_k.numel() == dim):
        return False
    if dim > 8192 or 3 * 3 * dim * 2 + 3 * (D // 2) * 16 > 200 * 1024:        # three stages of one token each
        return False
    return (all(t.stride(3) == 1 and t.stride(2) == D for t in (q, k, v))
            and weight_q.is_contiguous() and weight_k.is_contiguous()
            and weight_q.data_ptr() % 16 == 0 and weight_k.data_ptr() % 16 == 0)


def attn_kvcache(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_lens: Sequence[int], *,
                 out: Optional[torch.Tensor] = None, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """softmax(q k^T scale) v over cache[b, :seq_lens[b]] on the tensor cores (bf16)."""
    B, n_q, H, D = q.shape
    if q.dtype != torch.bfloat16:
        raise ValueError("the tensor-core attention kernel takes bf16; use attn_kvcache_simt for fp32")
    if out is None:
        out = torch.empty((B, n_q, H, D), dtype=q.dtype, device=q.device)
    ws = workspace(q.device)
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    views = [N.view(t) for t in (q, k_cache, v_cache, out)]
    args = [*[C.byref(x) for x in views], B, n_q, H, D, k_cache.shape[1], N.i32_array(seq_lens), scale, ws.data_ptr(),
            ws.numel(), N.stream_ptr(q.device)]
    fn = N.lib().sdv2_attn_kvcache
    with _Logged("attn_kvcache", 4.0 * n_q * D * H * float(sum(int(x) for x in seq_lens[:B]))):
        rc = fn(*args)
    N.check(rc, "sdv2_attn_kvcache")
    return out


def cross_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, out: Optional[torch.Tensor] = None,
               softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Every query attends all k.shape[1] context slots; k/v may be stride-0 expands over rows."""
    B, n_q, H, D = q.shape
    if q.dtype != torch.bfloat16:
        raise ValueError("the tensor-core attention kernel takes bf16")
    if out is None:
        out = torch.empty((B, n_q, H, D), dtype=q.dtype, device=q.device)
    ws = workspace(q.device)
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    views = [N.view(t) for t in (q, k, v, out)]
    args = [*[C.byref(x) for x in views], B, n_q, H, D, k.shape[1], scale, ws.data_ptr(), ws.numel(),
            N.stream_ptr(q.device)]
    fn = N.lib().sdv2_cross_attn
    with _Logged("cross_attn", 4.0 * B * n_q * D * H * k.shape[1]):
        rc = fn(*args)
    N.check(rc, "sdv2_cross_attn")
    return out


def attn_kvcache_simt(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_lens: Sequence[int], *,
                      out: Optional[torch.Tensor] = None, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Same contraction on CUDA cores in fp32 math; bf16 or fp32 tensors."""
    B, n_q, H, D = q.shape
    if out is None:
        out = torch.empty((B, n_q, H, D), dtype=q.dtype, device=q.device)
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    views = [N.view(t) for t in (q, k_cache, v_cache, out)]
    rc = N.lib().sdv2_attn_kvcache_simt(*[C.byref(x) for x in views], B, n_q, H, D, k_cache.shape[1],
                                        N.i32_array(seq_lens), scale, N.dtype_code(q.dtype),
                                        N.stream_ptr(q.device))
    N.check(rc, "sdv2_attn_kvcache_simt")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm over the last dimension of a bf16 tensor whose rows are contiguous runs of `dim`
    (rows themselves may be strided, e.g. a slice of a fused projection)."""
    dim = x.shape[-1]
    if x.stride(-1) != 1:
        x = x.contiguous()
    x2 = x.reshape(-1, dim) if x.is_contiguous() else x.flatten(0, -2)
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    with _Logged("rmsnorm", 2.0 * x.numel() * 2):
        rc = N.lib().sdv2_rmsnorm(x2.data_ptr(), x2.stride(0), weight.data_ptr(), out.data_ptr(), dim,
                                  x2.shape[0], dim, eps, N.stream_ptr(x.device))
    N.check(rc, "sdv2_rmsnorm")
    return out


def _mod_rows(t: torch.Tensor, B: int, frames: int, dim: int):
    """(pointer, row stride) of a [B, frames, (1,) dim] chunk of the modulation tensor, in place
    when rows are evenly spaced (a chunk of [B, frames, 6, dim] is), else through a copy."""
    t = t.reshape(B, frames, dim) if t.is_contiguous() else t.squeeze(2) if t.dim() == 4 else t
    if t.stride(-1) == 1 and (B == 1 or t.stride(0) == frames * t.stride(1)) and t.stride(1) % 8 == 0:
        return t, t.stride(1)
    t = t.contiguous()
    return t, dim


def ln_modulate(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, frames: int, eps: float) -> torch.Tensor:
    """bf16(bf16(bf16(LN(x)) * bf16(1 + scale)) + shift) with per-frame scale / shift
    [B, frames, (1,) dim], read in place from the modulation tensor."""
    B, L, dim = x.shape
    x = x.contiguous()
    out = torch.empty_like(x)
    sc, stride = _mod_rows(scale, B, frames, dim)
    sh, stride2 = _mod_rows(shift, B, frames, dim)
    if stride2 != stride:
        sc, sh, stride = sc.contiguous(), sh.contiguous(), dim
    with _Logged("ln_modulate", 2.0 * x.numel() * 2):
        rc = N.lib().sdv2_ln_modulate(x.data_ptr(), sc.data_ptr(), sh.data_ptr(), stride, out.data_ptr(), B, frames,
                                      L // frames, dim, eps, N.stream_ptr(x.device))
    N.check(rc, "sdv2_ln_modulate")
    return out


def layernorm_affine(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """torch.nn.LayerNorm with weight and bias over the last dimension of a bf16 tensor, one launch."""
    dim = x.shape[-1]
    x = x.contiguous()
    out = torch.empty_like(x)
    with _Logged("layernorm_affine", 2.0 * x.numel() * 2):
        rc = N.lib().sdv2_layernorm_affine(x.data_ptr(), weight.data_ptr(), bias.data_ptr(), out.data_ptr(),
                                           x.numel() // dim, dim, eps, N.stream_ptr(x.device))
    N.check(rc, "sdv2_layernorm_affine")
    return out


def residual_layernorm(x: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor], frames: int, eps: float, *,
                       weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                       scale: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None):
    """(x_new, normed): x_new = gate_residual(x, y, gate) (gate None: x + y), normed = layernorm_affine(x_new,
    weight, bias) when weight / bias are given, else ln_modulate(x_new, scale, shift) - one launch, the same
    values as the separate calls.  x [B, L, dim] with L a multiple of frames; dim at most 5120."""
    B, L, dim = x.shape
    x, y = x.contiguous(), y.contiguous()
    x_new, out = torch.empty_like(x), torch.empty_like(x)
    gt, gstride = (None, 0) if gate is None else _mod_rows(gate, B, frames, dim)
    affine = weight is not None
    if affine:
        mul, add, stride = weight, bias, 0
    else:
        mul, stride = _mod_rows(scale, B, frames, dim)
        add, stride2 = _mod_rows(shift, B, frames, dim)
        if stride2 != stride:
            mul, add, stride = mul.contiguous(), add.contiguous(), dim
    with _Logged("residual_layernorm", 4.0 * x.numel() * 2):
        rc = N.lib().sdv2_residual_layernorm(x.data_ptr(), y.data_ptr(), None if gt is None else gt.data_ptr(), gstride,
                                             x_new.data_ptr(), 1 if affine else 0, mul.data_ptr(), add.data_ptr(),
                                             stride, out.data_ptr(), B, frames, L // frames, dim, eps,
                                             N.stream_ptr(x.device))
    N.check(rc, "sdv2_residual_layernorm")
    return x_new, out


def gelu_tanh_(x: torch.Tensor) -> torch.Tensor:
    """tanh-approximated GELU of a contiguous bf16 tensor, in place."""
    with _Logged("gelu_tanh", 2.0 * x.numel() * 2):
        rc = N.lib().sdv2_gelu_tanh(x.data_ptr(), x.data_ptr(), x.numel(), N.stream_ptr(x.device))
    N.check(rc, "sdv2_gelu_tanh")
    return x


def ffn(seq, h: torch.Tensor) -> torch.Tensor:
    """`seq(h)` for the block's FFN.  Linear -> GELU(tanh) -> Linear on a bf16 CUDA tensor runs the activation
    with `gelu_tanh_` in place on the first projection's output; anything else runs the module as it is."""
    if (h.is_cuda and h.dtype == torch.bfloat16 and isinstance(seq, torch.nn.Sequential) and len(seq) == 3
            and isinstance(seq[1], torch.nn.GELU) and getattr(seq[1], "approximate", "none") == "tanh"
            and isinstance(seq[0], torch.nn.Linear) and not torch.is_grad_enabled()):
        u = seq[0](h)
        if u.dtype == torch.bfloat16 and u.is_contiguous() and u.numel() % 8 == 0:
            return seq[2](gelu_tanh_(u))
        return seq[2](seq[1](u))
    return seq(h)


def can_fuse_layernorm(x: torch.Tensor, norm) -> bool:
    """Whether `norm` (an affine LayerNorm over the last dimension) applied to `x` can run as
    `layernorm_affine`."""
    w, b = getattr(norm, "weight", None), getattr(norm, "bias", None)
    return (w is not None and b is not None and x.is_cuda and x.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and w.is_contiguous() and b.is_contiguous()
            and x.shape[-1] % 8 == 0 and x.shape[-1] <= 5120 and tuple(getattr(norm, "normalized_shape", ())) ==
            (x.shape[-1],))


def gate_residual(x: torch.Tensor, y: torch.Tensor, gate: torch.Tensor, frames: int) -> torch.Tensor:
    """bf16(x + bf16(y * gate)) with per-frame gate [B, frames, (1,) dim] read in place."""
    B, L, dim = x.shape
    x, y = x.contiguous(), y.contiguous()
    out = torch.empty_like(x)
    gt, stride = _mod_rows(gate, B, frames, dim)
    with _Logged("gate_residual", 3.0 * x.numel() * 2):
        rc = N.lib().sdv2_gate_residual(x.data_ptr(), y.data_ptr(), gt.data_ptr(), stride, out.data_ptr(), B, frames,
                                        L // frames, dim, N.stream_ptr(x.device))
    N.check(rc, "sdv2_gate_residual")
    return out


def read_status(device: torch.device) -> None:
    """Synchronise the current stream and raise if a device-side wait ran out since the last call."""
    ws = workspace(device)
    detail = C.c_int(0)
    rc = N.lib().sdv2_read_status(ws.data_ptr(), C.byref(detail), N.stream_ptr(device))
    if rc == N.ERR_TIMEOUT:
        raise N.NativeError(rc, "attention kernel", f"device-side wait timed out at site {detail.value & 0xFF} "
                                                    f"(block {detail.value >> 8})")
    if rc == N.ERR_INVALID_ARG and detail.value:
        raise N.NativeError(rc, "rope_kv_append", "device-resident slot parameters were out of range; "
                                                  "that launch wrote nothing")
    N.check(rc, "sdv2_read_status")


class _StatusPoll:
    """Asynchronous watch on a device's status word: a 4-byte copy to pinned host memory rides the
    launching stream, and its result is looked at by a later poll once the copy's event has
    completed.  Never blocks the host; a raised status is seen one or two polls late."""

    def __init__(self, device: torch.device):
        self.device = device
        self.word = workspace(device)[:4].view(torch.int32)
        self.pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event: Optional[torch.cuda.Event] = None

    def poll(self) -> None:
        if self.event is not None:
            if not self.event.query():
                return
            self.event = None
            seen = int(self.pinned[0])
            if seen != 0:
                read_status(self.device)        # synchronises, decodes, clears and raises
                raise N.NativeError(N.ERR_TIMEOUT, "device status",
                                    f"a kernel reported status {seen:#x} earlier; its outputs are not valid")
        self.pinned.copy_(self.word, non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record()


_polls: Dict[int, _StatusPoll] = {}


def poll_status(device: torch.device) -> None:
    """Cheap, non-blocking check that no kernel of this library gave up a bounded wait or refused
    device-resident parameters since the last check; raises NativeError if one did (its launch
    wrote nothing, so everything computed from its outputs is garbage).  Called by the attention
    forwards every few dozen launches and after every graph replay; not during stream capture."""
    device = torch.device(device)
    if device.type != "cuda" or torch.cuda.is_current_stream_capturing():
        return
    idx = device.index if device.index is not None else torch.cuda.current_device()
    p = _polls.get(idx)
    if p is None:
        p = _polls[idx] = _StatusPoll(torch.device("cuda", idx))
    p.poll()


def selftest_wait_timeout(device: torch.device, budget_cycles: int = 2_000_000) -> None:
    """Launch the self-test block whose wait nobody satisfies, into this device's status word.  The
    next `read_status` / `poll_status` then reports a timeout at the probe site (7)."""
    ws = workspace(device)
    rc = N.lib().sdv2_selftest_wait_timeout(ws.data_ptr(), int(budget_cycles), N.stream_ptr(device))
    N.check(rc, "sdv2_selftest_wait_timeout")


def attn_partial_slots(rows: int, q_tokens: int, heads: int, min_seq_len: int, sm_count: int) -> int:
    """Scratch slots the attention launch for this problem uses on a device with `sm_count` SMs."""
    return int(N.lib().sdv2_attn_partial_slots(rows, q_tokens, heads, min_seq_len, sm_count))


def selftest_umma(a: torch.Tensor, b: torch.Tensor, p: torch.Tensor, v: torch.Tensor):
    """(a @ b^T, p @ v) for 128x128 bf16 matrices through the two tensor-core code paths."""
    dev = a.device
    s_out = torch.full((128, 128), float("nan"), dtype=torch.float32, device=dev)
    o_out = torch.full((128, 128), float("nan"), dtype=torch.float32, device=dev)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    ts = [t.contiguous() for t in (a, b, p, v)]
    rc = N.lib().sdv2_selftest_umma(*[t.data_ptr() for t in ts], s_out.data_ptr(), o_out.data_ptr(),
                                    status.data_ptr(), N.stream_ptr(dev))
    N.check(rc, "sdv2_selftest_umma")
    torch.cuda.synchronize(dev)
    st = int(status[0].item())
    if st != 0:
        raise N.NativeError(N.ERR_TIMEOUT, "sdv2_selftest_umma", f"device-side wait timed out at site {st & 0xFF}")
    return s_out, o_out

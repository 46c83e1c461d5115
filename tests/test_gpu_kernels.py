"""Parity of the CUDA path (through the C ABI) with the oracle and the reference fixtures."""
import math

import numpy as np
import pytest
import torch

import cases
from oracle import causal_attention_oracle as orc
from replay import replay_cuda, replay_oracle

pytestmark = pytest.mark.gpu

# attention output tolerance in bf16 with fp32 accumulation (max-abs, mean-abs)
TOL_MAX, TOL_MEAN = 2e-2, 1e-3


def assert_close_bf16(out, ref, what=""):
    """|out - ref| <= 2e-2 everywhere and <= 1e-3 on average.  An output that is one bf16 step
    away from the reference is still accepted where that step itself exceeds 2e-2 (|ref| >= 4:
    the spacing of bf16 there is 2^-5 or more), since both sides round to bf16 at the end."""
    out, ref = out.float().cpu(), ref.float().cpu()
    err = (out - ref).abs()
    allowed = torch.maximum(torch.full_like(ref, TOL_MAX), ref.abs() * 2.0 ** -7)
    worst = (err - allowed).max().item()
    assert worst <= 0, (what, "max-abs", err.max().item())
    assert err.mean().item() <= TOL_MEAN, (what, "mean-abs", err.mean().item())


def _ops():
    from streamdiffusionv2_b200 import ops
    return ops


def test_library_loads_on_gpu():
    from streamdiffusionv2_b200 import _native
    assert _native.lib().sdv2_abi_version() == 1


def test_umma_selftest_contractions():
    """The two tensor-core contractions in isolation: Q K^T (both operands K-major from shared
    memory) and P V (P from tensor memory, V MN-major)."""
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    a, b, p, v = (torch.randn(128, 128, generator=g).to(torch.bfloat16).cuda() for _ in range(4))
    s, o = ops.selftest_umma(a, b, p, v)
    s_ref = a.float() @ b.float().t()
    o_ref = p.float() @ v.float()
    assert torch.isfinite(s).all() and torch.isfinite(o).all()
    assert (s - s_ref).abs().max().item() < 1e-3 * 128, "Q K^T contraction wrong"
    assert (o - o_ref).abs().max().item() < 1e-3 * 128, "P V contraction wrong"


@pytest.mark.parametrize("name", sorted(cases.KERNEL_CASES))
def test_cuda_path_matches_reference_fixture(name):
    """Cache bytes, index tensors, evict queues and step counter bit-exact after every call;
    attention output within tolerance of the reference's output."""
    case = cases.KERNEL_CASES[name]
    meta, z = cases.load_fixture(name)
    ops = _ops()
    n = 0
    for i, out, kv, mod in replay_cuda(case):
        g = meta["steps"][i]
        assert kv["global_end_index"].tolist() == g["global_end"], (name, i)
        assert kv["local_end_index"].tolist() == g["local_end"], (name, i)
        assert mod.evict_idx == g["evict_idx"], (name, i)
        assert kv["current_step"] == g["current_step"], (name, i)
        assert cases.sha(kv["k"]) == g["k_sha"], f"K cache differs at call {i}"
        assert cases.sha(kv["v"]) == g["v_sha"], f"V cache differs at call {i}"
        ref = cases.from_numpy_bits(z[f"out_{i}"], g["out_dtype"]).float()
        assert_close_bf16(out, ref, (name, i))
        n += 1
    assert n == len(meta["steps"])
    ops.read_status(torch.device("cuda"))


def _rand_case(B, N, H, S, seed, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, N, H, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, H, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, H, 128, generator=g).to(torch.bfloat16)
    return q, k, v


@pytest.mark.parametrize("B,N,H,S,lens", [
    (1, 128, 1, 128, [128]),
    (1, 256, 1, 256, [256]),
    (1, 100, 2, 300, [300]),           # ragged q tile and kv tail
    (2, 300, 3, 1000, [1000, 517]),    # per-row lengths, odd tile counts
    (2, 48, 2, 2000, [1, 1999]),       # a single key; long with tail
    (1, 3120, 2, 4680, [4680]),        # production chunk size, short cache
])
def test_attention_vs_oracle(B, N, H, S, lens):
    ops = _ops()
    q, k, v = _rand_case(B, N, H, S, seed=N + S)
    out = ops.attn_kvcache(q.cuda(), k.cuda(), v.cuda(), lens)
    ref = orc.attend_explicit(q, k, v, lens, dtype=torch.float32)
    err = (out.float().cpu() - ref).abs()
    assert torch.isfinite(out).all()
    assert err.max().item() <= TOL_MAX and err.mean().item() <= TOL_MEAN, err.max().item()
    simt = ops.attn_kvcache_simt(q.cuda(), k.cuda(), v.cuda(), lens)
    err2 = (simt.float().cpu() - ref).abs()
    assert err2.max().item() <= TOL_MAX and err2.mean().item() <= TOL_MEAN
    ops.read_status(torch.device("cuda"))


def test_attention_large_logits_rescale_path():
    """Row maxima that keep growing along the cache force the lazy accumulator rescale."""
    ops = _ops()
    B, N, H, S = 1, 128, 1, 1024
    q, k, v = _rand_case(B, N, H, S, seed=3)
    ramp = torch.linspace(0.2, 3.0, S).view(1, S, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    q = (q.float() * 2).to(torch.bfloat16)
    out = ops.attn_kvcache(q.cuda(), k.cuda(), v.cuda(), [S])
    ref = orc.attend_explicit(q, k, v, [S], dtype=torch.float32)
    err = (out.float().cpu() - ref).abs()
    assert err.max().item() <= 4e-2 and err.mean().item() <= 2e-3, err.max().item()


def test_attention_strided_views():
    """q/k/v as slices of a fused projection and caches as slices of a larger buffer."""
    ops = _ops()
    B, N, H, S = 2, 200, 2, 700
    g = torch.Generator().manual_seed(21)
    qkv = torch.randn(B, N, 3, H, 128, generator=g).to(torch.bfloat16).cuda()
    kc = torch.randn(B, S + 100, H, 128, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(B, S + 100, H, 128, generator=g).to(torch.bfloat16).cuda()
    q = qkv[:, :, 0]
    out = ops.attn_kvcache(q, kc[:, :S], vc[:, :S], [S, S - 33])
    ref = orc.attend_explicit(q.cpu(), kc[:, :S].cpu(), vc[:, :S].cpu(), [S, S - 33], dtype=torch.float32)
    err = (out.float().cpu() - ref).abs()
    assert err.max().item() <= TOL_MAX and err.mean().item() <= TOL_MEAN


@pytest.mark.parametrize("name", sorted(cases.CROSS_CASES))
def test_cross_attention_fixture(name):
    ops = _ops()
    case = cases.CROSS_CASES[name]
    meta, z = cases.load_fixture(name)
    dtype = cases.DTYPES[case["dtype"]]
    g = torch.Generator().manual_seed(case["seed"])
    H, D = case["heads"], case["head_dim"]
    q = torch.randn(case["rows"], case["n"], H, D, generator=g).to(dtype)
    k1 = torch.randn(1, case["lk"], H, D, generator=g).to(dtype)
    v1 = torch.randn(1, case["lk"], H, D, generator=g).to(dtype)
    assert cases.sha(q) == meta["in_sha"]
    k = k1.cuda().expand(case["rows"], -1, -1, -1)   # stride-0 rows, as the pipeline stores them
    v = v1.cuda().expand(case["rows"], -1, -1, -1)
    if dtype == torch.bfloat16:
        out = ops.cross_attn(q.cuda(), k, v)
    else:
        out = ops.attn_kvcache_simt(q.cuda(), k, v, [case["lk"]] * case["rows"])
    ref = cases.from_numpy_bits(z["out"], meta["out_dtype"]).float()
    err = (out.float().cpu() - ref).abs()
    assert err.max().item() <= TOL_MAX and err.mean().item() <= TOL_MEAN


def test_rope_append_full_size_bitexact():
    """One production-size call (2 rows x 3120 tokens x 12 heads, 21-frame cache): the written
    slots equal the oracle's rope bit for bit, everything else in the cache stays untouched, and
    the roped queries match too."""
    ops = _ops()
    B, N, H, D, S = 2, 3120, 12, 128, 32760
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(B, N, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    table = orc.rope_table(D)
    starts = [17 * 1560, 40 * 1560]
    dst = [3120, 28080]
    kc = torch.full((B, S, H, D), 7.0, dtype=torch.bfloat16, device="cuda")
    vc = torch.full((B, S, H, D), -3.0, dtype=torch.bfloat16, device="cuda")
    ge = torch.zeros(B, dtype=torch.long, device="cuda")
    le = torch.zeros(B, dtype=torch.long, device="cuda")
    tdev = ops.rope_table_device(table, torch.device("cuda"))
    rq = ops.rope_kv_append(q.cuda(), k.cuda(), v.cuda(), kc, vc, tdev, (2, 30, 52), [s // 1560 for s in starts], dst,
                            index_tensors=(ge, le), index_values=([11, 22], [33, 44]))
    rq_ref = orc.rope_apply(q, (2, 30, 52), table, [s // 1560 for s in starts])
    rk_ref = orc.rope_apply(k, (2, 30, 52), table, [s // 1560 for s in starts])
    assert torch.equal(rq.cpu().view(torch.int16), rq_ref.view(torch.int16))
    kc_c, vc_c = kc.cpu(), vc.cpu()
    for b in range(B):
        assert torch.equal(kc_c[b, dst[b]:dst[b] + N].view(torch.int16), rk_ref[b].view(torch.int16))
        assert torch.equal(vc_c[b, dst[b]:dst[b] + N].view(torch.int16), v[b].view(torch.int16))
        mask = torch.ones(S, dtype=torch.bool)
        mask[dst[b]:dst[b] + N] = False
        assert (kc_c[b, mask] == 7.0).all() and (vc_c[b, mask] == -3.0).all()
    assert ge.tolist() == [11, 22] and le.tolist() == [33, 44]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope_append_padded_heads_take_the_direct_kernel(dtype):
    """Heads that are not back to back in memory (a slice of a wider last dimension) cannot be
    staged as whole token rows; the per-vector kernel serves them, with the same bits."""
    ops = _ops()
    B, N, H, D, S = 2, 24, 3, 128, 60
    g = torch.Generator().manual_seed(4)
    wide = [torch.randn(B, N, H, 2 * D, generator=g).to(dtype) for _ in range(3)]
    q, k, v = (w[..., :D] for w in wide)
    table = orc.rope_table(D)
    kc = torch.zeros(B, S, H, D, dtype=dtype, device="cuda")
    vc = torch.zeros(B, S, H, D, dtype=dtype, device="cuda")
    tdev = ops.rope_table_device(table, torch.device("cuda"))
    rq = ops.rope_kv_append(*(w.cuda()[..., :D] for w in wide), kc, vc, tdev, (2, 3, 4), [5, 900], [0, 36])
    rq_ref = orc.rope_apply(q.contiguous(), (2, 3, 4), table, [5, 900])
    rk_ref = orc.rope_apply(k.contiguous(), (2, 3, 4), table, [5, 900])
    assert cases.sha(rq) == cases.sha(rq_ref)
    assert cases.sha(kc[0, :N]) == cases.sha(rk_ref[0]) and cases.sha(kc[1, 36:]) == cases.sha(rk_ref[1])
    assert cases.sha(vc[1, 36:]) == cases.sha(v[1].contiguous())


def test_rope_append_special_values_bitexact():
    """Zeros, subnormals, infinities and NaNs in q/k go through the hardware conversion path and
    still match the oracle bit for bit (NaN payloads excepted: compared as NaN)."""
    ops = _ops()
    B, N, H, D, S = 1, 12, 2, 128, 12
    g = torch.Generator().manual_seed(6)
    q, k, v = (torch.randn(B, N, H, D, generator=g) for _ in range(3))
    for t in (q, k):
        flat = t.view(-1)
        flat[0::7] = 0.0
        flat[1::11] = -0.0
        flat[2::13] = 1e-39           # subnormal in bf16 and fp32
        flat[3::17] = float("inf")
        flat[4::19] = float("nan")
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    table = orc.rope_table(D)
    kc = torch.zeros(B, S, H, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    rq = ops.rope_kv_append(q.cuda(), k.cuda(), v.cuda(), kc, vc, ops.rope_table_device(table, torch.device("cuda")),
                            (2, 2, 3), [3], [0]).cpu()
    rq_ref = orc.rope_apply(q, (2, 2, 3), table, [3])
    rk_ref = orc.rope_apply(k, (2, 2, 3), table, [3])
    for got, ref in ((rq, rq_ref), (kc.cpu(), rk_ref)):
        nan = torch.isnan(ref)
        assert torch.equal(torch.isnan(got), nan)
        assert torch.equal(got.view(torch.int16)[~nan], ref.view(torch.int16)[~nan])


def test_rope_append_rejects_bad_slots():
    from streamdiffusionv2_b200 import _native
    ops = _ops()
    q = torch.zeros(1, 12, 1, 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(1, 24, 1, 128, dtype=torch.bfloat16, device="cuda")
    t = ops.rope_table_device(orc.rope_table(128), torch.device("cuda"))
    with pytest.raises(_native.NativeError):
        ops.rope_kv_append(q, q, q, kc, kc.clone(), t, (2, 2, 3), [0], [13])       # slot runs past the cache
    with pytest.raises(_native.NativeError):
        ops.rope_kv_append(q, q, q, kc, kc.clone(), t, (2, 2, 3), [1023], [0])     # frame index past the table
    with pytest.raises(_native.NativeError):
        ops.rope_kv_append(q, q, q, kc, kc.clone(), t, (2, 2, 2), [0], [0])        # grid does not match tokens


def test_attention_full_size_tensor_core_vs_cuda_core():
    """Production shape (3120 queries x 32760 keys x 12 heads): tensor-core kernel against the
    CUDA-core kernel on the device, and both against the oracle on a sample of query rows."""
    ops = _ops()
    B, N, H, S = 1, 3120, 12, 32760
    q, k, v = _rand_case(B, N, H, S, seed=1)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    out = ops.attn_kvcache(qd, kd, vd, [S])
    simt = ops.attn_kvcache_simt(qd, kd, vd, [S])
    ops.read_status(torch.device("cuda"))
    err = (out.float() - simt.float()).abs()
    assert err.max().item() <= TOL_MAX and err.mean().item() <= TOL_MEAN, err.max().item()
    rows = [0, 1, 127, 128, 1559, 3071, 3072, 3119]
    ref = orc.attend_explicit(q[:, rows], k, v, [S], dtype=torch.float32)
    e2 = (out[:, rows].float().cpu() - ref).abs()
    assert e2.max().item() <= TOL_MAX and e2.mean().item() <= TOL_MEAN


def test_fused_block_elementwise_match_their_op_chains():
    """rmsnorm / ln_modulate / gate_residual against the PyTorch op chains they replace, on the
    GPU in bf16: identical up to isolated single-bf16-step differences (reduction order)."""
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    B, F, fs, dim = 2, 2, 1560, 1536
    L = F * fs
    x = (torch.randn(B, L, dim, generator=g) * 2).to(torch.bfloat16).cuda()
    y = torch.randn(B, L, dim, generator=g).to(torch.bfloat16).cuda()
    w = (1 + 0.1 * torch.randn(dim, generator=g)).to(torch.bfloat16).cuda()
    mod = (0.3 * torch.randn(B, F, 3, dim, generator=g)).to(torch.bfloat16).cuda()
    scale, shift, gate = mod.chunk(3, dim=2)

    def close(a, b, what, scale_ref=None):
        # two chained bf16 roundings: a last-bit difference in the statistics can move the result
        # by up to two bf16 steps (of the largest intermediate) on isolated elements; almost all
        # elements are identical
        d = (a.float() - b.float()).abs()
        mag = b.float().abs() if scale_ref is None else torch.maximum(b.float().abs(), scale_ref.float().abs())
        step = mag.clamp_min(2.0 ** -120) * 2.0 ** -6
        assert (d <= step).all(), (what, d.max().item())
        assert (a == b).float().mean().item() > 0.995, what

    xf = x.float()
    want = (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + 1e-6)).type_as(x) * w
    close(ops.rmsnorm(x, w, 1e-6), want, 'rmsnorm')
    # a strided slice of a wider projection
    wide = torch.randn(B, L, 3 * dim, generator=g).to(torch.bfloat16).cuda()
    sl = wide[..., dim:2 * dim]
    sf = sl.float()
    close(ops.rmsnorm(sl, w, 1e-6), (sf * torch.rsqrt(sf.pow(2).mean(dim=-1, keepdim=True) + 1e-6)).type_as(sl) * w,
          'rmsnorm strided')

    ln = torch.nn.functional.layer_norm(x, (dim,), eps=1e-6)
    want = (ln.unflatten(1, (F, fs)) * (1 + scale) + shift).flatten(1, 2)
    close(ops.ln_modulate(x, scale, shift, F, 1e-6), want, 'ln_modulate',
          scale_ref=(ln.unflatten(1, (F, fs)) * (1 + scale)).flatten(1, 2))

    want = x + (y.unflatten(1, (F, fs)) * gate).flatten(1, 2)
    got = ops.gate_residual(x, y, gate, F)
    assert torch.equal(got, want)

    # norm3: LayerNorm with weight and bias, at the 1.3B and the 14B row length
    for d in (dim, 5120, 264):
        xd = (torch.randn(3, 777, d, generator=g) * 3 + 0.5).to(torch.bfloat16).cuda()
        norm = torch.nn.LayerNorm(d, eps=1e-6).cuda().to(torch.bfloat16)
        with torch.no_grad():
            norm.weight.copy_(1 + 0.2 * torch.randn(d, generator=g))
            norm.bias.copy_(0.3 * torch.randn(d, generator=g))
            assert ops.can_fuse_layernorm(xd, norm)
            # where weight * normalised and bias cancel, the step is that of the bias, not of the small sum
            close(ops.layernorm_affine(xd, norm.weight, norm.bias, norm.eps), norm(xd), f'layernorm_affine {d}',
                  scale_ref=norm.bias.expand_as(xd))
    assert not ops.can_fuse_layernorm(xd.float(), norm)

    # tanh GELU as x * sigmoid(2u): the op chain's values except isolated single-step differences
    u = (torch.randn(4, 1000, 8960, generator=g) * 2.5).to(torch.bfloat16).cuda()
    want = torch.nn.functional.gelu(u, approximate="tanh")
    got = ops.gelu_tanh_(u.clone())
    # for x > -2.9 the op chain's values (isolated single-step differences); below that the chain's own
    # 1 + tanh(u) cancels (its results are off by up to 3e-7, whole bf16 steps of values that small) and
    # this form stays exact: compare both with the function in float64
    mild = u.float() > -2.9
    close(torch.where(mild, got, want), want, 'gelu_tanh')
    assert (got == want)[mild].float().mean().item() > 0.999
    assert ((got.float() - want.float()).abs() <= want.float().abs() * 2.0 ** -7 + 4e-7).all()   # one bf16 step, or the chain's fp32 error
    ud = u.double()
    exact = (0.5 * ud * (1 + torch.tanh(0.7978845608028654 * (ud + 0.044715 * ud ** 3)))).to(torch.bfloat16)
    assert (got != exact).float().mean().item() < 0.01
    assert (got != exact).float().mean().item() <= (want != exact).float().mean().item()
    lin = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(approximate="tanh"),
                              torch.nn.Linear(256, 64)).cuda().to(torch.bfloat16)
    hh = torch.randn(2, 24, 64, generator=g).to(torch.bfloat16).cuda()
    with torch.no_grad():
        close(ops.ffn(lin, hh), lin(hh), 'ffn', scale_ref=torch.ones_like(hh))

    # a residual addition and the LayerNorm of its result in one launch: the values of the separate launches
    norm = torch.nn.LayerNorm(dim, eps=1e-6).cuda().to(torch.bfloat16)
    with torch.no_grad():
        norm.weight.copy_(1 + 0.2 * torch.randn(dim, generator=g))
        norm.bias.copy_(0.3 * torch.randn(dim, generator=g))
        x_sep = ops.gate_residual(x, y, gate, F)
        x_new, normed = ops.residual_layernorm(x, y, gate, F, 1e-6, weight=norm.weight, bias=norm.bias)
        assert torch.equal(x_new, x_sep)
        assert torch.equal(normed, ops.layernorm_affine(x_sep, norm.weight, norm.bias, 1e-6))
        x_new, normed = ops.residual_layernorm(x, y, None, F, 1e-6, scale=scale, shift=shift)
        assert torch.equal(x_new, x + y)
        assert torch.equal(normed, ops.ln_modulate(x + y, scale, shift, F, 1e-6))


def test_block_forward_with_reference_arguments_equals_the_block_it_replaces():
    """`install()` binds `block_forward` (the reference block's argument list) onto reference blocks.
    Here it runs on one of this package's blocks, on CUDA bf16 so that the fused launches are taken,
    against that block's own forward on the same inputs and cache state."""
    import copy
    import types

    from streamdiffusionv2_b200 import causal_attention as CA
    from streamdiffusionv2_b200.wan_model import DiTBlock, build_rope_table
    torch.manual_seed(3)
    dim, heads, fs, frames, rows = 256, 2, 6, 2, 2
    blk = DiTBlock(dim, 512, heads, qk_norm=True, cross_attn_norm=True).cuda().to(torch.bfloat16).eval()
    blk.self_attn.sink_size, blk.self_attn.adapt_sink_thr = 1, -1
    x = torch.randn(rows, frames * fs, dim).cuda().bfloat16()
    e = torch.randn(rows, frames, 6, dim).cuda().bfloat16()
    ctx = torch.randn(rows, 512, dim).cuda().bfloat16()
    freqs = build_rope_table(128)
    grid = torch.tensor([[frames, 2, 3]] * rows)

    def caches():
        kv = {"k": torch.zeros(rows, 8 * fs, heads, 128, device="cuda", dtype=torch.bfloat16),
              "v": torch.zeros(rows, 8 * fs, heads, 128, device="cuda", dtype=torch.bfloat16),
              "global_end_index": torch.zeros(rows, dtype=torch.long, device="cuda"),
              "local_end_index": torch.zeros(rows, dtype=torch.long, device="cuda"), "total_steps": 2, "current_step": 2}
        return kv, {"k": None, "v": None, "is_init": False}

    outs = []
    with torch.no_grad():
        for use_adapter in (False, True):
            b2 = copy.deepcopy(blk)
            b2.self_attn.evict_idx = None
            kv, cc = caches()
            starts = CA.HostStarts(torch.zeros(rows, dtype=torch.long, device="cuda"), [0] * rows)
            if use_adapter:
                fwd = types.MethodType(CA.block_forward, b2)
                outs.append((fwd(x, e, None, grid, freqs, ctx, None, None, kv, cc, starts, None), kv))
            else:
                outs.append((b2(x, e, grid, freqs, ctx, kv, cc, starts), kv))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1]["k"], outs[1][1]["k"]) and torch.equal(outs[0][1]["v"], outs[1][1]["v"])


def test_attention_ignores_whatever_lies_past_the_valid_length():
    """Cache rows at and beyond seq_len may hold anything (an uninitialised cache, NaN): they are
    never attended, and a NaN there must not leak into the output through 0 x NaN in P V.  One
    tile, two tiles with a ragged second one, and a split long row."""
    ops = _ops()
    for B, N, H, S, lens in [(1, 128, 1, 128, [77]), (2, 200, 2, 384, [130, 255]), (1, 300, 2, 4096, [3000])]:
        q, k, v = _rand_case(B, N, H, S, seed=S + N)
        kd, vd = k.cuda(), v.cuda()
        for b, L in enumerate(lens):
            kd[b, L:] = float("nan")
            vd[b, L:] = float("nan")
        out = ops.attn_kvcache(q.cuda(), kd, vd, lens)
        assert torch.isfinite(out).all(), (B, N, S)
        ref = orc.attend_explicit(q, k, v, lens, dtype=torch.float32)
        err = (out.float().cpu() - ref).abs()
        assert err.max().item() <= TOL_MAX and err.mean().item() <= TOL_MEAN, err.max().item()
    ops.read_status(torch.device("cuda"))


def test_bounded_wait_runs_out_and_is_reported():
    """Every device-side wait in the kernels is bounded.  The self-test block waits, with a short
    budget, on a barrier nothing completes: the kernel returns normally, the status word names
    the site, the host decodes it as a timeout, and the device keeps working afterwards."""
    from streamdiffusionv2_b200 import _native
    ops = _ops()
    dev = torch.device("cuda")
    ops.read_status(dev)                                   # clean slate
    ops.selftest_wait_timeout(dev, budget_cycles=2_000_000)
    with pytest.raises(_native.NativeError) as e:
        ops.read_status(dev)
    assert e.value.code == _native.ERR_TIMEOUT and "site 7" in str(e.value)
    ops.read_status(dev)                                   # reading cleared the word
    # the non-blocking watch the forwards use sees it too (within two polls)
    ops.selftest_wait_timeout(dev, budget_cycles=2_000_000)
    torch.cuda.synchronize()
    with pytest.raises(_native.NativeError):
        for _ in range(3):
            ops.poll_status(dev)
            torch.cuda.synchronize()
    ops.read_status(dev)
    # and the context is intact: a real launch still gives the right answer
    q, k, v = _rand_case(1, 128, 1, 256, seed=5)
    out = ops.attn_kvcache(q.cuda(), k.cuda(), v.cuda(), [256])
    ref = orc.attend_explicit(q, k, v, [256], dtype=torch.float32)
    assert (out.float().cpu() - ref).abs().max().item() <= TOL_MAX


@pytest.mark.parametrize("B,N,H,grid,fused_proj", [
    (2, 3120, 12, (2, 30, 52), True),      # the 1.3B chunk, q/k/v as slices of one fused projection
    (4, 1560, 40, (1, 30, 52), True),      # 14B heads
    (1, 24, 2, (2, 3, 4), False),          # tiny, separate tensors
    (3, 50, 5, (2, 5, 5), True),           # odd sizes: ragged tiles, 640-element rows
])
def test_fused_norm_append_equals_rmsnorm_then_append_bit_for_bit(B, N, H, grid, fused_proj):
    """The RMS norm of q and k folded into the append launch sums the row statistics in the order
    the stand-alone norm kernel uses, so roped q, the K slots and the V slots are identical to
    norm -> append; and both stay within two bf16 steps of the PyTorch op chain."""
    ops = _ops()
    D, S = 128, N + 40
    dim = H * D
    g = torch.Generator().manual_seed(B * 1000 + H)
    if fused_proj:
        qkv = (torch.randn(B, N, 3, H, D, generator=g) * 1.7).to(torch.bfloat16).cuda()
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    else:
        q, k, v = ((torch.randn(B, N, H, D, generator=g) * 1.7).to(torch.bfloat16).cuda() for _ in range(3))
    wq = (1 + 0.2 * torch.randn(dim, generator=g)).to(torch.bfloat16).cuda()
    wk = (1 + 0.2 * torch.randn(dim, generator=g)).to(torch.bfloat16).cuda()
    eps = 1e-6
    assert ops.can_fuse_norm(q, k, v, wq, wk)
    table = ops.rope_table_device(orc.rope_table(D), torch.device("cuda"))
    sf = [(3 * b + 1) % 50 for b in range(B)]
    dst = [(7 * b) % 41 for b in range(B)]

    def caches():
        return (torch.zeros(B, S, H, D, dtype=torch.bfloat16, device="cuda"),
                torch.zeros(B, S, H, D, dtype=torch.bfloat16, device="cuda"))

    kc1, vc1 = caches()
    qn = ops.rmsnorm(q.reshape(B, N, dim), wq, eps).view(B, N, H, D)
    kn = ops.rmsnorm(k.reshape(B, N, dim), wk, eps).view(B, N, H, D)
    rq1 = ops.rope_kv_append(qn, kn, v, kc1, vc1, table, grid, sf, dst)
    kc2, vc2 = caches()
    ge, le = torch.zeros(B, dtype=torch.long, device="cuda"), torch.zeros(B, dtype=torch.long, device="cuda")
    rq2 = ops.rope_kv_append(q, k, v, kc2, vc2, table, grid, sf, dst, norm=(wq, wk, eps), index_tensors=(ge, le),
                             index_values=(list(range(B)), list(range(10, 10 + B))))
    assert torch.equal(rq1, rq2), "roped q differs"
    assert torch.equal(kc1, kc2), "K slots differ"
    assert torch.equal(vc1, vc2), "V slots differ"
    assert ge.tolist() == list(range(B)) and le.tolist() == list(range(10, 10 + B))
    # device-resident slot parameters (the form a captured graph uses)
    kc3, vc3 = caches()
    sp = torch.tensor([sf, dst, [0] * B, [0] * B], dtype=torch.long, device="cuda")
    rq3 = ops.rope_kv_append(q, k, v, kc3, vc3, table, grid, sf, dst, norm=(wq, wk, eps), step_params=sp)
    assert torch.equal(rq3, rq2) and torch.equal(kc3, kc2) and torch.equal(vc3, vc2)
    # against the PyTorch chain of the reference's norm, then the oracle's rope
    qf = q.float().reshape(B, N, dim)
    want_n = ((qf * torch.rsqrt(qf.pow(2).mean(dim=-1, keepdim=True) + eps)).to(torch.bfloat16) * wq).view(B, N, H, D)
    assert (qn == want_n).float().mean().item() > 0.995
    want = orc.rope_apply(qn.cpu(), grid, orc.rope_table(D), sf)
    assert torch.equal(rq2.cpu().view(torch.int16), want.view(torch.int16))
    ops.read_status(torch.device("cuda"))


def test_device_plan_kernel_follows_the_host_statement_of_the_queue_logic():
    """The kernel that keeps the evict queue on the device (adaptive sink refresh) against
    `RingState.queue_step`, its host-side specification (itself checked against the oracle's slot
    logic on the CPU): random similarities, branches, pops and pushes over many calls, both ways of
    passing the host inputs, bf16 and fp32 similarities."""
    import random
    from streamdiffusionv2_b200.ring_state import RingState
    ops = _ops()
    dev = torch.device("cuda")
    rnd = random.Random(9)
    for dtype in (torch.bfloat16, torch.float32):
        rows, sink, fs, n_new, thr = 5, 3, 60, 60, 0.2
        cap = RingState.QUEUE_CAP
        queues = [[(j + 4) * fs for j in range(rnd.randrange(1, 6))] for _ in range(rows)]
        qdev = torch.zeros(rows, 1 + cap, dtype=torch.int64)
        for i, lst in enumerate(queues):
            qdev[i, 0] = len(lst)
            qdev[i, 1:1 + len(lst)] = torch.tensor(lst)
        qdev = qdev.to(dev)
        step = torch.zeros(4, rows, dtype=torch.int64, device=dev)
        for call in range(40):
            sim = (torch.rand(rows, sink) * 0.6).to(dtype)
            inputs = [[rnd.randrange(900) for _ in range(rows)], [rnd.randrange(10 ** 6) for _ in range(rows)],
                      [rnd.randrange(10 ** 6) for _ in range(rows)], [], [], [], []]
            want_slots = []
            for i in range(rows):
                evict = bool(queues[i]) and rnd.random() < 0.6
                pop = evict and rnd.random() < 0.7
                push = -1 if evict or rnd.random() < 0.3 else (rnd.randrange(4, 12)) * fs
                begin = rnd.randrange(0, 500)
                for lst, val in zip(inputs[3:], (int(evict), int(pop), push, begin)):
                    lst.append(val)
                row = sim[i].float()
                lo = float(row.min())
                thr_t = float(torch.tensor(thr, dtype=dtype))
                front = (int(torch.argmin(row)) + 1) * fs if lo < thr_t else None
                if len(queues[i]) + 2 > cap:
                    front = None if front is None else front          # never reached with these sizes
                want_slots.append(RingState.queue_step(queues[i], front, evict, pop, push, begin, n_new, sink * fs))
            kw = {"host_inputs": inputs} if call % 2 == 0 else {
                "host_inputs_dev": torch.tensor(inputs, dtype=torch.int64, device=dev)}
            ops.ring_plan_adaptive(sim.to(dev), thr, qdev, fs, n_new, step, **kw)
            got = step.cpu()
            assert got[0].tolist() == inputs[0] and got[2].tolist() == inputs[1] and got[3].tolist() == inputs[2]
            assert got[1].tolist() == want_slots, (call, got[1].tolist(), want_slots)
            host = qdev.cpu().tolist()
            assert [r[1:1 + r[0]] for r in host] == queues, call
        ops.read_status(dev)
    # an empty queue in the evict branch is refused (the reference raises there): slot -1 and a status report
    from streamdiffusionv2_b200 import _native
    qdev.zero_()
    ops.ring_plan_adaptive(None, thr, qdev, fs, n_new, step,
                           host_inputs=[[0] * rows, [0] * rows, [0] * rows, [1] * rows, [1] * rows, [-1] * rows, [0] * rows])
    assert step[1].tolist() == [-1] * rows
    with pytest.raises(_native.NativeError, match="out of range"):
        ops.read_status(dev)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_frame_means_match_the_reference_reductions(dtype):
    """The per-frame means the adaptive sink test needs (sink frames of the K / V cache, the new
    frame), two launches for all rows, against the `.mean` reductions of the reference's op chain:
    same fp32 sums up to the order of the additions, rounded once to the tensors' type."""
    ops = _ops()
    rows, sink, fs, H, D, S = 3, 3, 1560, 12, 128, 9 * 1560
    g = torch.Generator().manual_seed(17)
    kc = (torch.randn(rows, S, H, D, generator=g) + 0.3).to(dtype).cuda()
    vc = (torch.randn(rows, S, H, D, generator=g) - 0.2).to(dtype).cuda()
    kn = (torch.randn(rows, fs, H, D, generator=g) + 0.1).to(dtype).cuda()
    vn = torch.randn(rows, fs, H, D, generator=g).to(dtype).cuda()
    means = ops.frame_means(kc, vc, kn, vn, sink, fs)
    assert means.shape == (rows, sink + 1, 2, H * D) and means.dtype == dtype
    for tensor, cache, new in ((0, kc, kn), (1, vc, vn)):
        want_sink = cache[:, :sink * fs].reshape(rows, sink, fs, -1).mean(2)
        want_new = new.reshape(rows, 1, fs, -1).mean(2)
        for got, want in ((means[:, :sink, tensor], want_sink), (means[:, sink:, tensor], want_new)):
            if dtype == torch.float32:
                assert torch.allclose(got, want, rtol=0, atol=2e-6)
            else:
                assert (got == want).float().mean().item() > 0.995
                assert ((got.float() - want.float()).abs() <= want.float().abs() * 2.0 ** -7 + 1e-9).all()
    # a cache that is a slice of a larger buffer (row stride != tokens x row) works too
    big = torch.zeros(rows, S + 50, H, D, dtype=dtype, device="cuda")
    big[:, :S] = kc
    m2 = ops.frame_means(big[:, :S], vc, kn, vn, sink, fs)
    assert torch.equal(m2, means)
    ops.read_status(torch.device("cuda"))


def test_adaptive_queue_follows_a_replaced_evict_idx():
    """With the adaptive sink test the evict queue is kept on the device, but `evict_idx` stays the
    reference's attribute: a tool that assigns a new list (the demo's cache resizer copies row 0 to
    every row, demo/vid2vid.py:146-148) must be obeyed from the next call on.  CUDA path and oracle
    in lockstep, the same rewrite applied to both half-way."""
    from streamdiffusionv2_b200 import causal_attention as ca
    case = cases.KERNEL_CASES["k_bf16_adaptive"]
    rewritten = False
    for (i, _, _, cache, _, _, _), (j, out, kv, mod) in zip(replay_oracle(case), replay_cuda(case)):
        assert i == j
        st = cache.state
        assert mod.evict_idx == st.evict_idx, i
        assert kv["global_end_index"].tolist() == st.global_end and kv["local_end_index"].tolist() == st.local_end
        assert cases.sha(kv["k"]) == cases.sha(cache.k), f"K cache differs at call {i}"
        if i == 9:
            rows = len(st.evict_idx)
            st.evict_idx = [list(st.evict_idx[0]) + [4 * 6] for _ in range(rows)]      # row 0 everywhere, one more slot
            mod.evict_idx = [list(r) for r in st.evict_idx]                             # a new list: what a tool would assign
            rewritten = True
    assert rewritten and i > 12
    _ops().read_status(torch.device("cuda"))

"""The tiny causal DiT on the GPU against the fixtures recorded from the reference's own model and
streaming pipeline: this package's model + scheduler, and the reference's own classes with
`install()` bound onto them, both running the CUDA kernels.

Index tensors, evict queues and step counters do not depend on the data, so they are checked
bit-exact for EVERY layer after every chunk, in fp32 and in bf16.  In fp32 the re-noising draws are
taken from the CPU generator exactly as when the fixtures were recorded, so the denoised latents
are also compared with the reference's (2e-3: fp32 GEMMs and attention on another device)."""
import numpy as np
import pytest
import torch

import cases
from model_harness import build_pipeline, snapshot
from oracle.reference_shim import import_reference, reference_root, set_flash_attn

pytestmark = pytest.mark.gpu
INDEX_KEYS = ("global_end", "local_end", "evict_idx", "current_step")


@pytest.fixture
def cpu_noise(monkeypatch):
    """torch.randn_like drawing from the default CPU generator whatever the tensor's device, so a
    GPU run consumes the same noise as the CPU run that produced the fixtures."""
    def randn_like(t, **kw):
        return torch.randn(t.shape, dtype=torch.float32).to(device=t.device, dtype=t.dtype)
    monkeypatch.setattr(torch, "randn_like", randn_like)


def _run_stream(pipe, case, dtype, snapshot_fn, n_layers, meta, z, out_tol):
    dev = torch.device("cuda")
    prompt, first, chunks = cases.model_inputs(case)
    fs, sched = cases.model_schedule(case)
    torch.manual_seed(case["seed"] + 1)
    outs = []
    with torch.no_grad():
        out0 = pipe.prepare(text_prompts=["p"], device=dev, dtype=dtype, noise=first.to(dev, dtype), current_start=0,
                            current_end=fs * (1 + case["frames"]))
        for l in range(n_layers):
            got = snapshot_fn(pipe, l)
            for k in INDEX_KEYS:
                assert got[k] == meta["prepare"]["layer0"][k], ("prepare", l, k)
        if out_tol is not None:
            assert np.abs(out0.float().cpu().numpy() - z["prepare"]).max() < out_tol
        for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
            hs = pipe.inference_stream(noise=noise.to(dev, dtype), current_start=cs, current_end=ce, current_step=None)
            assert torch.isfinite(hs).all()
            want = meta["steps"][i]["layer0"]
            assert all(meta["steps"][i]["layerL"][k] == want[k] for k in INDEX_KEYS)   # data independent
            for l in range(n_layers):
                got = snapshot_fn(pipe, l)
                for k in INDEX_KEYS:
                    assert got[k] == want[k], (i, l, k, got[k], want[k])
            if out_tol is not None:
                assert np.abs(hs.float().cpu().numpy() - z[f"out_{i}"]).max() < out_tol, i
            outs.append(hs.float().cpu())
    from streamdiffusionv2_b200 import ops
    ops.read_status(dev)
    return outs


@pytest.mark.parametrize("name", ["m_stream", "m_stream_1f"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_package_model_on_gpu_reproduces_reference_fixture(name, dtype, cpu_noise):
    case = cases.MODEL_CASES[name]
    meta, z = cases.load_fixture(name)
    pipe, _, _ = build_pipeline(case, device="cuda", dtype=dtype)
    _run_stream(pipe, case, dtype, snapshot, cases.MODEL_KW["num_layers"], meta, z,
                2e-3 if dtype == torch.float32 else None)


# ------------------------------------------------------------------------------------------------
# the reference's own classes, kernels bound onto them
# ------------------------------------------------------------------------------------------------
REFERENCE = reference_root()
needs_reference = pytest.mark.skipif(REFERENCE is None, reason="reference not present (checkout or baseline/_ref)")


def _reference_pipeline(case, dtype, flash):
    import make_golden_model
    ref = import_reference(REFERENCE, flash_attn=flash)
    return ref, make_golden_model.build_reference_pipeline(ref, case, device="cuda", dtype=dtype)


@needs_reference
@pytest.mark.parametrize("name", ["m_stream", "m_stream_1f"])
def test_install_on_reference_classes_fp32_on_gpu(name, cpu_noise):
    """Drop-in check with real kernels: the reference's CausalWanModel under its own
    CausalStreamInferencePipeline, attention forwards replaced by `install()`, on the GPU in fp32
    (append kernel + CUDA-core attention): reference fixture reproduced, index state of every
    layer exact, parameters untouched."""
    import make_golden_model
    from streamdiffusionv2_b200.causal_attention import install
    case = cases.MODEL_CASES[name]
    meta, z = cases.load_fixture(name)
    ref, pipe = _reference_pipeline(case, torch.float32, flash=False)
    names = [n for n, _ in pipe.generator.model.named_parameters()]
    assert install(pipe.generator.model) == cases.MODEL_KW["num_layers"]
    assert [n for n, _ in pipe.generator.model.named_parameters()] == names
    _run_stream(pipe, case, torch.float32, make_golden_model.snapshot, cases.MODEL_KW["num_layers"], meta, z, 2e-3)
    assert set(pipe.kv_cache1[0]) - {"_sdv2_host"} == {"k", "v", "global_end_index", "local_end_index",
                                                        "total_steps", "current_step"}


@needs_reference
@pytest.mark.parametrize("name", ["m_stream", "m_stream_1f"])
def test_install_on_reference_classes_bf16_against_the_reference_gpu_path(name, cpu_noise):
    """bf16 on the GPU: the stock reference (its flash-attn / PyTorch GPU path) and the same classes
    after `install()` (tensor-core attention, fused append, fused element-wise chains) stream the
    same chunks; index state exact in both, latents equal to bf16 accuracy."""
    import make_golden_model
    from streamdiffusionv2_b200.causal_attention import install
    case = cases.MODEL_CASES[name]
    meta, z = cases.load_fixture(name)
    nl = cases.MODEL_KW["num_layers"]
    ref, stock = _reference_pipeline(case, torch.bfloat16, flash=True)
    try:
        want = _run_stream(stock, case, torch.bfloat16, make_golden_model.snapshot, nl, meta, z, None)
    finally:
        set_flash_attn(ref, False)
    ref, ours = _reference_pipeline(case, torch.bfloat16, flash=False)
    install(ours.generator.model)
    got = _run_stream(ours, case, torch.bfloat16, make_golden_model.snapshot, nl, meta, z, None)
    for i, (a, b) in enumerate(zip(got, want)):
        err = (a - b).abs()
        scale = b.abs().mean().item()
        assert err.mean().item() <= 0.03 * scale and err.max().item() <= 0.5 * b.abs().max().item(), \
            (i, err.mean().item(), err.max().item(), scale)


# ------------------------------------------------------------------------------------------------
# one layer, teacher-forced: the reference's own module on the GPU beside the kernels
# ------------------------------------------------------------------------------------------------
@needs_reference
@pytest.mark.parametrize("name", ["k_bf16_stream", "k_bf16_single_2level", "k_bf16_1frame_sink3", "k_bf16_sink0_3frames"])
def test_layer_against_the_reference_module_on_the_gpu(name):
    """The reference's CausalWanSelfAttention on the GPU in bf16 (its stock path: fp64 complex rope on
    the device, slice writes, flash_attn_with_kvcache) and the kernels are fed the same projected
    q/k/v call after call, each against its own cache.  Index tensors, evict queues and step counters
    must be identical after every call; the caches equal - bit for bit, except where the device's
    fused multiply-add in the reference's complex product rounds the last place the other way
    (allowed: at most 1e-5 of the elements, one bf16 step) - and the outputs equal to the attention
    tolerance, against flash-attn itself."""
    import make_golden
    import replay
    from streamdiffusionv2_b200 import causal_attention as ca
    ref = import_reference(REFERENCE, flash_attn=True)
    try:
        case = cases.KERNEL_CASES[name]
        H, D = case["heads"], case["head_dim"]
        dtype, dev = torch.bfloat16, torch.device("cuda")
        h, w = case["grid_hw"]
        fs = h * w
        smax = case["cache_frames"] * fs
        layer = make_golden.make_ref_layer(ref, H, D, case["sink_size"], case["adapt_sink_thr"]).to(dev)
        table = make_golden.ref_table(ref, D).to(dev)
        mk = lambda: {"k": torch.zeros(1, smax, H, D, dtype=dtype, device=dev),
                      "v": torch.zeros(1, smax, H, D, dtype=dtype, device=dev),
                      "global_end_index": torch.tensor([0], dtype=torch.long, device=dev),
                      "local_end_index": torch.tensor([0], dtype=torch.long, device=dev),
                      "total_steps": case["total_steps"], "current_step": case["total_steps"]}
        kv_ref, kv = mk(), mk()
        mod = replay._AttnState(H, D, case["sink_size"], case["adapt_sink_thr"])
        freqs = make_golden.ref_table(ref, D)            # complex128 on the host: the table both sides were built from
        gen = cases.InputStream(case)
        n_calls = 0
        for call in cases.schedule(case):
            if call["op"] == "replicate":
                for c in (kv_ref, kv):
                    b = call["rows"]
                    c["k"], c["v"] = c["k"].repeat(b, 1, 1, 1), c["v"].repeat(b, 1, 1, 1)
                    c["global_end_index"] = c["global_end_index"].repeat(b)
                    c["local_end_index"] = c["local_end_index"].repeat(b)
                continue
            starts, frames = call["starts"], call["frames"]
            q, k, v = (t.to(dev) for t in gen.next(len(starts), frames * fs))
            layer.q.value, layer.k.value, layer.v.value = (t.flatten(2) for t in (q, k, v))
            grid = torch.tensor([[frames, h, w]] * len(starts), dtype=torch.long)
            cs = torch.tensor(starts, dtype=torch.long, device=dev)
            x = torch.zeros(len(starts), frames * fs, H * D, dtype=dtype, device=dev)
            with torch.no_grad():
                want = layer(x, None, grid, table, None, kv_ref, cs, cs + frames * fs).view(len(starts), -1, H, D)
            got = ca.cached_attention(mod, q, k, v, grid, freqs, kv, cs)
            assert kv["global_end_index"].tolist() == kv_ref["global_end_index"].tolist(), (name, n_calls)
            assert kv["local_end_index"].tolist() == kv_ref["local_end_index"].tolist(), (name, n_calls)
            assert mod.evict_idx == [list(map(int, r)) for r in layer.evict_idx], (name, n_calls)
            assert kv["current_step"] == kv_ref["current_step"], (name, n_calls)
            assert torch.equal(kv["v"], kv_ref["v"]), (name, n_calls)
            diff = kv["k"].view(torch.int16) != kv_ref["k"].view(torch.int16)
            if diff.any():
                assert diff.float().mean().item() <= 1e-5, (name, n_calls, diff.float().mean().item())
                a, b = kv["k"][diff].float(), kv_ref["k"][diff].float()
                assert ((a - b).abs() <= b.abs() * 2.0 ** -7).all(), (name, n_calls)
                kv["k"].copy_(kv_ref["k"])           # teacher forcing: the next call starts from the reference's cache
            err = (got.float() - want.float()).abs()
            assert err.max().item() <= 2e-2 and err.mean().item() <= 1e-3, (name, n_calls, err.max().item())
            n_calls += 1
        assert n_calls > 8
    finally:
        set_flash_attn(ref, False)

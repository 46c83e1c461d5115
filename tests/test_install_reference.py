"""Drop-in check on the reference's own classes: `install()` rebinds the attention forwards of a
reference CausalWanModel, and the reference's unmodified CausalStreamInferencePipeline
(prepare / inference_stream) then reproduces the fixture it produced without `install()`.
Needs the reference checkout, so it only runs where that exists; the kernels are replaced by the
oracle (tests/fake_ops.py) because this machine has no GPU - what is under test is the wiring:
signatures, cache dict keys, module attributes, index state, parameter names."""
import os
import sys

import numpy as np
import pytest
import torch

import cases
import fake_ops

from oracle.reference_shim import reference_root

# $SDV2_REFERENCE (a checkout) or baseline/_ref (the reference pip-installed with --target)
REFERENCE = reference_root()
pytestmark = pytest.mark.skipif(REFERENCE is None, reason="reference not present (checkout or baseline/_ref)")


@pytest.fixture(scope="module")
def ref():
    import make_golden
    return make_golden.import_reference(REFERENCE)


@pytest.mark.parametrize("name", ["m_stream", "m_stream_1f"])
def test_reference_pipeline_runs_on_installed_forwards(ref, name, monkeypatch):
    import make_golden_model
    from streamdiffusionv2_b200.causal_attention import install
    fake_ops.install(monkeypatch)
    case = cases.MODEL_CASES[name]
    meta, z = cases.load_fixture(name)
    pipe = make_golden_model.build_reference_pipeline(ref, case)
    names_before = [n for n, _ in pipe.generator.model.named_parameters()]
    assert install(pipe.generator.model) == cases.MODEL_KW["num_layers"]
    assert [n for n, _ in pipe.generator.model.named_parameters()] == names_before
    prompt, first, chunks = cases.model_inputs(case)
    fs, sched = cases.model_schedule(case)
    torch.manual_seed(case["seed"] + 1)
    with torch.no_grad():
        out0 = pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                            current_start=0, current_end=fs * (1 + case["frames"]))
        assert np.abs(out0.numpy() - z["prepare"]).max() < 2e-4
        for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
            hs = pipe.inference_stream(noise=noise, current_start=cs, current_end=ce, current_step=None)
            assert np.abs(hs.numpy() - z[f"out_{i}"]).max() < 5e-4, (name, i)
            got = make_golden_model.snapshot(pipe, 0)
            want = meta["steps"][i]["layer0"]
            for k in ("global_end", "local_end", "evict_idx", "current_step", "k_sha", "v_sha"):
                assert got[k] == want[k], (name, i, k)
    # the cache dicts keep the reference's keys (plus one private key)
    assert set(pipe.kv_cache1[0]) - {"_sdv2_host"} == {"k", "v", "global_end_index", "local_end_index",
                                                        "total_steps", "current_step"}

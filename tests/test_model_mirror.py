"""Host logic of the model mirror and the streaming scheduler against fixtures recorded from the
reference's CausalWanModel + CausalStreamInferencePipeline (CPU, fp32).  Attention arithmetic is
supplied by the oracle through tests/fake_ops.py; what is under test is everything around it:
parameter naming, block wiring, stage slicing, cache ownership, row shifting, index state."""
import numpy as np
import pytest
import torch

import cases
import fake_ops
from model_harness import build_pipeline, snapshot

INDEX_KEYS = ("global_end", "local_end", "evict_idx", "current_step")


def _check_state(got, want, where):
    for k in INDEX_KEYS:
        assert got[k] == want[k], (where, k, got[k], want[k])


@pytest.mark.parametrize("name", ["m_stream", "m_stream_1f"])
def test_stream_pipeline_matches_reference(name, monkeypatch):
    fake_ops.install(monkeypatch)
    case = cases.MODEL_CASES[name]
    meta, z = cases.load_fixture(name)
    pipe, first, chunks = build_pipeline(case)
    fs, sched = cases.model_schedule(case)
    nl = cases.MODEL_KW["num_layers"]
    torch.manual_seed(case["seed"] + 1)
    with torch.no_grad():
        out0 = pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                            current_start=0, current_end=fs * (1 + case["frames"]))
        assert np.abs(out0.numpy() - z["prepare"]).max() < 2e-4
        _check_state(snapshot(pipe, 0), meta["prepare"]["layer0"], "prepare")
        # layer 0 sees identical inputs, so its cache must match the reference bit for bit
        assert snapshot(pipe, 0)["k_sha"] == meta["prepare"]["layer0"]["k_sha"]
        for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
            hs = pipe.inference_stream(noise=noise, current_start=cs, current_end=ce, current_step=None)
            assert np.abs(hs.numpy() - z[f"out_{i}"]).max() < 5e-4, (name, i)
            _check_state(snapshot(pipe, 0), meta["steps"][i]["layer0"], (name, i, 0))
            _check_state(snapshot(pipe, nl - 1), meta["steps"][i]["layerL"], (name, i, nl - 1))


def test_two_stage_pipeline_matches_reference(monkeypatch):
    fake_ops.install(monkeypatch)
    case = cases.MODEL_CASES["m_stages"]
    meta, z = cases.load_fixture("m_stages")
    split, nblk = case["split"], cases.MODEL_KW["num_layers"]
    fs, sched = cases.model_schedule(case)
    pa, first, chunks = build_pipeline(case)
    pb, _, _ = build_pipeline(case)
    with torch.no_grad():
        for pipe, mode in ((pa, "input"), (pb, "output")):
            torch.manual_seed(case["seed"] + 1)
            pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                         current_start=0, current_end=fs * (1 + case["frames"]), block_mode=mode)
        torch.manual_seed(case["seed"] + 2)
        world, returns = 2, []
        for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
            if i >= world:                      # ring depth: the return of chunk i-2 arrives now
                lat, st, en = returns[i - world]
                pa.hidden_states.copy_(lat)
                pa.kv_cache_starts.copy_(torch.tensor(st))
                pa.kv_cache_ends.copy_(torch.tensor(en))
                pa._starts_host, pa._ends_host = list(st), list(en)
            act, pshape = pa.inference(noise=noise, current_start=cs, current_end=ce, current_step=None,
                                       block_mode="input", block_num=[0, split])
            st, en = list(pa._starts_host), list(pa._ends_host)
            assert st == meta["steps"][i]["starts"] and en == meta["steps"][i]["ends"]
            den, _ = pb.inference(noise=pa.hidden_states.clone(), current_start=st, current_end=en,
                                  current_step=None, block_mode="output", block_num=[split, nblk],
                                  patched_x_shape=pshape, block_x=act)
            returns.append((den.clone(), st, en))
            assert pshape.tolist() == meta["steps"][i]["pshape"]
            assert np.abs(act.numpy() - z[f"act_{i}"]).max() < 5e-4, i
            assert np.abs(den.numpy() - z[f"out_{i}"]).max() < 5e-4, i
            _check_state(snapshot(pa, 0), meta["steps"][i]["stageA_layer0"], (i, "A"))
            _check_state(snapshot(pb, nblk - 1), meta["steps"][i]["stageB_layerL"], (i, "B"))


def test_parameter_names_match_reference_layout():
    """Checkpoints written for the reference model must load with strict=True: same names/shapes."""
    from streamdiffusionv2_b200.wan_model import CausalWanModel
    m = CausalWanModel(**cases.MODEL_KW)
    names = dict((n, tuple(p.shape)) for n, p in m.named_parameters())
    for blk in range(cases.MODEL_KW["num_layers"]):
        for sub in ("self_attn", "cross_attn"):
            for lin in ("q", "k", "v", "o"):
                assert names[f"blocks.{blk}.{sub}.{lin}.weight"] == (256, 256)
            assert names[f"blocks.{blk}.{sub}.norm_q.weight"] == (256,)
        assert names[f"blocks.{blk}.modulation"] == (1, 6, 256)
        assert names[f"blocks.{blk}.norm3.weight"] == (256,)
        assert names[f"blocks.{blk}.ffn.0.weight"] == (512, 256)
    assert names["patch_embedding.weight"] == (256, 16, 1, 2, 2)
    assert names["head.head.weight"] == (64, 256) and names["head.modulation"] == (1, 2, 256)
    assert names["time_projection.1.weight"] == (1536, 256)
    assert names["text_embedding.0.weight"] == (256, 64)
    want = set(cases.load_fixture("m_stream")[0].get("param_names", [])) or None
    if want:
        assert set(names) == want


def test_external_index_writes_are_picked_up(monkeypatch):
    """A foreign writer (cache re-ownership, session tools) changes the index tensors; the host
    mirror must notice and re-read them instead of trusting its own copy."""
    fake_ops.install(monkeypatch)
    from streamdiffusionv2_b200.ring_state import RingState
    kv = {"k": torch.zeros(2, 60, 1, 128), "v": torch.zeros(2, 60, 1, 128),
          "global_end_index": torch.tensor([12, 12]), "local_end_index": torch.tensor([12, 12]),
          "total_steps": 2, "current_step": 2}
    st = RingState.of(kv)
    assert st.global_end == [12, 12]
    kv["global_end_index"] += 6          # in-place write by someone else
    kv["local_end_index"] = torch.tensor([18, 18])   # tensor replaced
    st2 = RingState.of(kv)
    assert st2.global_end == [18, 18] and st2.local_end == [18, 18]
    assert RingState.of(kv) is st2       # no re-read while nothing changed


def test_device_status_surfaces_from_the_streaming_entry_points(monkeypatch):
    """A kernel that gave up a bounded wait (or refused its parameters) writes nothing; the forwards
    look at the device status word every few attention calls so that the stream stops with an error
    instead of carrying garbage.  Here the look itself is replaced by a host-side fake."""
    fake_ops.install(monkeypatch)
    from streamdiffusionv2_b200 import _native, causal_attention, ops
    case = cases.MODEL_CASES["m_stream"]
    pipe, first, chunks = build_pipeline(case)
    fs, sched = cases.model_schedule(case)
    state = {"raised": False, "polls": 0}

    def poll(device):
        state["polls"] += 1
        if state["raised"]:
            raise _native.NativeError(_native.ERR_TIMEOUT, "device status", "a kernel reported status 0x7 earlier")

    monkeypatch.setattr(ops, "poll_status", poll)
    monkeypatch.setattr(causal_attention, "_POLL_EVERY", 2)
    with torch.no_grad():
        pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                     current_start=0, current_end=fs * (1 + case["frames"]))
        pipe.inference_stream(noise=chunks[0], current_start=sched[0][0], current_end=sched[0][1])
        assert state["polls"] >= 1               # the healthy path polls and goes on
        state["raised"] = True
        with pytest.raises(_native.NativeError, match="status"):
            pipe.inference_stream(noise=chunks[1], current_start=sched[1][0], current_end=sched[1][1])
        # the entry point the pipeline-stage runner calls
        with pytest.raises(_native.NativeError, match="status"):
            pipe.inference(noise=chunks[2], current_start=sched[2][0], current_end=sched[2][1], current_step=None,
                           block_mode="input", block_num=[0, 2])


def test_concatenated_qkv_weight_follows_the_parameters():
    """The q|k|v projection runs as one GEMM over a concatenated copy of the three weights; the copy is
    rebuilt whenever a parameter is written (load_state_dict, in-place updates) or replaced, and the
    parameters themselves keep their names and values."""
    from streamdiffusionv2_b200.causal_attention import _fused_qkv_weights
    from streamdiffusionv2_b200.wan_model import CausalSelfAttention
    torch.manual_seed(0)
    attn = CausalSelfAttention(256, 2)
    names = sorted(n for n, _ in attn.named_parameters())
    w, b = _fused_qkv_weights(attn)
    assert w.shape == (768, 256) and b.shape == (768,)
    assert torch.equal(w[256:512], attn.k.weight) and torch.equal(b[512:], attn.v.bias)
    assert _fused_qkv_weights(attn)[0] is w                                  # cached while nothing changes
    x = torch.randn(3, 5, 256)
    q, k, v = torch.nn.functional.linear(x, w, b).view(3, 5, 3, 256).unbind(2)
    assert torch.allclose(q, attn.q(x), atol=1e-5) and torch.allclose(v, attn.v(x), atol=1e-5)
    state = {n: torch.randn_like(p) for n, p in attn.state_dict().items()}
    attn.load_state_dict(state, strict=True)                                  # copies in place: version counters move
    w2, b2 = _fused_qkv_weights(attn)
    assert w2 is not w and torch.equal(w2[:256], state["q.weight"]) and torch.equal(b2[256:512], state["k.bias"])
    with torch.no_grad():
        attn.v.weight.mul_(2.0)
    assert torch.equal(_fused_qkv_weights(attn)[0][512:], attn.v.weight)
    attn.q.weight = torch.nn.Parameter(torch.zeros(256, 256))                 # replaced outright
    assert float(_fused_qkv_weights(attn)[0][:256].abs().max()) == 0.0
    assert sorted(n for n, _ in attn.named_parameters()) == names            # nothing was registered on the module


def test_stacked_modulation_follows_the_parameters():
    """The blocks' `modulation + e` sums are formed in one launch from a stacked copy of the blocks' modulation
    parameters; the copy is rebuilt when a parameter is written or replaced, covers exactly the block range
    asked for, and registers nothing on the model."""
    from streamdiffusionv2_b200.wan_model import CausalWanModel
    torch.manual_seed(0)
    m = CausalWanModel(**cases.MODEL_KW)
    names = sorted(n for n, _ in m.named_parameters())
    n = len(m.blocks)
    s = m._stacked_modulation(0, n)
    assert s.shape == (n, 1, 1, 6, m.dim)
    assert all(torch.equal(s[i, 0], m.blocks[i].modulation) for i in range(n))
    assert m._stacked_modulation(0, n) is s                                   # cached while nothing changes
    with torch.no_grad():
        m.blocks[1].modulation.add_(1.0)                                      # in place: the version counter moves
    s2 = m._stacked_modulation(0, n)
    assert s2 is not s and torch.equal(s2[1, 0], m.blocks[1].modulation)
    m.blocks[0].modulation = torch.nn.Parameter(torch.zeros_like(m.blocks[0].modulation))   # replaced outright
    assert float(m._stacked_modulation(0, n)[0].abs().max()) == 0.0
    part = m._stacked_modulation(1, n)                                        # a stage's own range
    assert part.shape[0] == n - 1 and torch.equal(part[0, 0], m.blocks[1].modulation)
    e = torch.randn(2, 3, 6, m.dim)
    assert torch.equal((part + e.unsqueeze(0))[0], m.blocks[1].modulation.unsqueeze(1) + e)
    assert sorted(k for k, _ in m.named_parameters()) == names

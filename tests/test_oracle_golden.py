"""The oracle is pinned against outputs of the reference implementation (tests/golden/*.npz,
index_traces.json): K/V cache bytes, index state and evict queues bit-exact, attention outputs
bit-exact too (same library arithmetic on the same CPU path)."""
import numpy as np
import pytest
import torch

import cases
from oracle import causal_attention_oracle as orc
from replay import replay_oracle


@pytest.mark.parametrize("name", sorted(cases.KERNEL_CASES))
def test_oracle_matches_reference_fixture(name):
    case = cases.KERNEL_CASES[name]
    meta, z = cases.load_fixture(name)
    n = 0
    for i, (q, k, v), out, cache, rq, sl, dst in replay_oracle(case):
        g = meta["steps"][i]
        assert cases.sha(torch.stack([q, k, v])) == g["in_sha"], "seeded inputs changed"
        st = cache.state
        assert st.global_end == g["global_end"]
        assert st.local_end == g["local_end"]
        assert st.evict_idx == g["evict_idx"]
        assert st.current_step == g["current_step"]
        assert cases.sha(cache.k) == g["k_sha"], f"K cache differs at call {i}"
        assert cases.sha(cache.v) == g["v_sha"], f"V cache differs at call {i}"
        ref_out = cases.from_numpy_bits(z[f"out_{i}"], g["out_dtype"])
        assert list(out.shape) == g["out_shape"]
        # same SDPA call on the same host: normally bit-identical; allow 1 ulp-level slack for
        # a different core count changing the reduction blocking
        tol = 1e-5 if out.dtype == torch.float32 else 8e-3
        assert (out.float() - ref_out.float()).abs().max().item() <= tol
        n += 1
    assert n == len(meta["steps"])


@pytest.mark.parametrize("name", sorted(cases.TRACE_CASES))
def test_ring_plan_matches_reference_trace(name):
    """Integer-only slot logic against traces recorded from the reference at 1560 tokens/frame."""
    case = cases.TRACE_CASES[name]
    trace = cases.load_traces()[name]
    h, w = case["grid_hw"]
    fs = h * w
    st = orc.RingLayerState(case["cache_frames"] * fs, 1, total_steps=case["total_steps"],
                            current_step=case["total_steps"])
    i = 0
    for call in cases.schedule(case):
        if call["op"] == "replicate":
            st.rows = call["rows"]
            st.global_end = st.global_end * st.rows
            st.local_end = st.local_end * st.rows
            continue
        dst, sl = orc.ring_plan(st, call["starts"], call["frames"] * fs, fs, case["sink_size"])
        g = trace[i]
        assert st.global_end == g["global_end"], i
        assert st.local_end == g["local_end"], i
        assert st.evict_idx == g["evict_idx"], i
        assert st.current_step == g["current_step"], i
        assert sl == g["local_end"]
        for b, d in enumerate(dst):
            assert 0 <= d and d + call["frames"] * fs <= st.cache_tokens
        i += 1
    assert i == len(trace)


def test_config1_trace_facts():
    """The properties of the config-1 run spelled out: 9 rotating slots, first chunk never
    evicted, last 1560 tokens never written."""
    case = cases.TRACE_CASES["t_config1"]
    st = orc.RingLayerState(32760, 1)
    written = np.zeros(32760, dtype=bool)
    for s in range(24):
        dst, sl = orc.ring_plan(st, [3120 * s], 3120, 1560, 1)
        written[dst[0]:dst[0] + 3120] = True
        if s <= 9:
            assert dst == [3120 * s] and sl == [3120 * (s + 1)]
        else:
            assert sl == [32760]
            assert dst[0] == 3120 + 3120 * ((s - 10) % 9)
    assert not written[31200:].any() and written[:31200].all()
    assert case["chunks"] == 24


@pytest.mark.parametrize("name", sorted(cases.CROSS_CASES))
def test_cross_attention_oracle(name):
    case = cases.CROSS_CASES[name]
    meta, z = cases.load_fixture(name)
    dtype = cases.DTYPES[case["dtype"]]
    g = torch.Generator().manual_seed(case["seed"])
    H, D = case["heads"], case["head_dim"]
    q = torch.randn(case["rows"], case["n"], H, D, generator=g).to(dtype)
    k = torch.randn(1, case["lk"], H, D, generator=g).to(dtype).expand(case["rows"], -1, -1, -1)
    v = torch.randn(1, case["lk"], H, D, generator=g).to(dtype).expand(case["rows"], -1, -1, -1)
    assert cases.sha(q) == meta["in_sha"]
    out = orc.cross_attend(q, k, v)
    ref = cases.from_numpy_bits(z["out"], meta["out_dtype"])
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    assert (out.float() - ref.float()).abs().max().item() <= tol


def test_rope_unfused_form_is_what_the_library_multiply_does():
    """fp64 complex multiply == rn(rn(ac)-rn(bd)), rn(rn(ad)+rn(bc)); and the bf16 storage
    rounding is fp64 -> fp32 -> bf16 (two steps)."""
    g = torch.Generator().manual_seed(5)
    table = orc.rope_table(128)
    grid = (2, 3, 4)
    x = torch.randn(2, 24, 3, 128, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        xs = x.to(dt)
        a = orc.rope_apply(xs, grid, table, [3, 40])
        b64 = orc.rope_apply_unfused_numpy(xs.double().numpy(), grid, table.numpy(), [3, 40])
        if dt == torch.float32:
            assert np.array_equal(a.numpy(), b64.astype(np.float32))
        else:
            assert np.array_equal(cases.to_numpy_bits(a), orc.f64_to_bf16_bits_two_step(b64))
    # the two-step rounding differs from a single correctly rounded step on this value
    v = np.array([1 + 2.0 ** -8 + 2.0 ** -30])
    assert orc.f64_to_bf16_bits_two_step(v)[0] == 0x3F80
    assert torch.tensor(v).to(torch.bfloat16).view(torch.int16).item() == 0x3F80


def test_attend_explicit_agrees():
    g = torch.Generator().manual_seed(9)
    q = torch.randn(2, 10, 2, 128, generator=g)
    k = torch.randn(2, 50, 2, 128, generator=g)
    v = torch.randn(2, 50, 2, 128, generator=g)
    a = orc.attend_cache(q, k, v, [50, 33])
    b = orc.attend_explicit(q, k, v, [50, 33])
    assert (a.double() - b).abs().max() < 1e-5

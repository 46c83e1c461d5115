"""Generate the golden fixtures in this directory by running the reference implementation.

Run from the repository root in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/StreamDiffusionV2

The reference is imported unmodified (with stub modules for two packages that are not
installed and are not used on this path), forced onto its own PyTorch fallback attention,
and driven with the seeded inputs defined in tests/golden/cases.py.  The fixtures hold the
reference's outputs only: per-step SHA-256 digests of the K/V cache bytes, the index state,
the evict queues and the attention outputs.  Inputs are re-created from the seeds by the
tests; their digests are stored so a change in the generator is told apart from a parity
failure.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def import_reference(root: str):
    """The reference's modules, forced onto its own PyTorch attention paths (oracle/reference_shim.py)."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle.reference_shim import import_reference as _imp
    return _imp(root, flash_attn=False)


class _Feed(torch.nn.Module):
    """Stands in for a q/k/v Linear: returns the tensor queued for this call."""

    def __init__(self):
        super().__init__()
        self.value = None

    def forward(self, x):
        return self.value


def make_ref_layer(ref, heads, head_dim, sink_size, adapt_thr):
    layer = ref.cm.CausalWanSelfAttention(dim=heads * head_dim, num_heads=heads, qk_norm=False)
    layer.q, layer.k, layer.v = _Feed(), _Feed(), _Feed()
    layer.o = torch.nn.Identity()
    layer.sink_size = sink_size
    layer.adapt_sink_thr = adapt_thr
    return layer


def ref_table(ref, head_dim):
    d = head_dim
    return torch.cat([ref.wm.rope_params(1024, d - 4 * (d // 6)),
                      ref.wm.rope_params(1024, 2 * (d // 6)),
                      ref.wm.rope_params(1024, 2 * (d // 6))], dim=1)


def run_kernel_case(ref, case: dict) -> dict:
    """Drive one CausalWanSelfAttention layer through a seeded call schedule."""
    H, D = case["heads"], case["head_dim"]
    dtype = cases.DTYPES[case["dtype"]]
    layer = make_ref_layer(ref, H, D, case["sink_size"], case["adapt_sink_thr"])
    table = ref_table(ref, D)
    h, w = case["grid_hw"]
    fs = h * w
    smax = case["cache_frames"] * fs
    rows = 1
    kv = {"k": torch.zeros(rows, smax, H, D, dtype=dtype), "v": torch.zeros(rows, smax, H, D, dtype=dtype),
          "global_end_index": torch.tensor([0], dtype=torch.long),
          "local_end_index": torch.tensor([0], dtype=torch.long),
          "total_steps": case["total_steps"], "current_step": case["total_steps"]}
    gen = cases.InputStream(case)
    steps = []
    for call in cases.schedule(case):
        if call["op"] == "replicate":          # what prepare() does after the first chunk
            b = call["rows"]
            kv["k"] = kv["k"].repeat(b, 1, 1, 1)
            kv["v"] = kv["v"].repeat(b, 1, 1, 1)
            kv["global_end_index"] = kv["global_end_index"].repeat(b)
            kv["local_end_index"] = kv["local_end_index"].repeat(b)
            rows = b
            continue
        starts, frames = call["starts"], call["frames"]
        q, k, v = gen.next(len(starts), frames * fs)
        layer.q.value, layer.k.value, layer.v.value = (t.flatten(2) for t in (q, k, v))
        grid = torch.tensor([[frames, h, w]] * len(starts), dtype=torch.long)
        cs = torch.tensor(starts, dtype=torch.long)
        x = torch.zeros(len(starts), frames * fs, H * D, dtype=dtype)
        with torch.no_grad():
            out = layer(x, None, grid, table, None, kv, cs, cs + frames * fs)
        steps.append({
            "in_sha": cases.sha(torch.stack([q, k, v])),
            "k_sha": cases.sha(kv["k"]), "v_sha": cases.sha(kv["v"]),
            "global_end": kv["global_end_index"].tolist(), "local_end": kv["local_end_index"].tolist(),
            "evict_idx": [list(map(int, r)) for r in layer.evict_idx],
            "current_step": int(kv["current_step"]),
            "out": out.view(len(starts), frames * fs, H, D),
        })
    return {"steps": steps}


def run_cross_case(ref, case: dict) -> dict:
    H, D = case["heads"], case["head_dim"]
    dtype = cases.DTYPES[case["dtype"]]
    g = torch.Generator().manual_seed(case["seed"])
    q = torch.randn(case["rows"], case["n"], H, D, generator=g).to(dtype)
    k = torch.randn(1, case["lk"], H, D, generator=g).to(dtype).expand(case["rows"], -1, -1, -1)
    v = torch.randn(1, case["lk"], H, D, generator=g).to(dtype).expand(case["rows"], -1, -1, -1)
    out = ref.att.flash_attention(q, k, v, k_lens=None)
    return {"in_sha": cases.sha(q), "out": out}


def save_case(path: str, res: dict):
    meta, arrays = {"steps": []}, {}
    if "steps" in res:
        for i, st in enumerate(res["steps"]):
            out = st.pop("out")
            arrays[f"out_{i}"] = cases.to_numpy_bits(out)
            st["out_dtype"] = str(out.dtype)
            st["out_shape"] = list(out.shape)
            meta["steps"].append(st)
    else:
        out = res.pop("out")
        arrays["out"] = cases.to_numpy_bits(out)
        res["out_dtype"] = str(out.dtype)
        res["out_shape"] = list(out.shape)
        meta = res
    np.savez_compressed(path, meta=np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8), **arrays)


def run_trace_case(ref, case: dict) -> dict:
    """Index-state trace at production token counts (tiny heads so it stays cheap)."""
    res = run_kernel_case(ref, case)
    for st in res["steps"]:
        st.pop("out")
        st.pop("k_sha")
        st.pop("v_sha")
        st.pop("in_sha")
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SDV2_REFERENCE"), required="SDV2_REFERENCE" not in os.environ)
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    ref = import_reference(args.reference)
    torch.set_num_threads(os.cpu_count() or 1)
    for name, case in cases.KERNEL_CASES.items():
        if args.only and args.only not in name:
            continue
        save_case(os.path.join(HERE, f"{name}.npz"), run_kernel_case(ref, case))
        print("wrote", name)
    for name, case in cases.CROSS_CASES.items():
        if args.only and args.only not in name:
            continue
        save_case(os.path.join(HERE, f"{name}.npz"), run_cross_case(ref, case))
        print("wrote", name)
    traces = {}
    for name, case in cases.TRACE_CASES.items():
        if args.only and args.only not in name:
            continue
        traces[name] = run_trace_case(ref, case)["steps"]
        print("traced", name)
    if traces:
        p = os.path.join(HERE, "index_traces.json")
        old = json.load(open(p)) if os.path.exists(p) else {}
        old.update(traces)
        json.dump(old, open(p, "w"))
    if not args.only or "model" in args.only:
        import make_golden_model
        make_golden_model.generate(ref, HERE)


if __name__ == "__main__":
    main()

"""Model-level fixtures: the reference's own CausalWanModel + CausalStreamInferencePipeline on a
tiny seeded model (CPU, fp32).  Called from make_golden.py."""
from __future__ import annotations

import os

import numpy as np
import torch

import cases


def build_reference_pipeline(ref, case, block_mode="input", device="cpu", dtype=torch.float32):
    """The reference's own pipeline objects for a model case (oracle/reference_shim.py)."""
    from oracle.reference_shim import build_reference_pipeline as _build
    prompt, first, chunks = cases.model_inputs(case)
    h, w = case["latent_hw"]
    return _build(ref, cases.MODEL_KW, case["levels"], (h // 2) * (w // 2), case["cache_frames"], case["sink"],
                  case["frames"], prompt, device=device, dtype=dtype, init_parameters=cases.seed_parameters)


def snapshot(pipe, layer):
    kv = pipe.kv_cache1[layer]
    mod = pipe.generator.model.blocks[layer].self_attn
    return {"global_end": kv["global_end_index"].tolist(), "local_end": kv["local_end_index"].tolist(),
            "evict_idx": [list(map(int, r)) for r in mod.evict_idx], "current_step": int(kv["current_step"]),
            "k_sha": cases.sha(kv["k"]), "v_sha": cases.sha(kv["v"])}


def run_stream(ref, case):
    pipe = build_reference_pipeline(ref, case)
    prompt, first, chunks = cases.model_inputs(case)
    fs, sched = cases.model_schedule(case)
    torch.manual_seed(case["seed"] + 1)
    arrays, meta = {}, {"steps": []}
    with torch.no_grad():
        out0 = pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                            current_start=0, current_end=fs * (1 + case["frames"]))
        arrays["prepare"] = out0.numpy().copy()
        meta["prepare"] = {"layer0": snapshot(pipe, 0), "layerL": snapshot(pipe, len(pipe.kv_cache1) - 1)}
        for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
            hs = pipe.inference_stream(noise=noise, current_start=cs, current_end=ce, current_step=None)
            arrays[f"out_{i}"] = hs.numpy().copy()
            meta["steps"].append({"layer0": snapshot(pipe, 0), "layerL": snapshot(pipe, len(pipe.kv_cache1) - 1)})
    return meta, arrays


def run_stages(ref, case):
    """Two pipeline stages in one process: stage A owns blocks [0, split), stage B the rest."""
    split = case["split"]
    nblk = cases.MODEL_KW["num_layers"]
    pa = build_reference_pipeline(ref, case)
    pb = build_reference_pipeline(ref, case)
    prompt, first, chunks = cases.model_inputs(case)
    fs, sched = cases.model_schedule(case)
    arrays, meta = {}, {"steps": []}
    with torch.no_grad():
        for pipe, mode, rng in ((pa, "input", [0, split]), (pb, "output", [split, nblk])):
            torch.manual_seed(case["seed"] + 1)
            pipe.prepare(text_prompts=["p"], device=torch.device("cpu"), dtype=torch.float32, noise=first,
                         current_start=0, current_end=fs * (1 + case["frames"]), block_mode=mode)
        torch.manual_seed(case["seed"] + 2)
        world = 2
        returns = []     # what the last stage sent back for every chunk: (latents, starts, ends)
        for i, (noise, (cs, ce)) in enumerate(zip(chunks, sched)):
            # stage 0 adopts the packet that came back from chunk i - world before running chunk i
            # (streamv2v/inference_pipe.py:583-634: receive once `processed >= world_size`, copy into
            # the pipeline state after the send)
            if i >= world:
                lat, st, en = returns[i - world]
                pa.hidden_states.copy_(lat)
                pa.kv_cache_starts.copy_(st)
                pa.kv_cache_ends.copy_(en)
            act, pshape = pa.inference(noise=noise, current_start=cs, current_end=ce, current_step=None,
                                       block_mode="input", block_num=torch.tensor([0, split]))
            sent_starts, sent_ends = pa.kv_cache_starts.clone(), pa.kv_cache_ends.clone()
            den, _ = pb.inference(noise=pa.hidden_states.clone(), current_start=sent_starts,
                                  current_end=sent_ends, current_step=None, block_mode="output",
                                  block_num=torch.tensor([split, nblk]), patched_x_shape=pshape, block_x=act)
            returns.append((den.clone(), sent_starts, sent_ends))
            arrays[f"act_{i}"] = act.numpy().copy()
            arrays[f"out_{i}"] = den.numpy().copy()
            meta["steps"].append({"stageA_layer0": snapshot(pa, 0), "stageB_layerL": snapshot(pb, nblk - 1),
                                  "pshape": pshape.tolist(), "starts": sent_starts.tolist(),
                                  "ends": sent_ends.tolist()})
    return meta, arrays


def generate(ref, here):
    import json
    for name, case in cases.MODEL_CASES.items():
        meta, arrays = (run_stages if "split" in case else run_stream)(ref, case)
        np.savez_compressed(os.path.join(here, f"{name}.npz"),
                            meta=np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8), **arrays)
        print("wrote", name)

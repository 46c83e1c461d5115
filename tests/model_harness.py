"""Builds the package's model + streaming scheduler for a model-level golden case."""
import torch

import cases


def build_pipeline(case, device="cpu", dtype=torch.float32, adapt_sink_threshold=-1):
    from streamdiffusionv2_b200.stream_pipeline import DiffusionWrapper, StreamPipeline
    from streamdiffusionv2_b200.wan_model import CausalWanModel

    model = CausalWanModel(**cases.MODEL_KW)
    cases.seed_parameters(model)
    model = model.to(device=device, dtype=dtype).eval()
    prompt, first, chunks = cases.model_inputs(case)
    wrapper = DiffusionWrapper(model)
    h, w = case["latent_hw"]
    pipe = StreamPipeline(wrapper, lambda text_prompts: {"prompt_embeds": prompt.clone().to(device=device, dtype=dtype)},
                          case["levels"], cases.MODEL_KW["num_layers"], cases.MODEL_KW["num_heads"],
                          (h // 2) * (w // 2), case["cache_frames"], case["sink"], adapt_sink_threshold, case["frames"],
                          device=device)
    return pipe, first.to(device=device, dtype=dtype), [c.to(device=device, dtype=dtype) for c in chunks]


def snapshot(pipe, layer):
    from streamdiffusionv2_b200.ring_state import RingState
    kv = pipe.kv_cache1[layer]
    mod = pipe.generator.model.blocks[layer].self_attn
    RingState.sync_queue(mod)          # with the adaptive sink test the queue lives on the device
    return {"global_end": kv["global_end_index"].tolist(), "local_end": kv["local_end_index"].tolist(),
            "evict_idx": [list(map(int, r)) for r in mod.evict_idx], "current_step": int(kv["current_step"]),
            "k_sha": cases.sha(kv["k"]), "v_sha": cases.sha(kv["v"])}

"""Imports the UNMODIFIED reference implementation and builds its own streaming pipeline objects.

TEST INFRASTRUCTURE ONLY (like everything under oracle/): used by the fixture generators under
tests/golden/, by the tests that run the reference's classes, and by the benchmark's comparison
arm.  Nothing in the shipped package imports this module.

`root` is either the reference checkout or a directory the reference was pip-installed into
(`pip install --no-deps --target <dir> <checkout>`); both hold the `models/` and `streamv2v/`
packages.  Two packages the reference imports at module level are not installed here and are not
used on the attention path (`diffusers`, `ftfy`); they are replaced by empty stand-ins.
"""
from __future__ import annotations

import os
import sys
import types

import torch


def reference_root(candidates=None):
    """First existing directory that holds the reference's `models/wan` package, or None."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for c in candidates or (os.environ.get("SDV2_REFERENCE"), os.path.join(here, "baseline", "_ref")):
        if c and os.path.isdir(os.path.join(c, "models", "wan")):
            return c
    return None


def import_reference(root: str, flash_attn: bool = False):
    """Import the reference's modules from `root`.  flash_attn=False forces its own PyTorch
    attention paths (models/wan/causal_model.py:373-384, wan_base/modules/attention.py:168-185),
    which is what a machine without the optional flash-attn extra runs; True leaves the flags as
    the import found them (flash-attn where installed)."""
    sys.dont_write_bytecode = True

    def stub(name, **attrs):
        if name in sys.modules and not getattr(sys.modules[name], "_sdv2_stub", False):
            return                        # the real package is installed: use it
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        m._sdv2_stub = True
        sys.modules[name] = m

    class ConfigMixin:
        pass

    class ModelMixin(torch.nn.Module):
        pass

    stub("diffusers")
    stub("diffusers.configuration_utils", ConfigMixin=ConfigMixin, register_to_config=lambda f: f)
    stub("diffusers.models")
    stub("diffusers.models.modeling_utils", ModelMixin=ModelMixin)
    stub("diffusers.utils", export_to_video=lambda *a, **k: None)
    stub("ftfy", fix_text=lambda s: s)
    if root not in sys.path:
        sys.path.insert(0, root)
    import models.wan.causal_model as cm
    import models.wan.wan_base.modules.attention as att
    import models.wan.wan_base.modules.model as wm
    import models.wan.causal_stream_inference as csi
    import models.wan.wan_wrapper as ww
    import models.wan.flow_match as fm
    ns = types.SimpleNamespace(cm=cm, att=att, wm=wm, csi=csi, ww=ww, fm=fm, root=root)
    if not hasattr(cm, "_sdv2_found_flags"):
        cm._sdv2_found_flags = (cm.FLASH_ATTN_AVAILABLE, att.FLASH_ATTN_2_AVAILABLE, att.FLASH_ATTN_3_AVAILABLE)
    set_flash_attn(ns, flash_attn)
    return ns


def set_flash_attn(ref, enabled: bool) -> None:
    """Switch the reference between its flash-attn calls (as found at import) and its PyTorch paths."""
    found = ref.cm._sdv2_found_flags
    ref.cm.FLASH_ATTN_AVAILABLE = found[0] if enabled else False
    ref.att.FLASH_ATTN_2_AVAILABLE = found[1] if enabled else False
    ref.att.FLASH_ATTN_3_AVAILABLE = found[2] if enabled else False


def build_reference_pipeline(ref, model_kw: dict, levels, frame_seq_length: int, cache_frames: int, sink: int,
                             frames_per_chunk: int, prompt: torch.Tensor, device="cpu", dtype=torch.float32,
                             init_parameters=None, construct_on_device: bool = False):
    """The reference's CausalWanModel + CausalWanDiffusionWrapper + CausalStreamInferencePipeline,
    constructed without their checkpoint / text-encoder / VAE loading (object.__new__ plus the
    attributes their __init__ would set: models/wan/causal_stream_inference.py:37-70,
    models/wan/wan_wrapper.py:161-169).  `init_parameters(model)` seeds the weights;
    `construct_on_device` creates the parameters on `device` directly (a billion-parameter model
    takes a while to initialise on the host)."""
    device = torch.device(device)
    if construct_on_device:
        with torch.device(device):
            model = ref.cm.CausalWanModel(**model_kw)
    else:
        model = ref.cm.CausalWanModel(**model_kw)
    if init_parameters is not None:
        init_parameters(model)
    model = model.to(device=device, dtype=dtype).eval()
    wrapper = ref.ww.CausalWanDiffusionWrapper.__new__(ref.ww.CausalWanDiffusionWrapper)
    torch.nn.Module.__init__(wrapper)
    wrapper.model = model
    wrapper.uniform_timestep = False
    wrapper.scheduler = ref.fm.FlowMatchScheduler(shift=8.0, sigma_min=0.0, extra_one_step=True)
    wrapper.scheduler.set_timesteps(1000, training=True)
    wrapper.seq_len = 32760
    wrapper.post_init()

    pipe = ref.csi.CausalStreamInferencePipeline.__new__(ref.csi.CausalStreamInferencePipeline)
    torch.nn.Module.__init__(pipe)
    pipe.device = device
    pipe.generator = wrapper
    pipe.text_encoder = lambda text_prompts: {"prompt_embeds": prompt.clone().to(device=device, dtype=dtype)}
    pipe.scheduler = wrapper.get_scheduler()
    pipe.denoising_step_list = torch.tensor(list(levels), dtype=torch.long, device=device)
    pipe.num_transformer_blocks = model_kw["num_layers"]
    pipe.num_heads = model_kw["num_heads"]
    pipe.frame_seq_length = frame_seq_length
    pipe.num_kv_cache = cache_frames
    pipe.kv_cache_length = pipe.frame_seq_length * pipe.num_kv_cache
    pipe.num_sink_tokens = sink
    pipe.adapt_sink_threshold = -1
    pipe.num_frame_per_block = frames_per_chunk
    model.num_frame_per_block = frames_per_chunk
    pipe.conditional_dict = None
    pipe.kv_cache1 = pipe.kv_cache2 = pipe.hidden_states = pipe.block_x = None
    pipe.args = types.SimpleNamespace()
    return pipe

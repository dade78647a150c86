"""Run the reference's own model and pipeline code, unmodified, around this package's operators.

The harness imports ``wan/modules/causal_model.py``, ``utils/wan_wrapper.py`` and
``pipeline/causal_inference.py`` from a staged checkout (``baseline/_ref/``, see
``baseline/stage_reference.py``, or ``SF_REFERENCE_ROOT``) and builds what BASELINE's full-model
configurations describe: a random-init causal Wan DiT, a 21-frame latent generated in 7 chunks of 3
frames with 4 denoising steps per chunk, a random 512x4096 text context through cross-attention.

What is replaced, and only by registering modules before the reference files are imported:

* packages the reference imports at module scope that are not installed here and that the causal
  rollout never calls (``diffusers`` mixins, ``cuvs``, ``matplotlib``, ``ftfy``, ``loguru``): inert stand-ins;
* the heavy package ``__init__`` files (``wan/__init__.py`` pulls the upstream samplers): bare
  namespace packages that only carry the search path;
* with ``attention="ours"``: ``wan.modules.monarch_attn`` and ``wan.modules.attention`` by this
  package's operators (``install_into_reference``), and optionally the cache branch of
  ``CausalWanSelfAttention.forward`` (``patch_self_attention_forward``).

``from_pretrained`` is bypassed (no weights exist here): the wrapper object is assembled by hand
around ``CausalWanModel(dim=..., ...)`` the way ``WanDiffusionWrapper.__init__``
(utils/wan_wrapper.py:117-145) does after loading.  Text encoder and VAE are stand-ins: a callable
that returns a seeded random ``prompt_embeds`` and an object whose ``decode_to_pixel`` returns its input.
"""
from __future__ import annotations

import contextlib
import io
import os
import re
import sys
import types
from pathlib import Path
from types import SimpleNamespace
from typing import Optional

HERE = Path(__file__).resolve().parent

MODEL_SHAPES = {
    # wan/configs/wan_t2v_1_3B.py:20-29, wan_t2v_14B.py:20-29
    "1.3b": dict(dim=1536, ffn_dim=8960, num_heads=12, num_layers=30),
    "14b": dict(dim=5120, ffn_dim=13824, num_heads=40, num_layers=40),
}

BLOCKING_ENV = {
    # environment read by CausalWanSelfAttention.__init__ (causal_model.py:739-763)
    "framewise": {"MONARCH_ATTN_FRAMEWISE": "1", "MONARCH_ATTN_H_REDUCE": "1", "MONARCH_ATTN_W_REDUCE": "1"},
    "tied3frame": {"MONARCH_ATTN_FRAMEWISE": "0", "MONARCH_ATTN_H_REDUCE": "1", "MONARCH_ATTN_W_REDUCE": "1"},
    "reduce2xh": {"MONARCH_ATTN_FRAMEWISE": "1", "MONARCH_ATTN_H_REDUCE": "2", "MONARCH_ATTN_W_REDUCE": "1"},
    "reduce4xw2xh": {"MONARCH_ATTN_FRAMEWISE": "1", "MONARCH_ATTN_H_REDUCE": "2", "MONARCH_ATTN_W_REDUCE": "4"},
    "dense": {"DISABLE_MONARCH_ATTN": "1"},
}
_ENV_KEYS = ["MONARCH_ATTN_FRAMEWISE", "MONARCH_ATTN_H_REDUCE", "MONARCH_ATTN_W_REDUCE", "MONARCH_ATTN_NUM_ITERS",
             "DISABLE_MONARCH_ATTN", "USE_DENSE_INIT"]


def reference_root() -> Optional[Path]:
    """Where the reference sources are: ``SF_REFERENCE_ROOT`` if set, else the staged copy, else None."""
    env = os.environ.get("SF_REFERENCE_ROOT")
    for cand in ([Path(env)] if env else []) + [HERE / "_ref"]:
        if (cand / "wan" / "modules" / "causal_model.py").is_file():
            return cand
    return None


def _stub(name: str, **attrs) -> types.ModuleType:
    mod = types.ModuleType(name)
    mod.__dict__.update(attrs)
    sys.modules[name] = mod
    parent, _, leaf = name.rpartition(".")
    if parent and parent in sys.modules:
        setattr(sys.modules[parent], leaf, mod)
    return mod


def _missing(name: str) -> bool:
    import importlib.util
    try:
        return importlib.util.find_spec(name) is None
    except (ImportError, ValueError):
        return True


def _register_stand_ins(cuda: bool) -> None:
    import torch
    from torch import nn

    if _missing("diffusers"):
        class ConfigMixin:
            pass

        def register_to_config(fn):
            return fn

        class ModelMixin(nn.Module):
            pass

        _stub("diffusers")
        _stub("diffusers.configuration_utils", ConfigMixin=ConfigMixin, register_to_config=register_to_config)
        _stub("diffusers.models")
        _stub("diffusers.models.modeling_utils", ModelMixin=ModelMixin)
    if _missing("cuvs"):
        _stub("cuvs")
        _stub("cuvs.cluster")
        _stub("cuvs.cluster.kmeans", KMeansParams=object, fit=None)
    if _missing("matplotlib"):
        _stub("matplotlib")
        _stub("matplotlib.pyplot")
    if _missing("ftfy"):
        _stub("ftfy", fix_text=lambda s: s)
    if _missing("loguru"):
        import logging
        _stub("loguru", logger=logging.getLogger("loguru-stand-in"))
    if _missing("fastvideo_kernel"):
        pass                                   # imported under try/except by the reference
    if not cuda:
        # these evaluate torch.cuda.current_device() at import; the rollout uses nothing of them
        _stub("demo_utils")
        _stub("demo_utils.memory", gpu=torch.device("cpu"), get_cuda_free_memory_gb=lambda *_: 0.0,
              DynamicSwapInstaller=object, move_model_to_device_with_memory_preservation=lambda *a, **k: None)


def prepare_imports(root: Path, attention: str = "ours", replace_dense: bool = True) -> None:
    """Make ``wan.modules.causal_model``, ``utils.wan_wrapper`` and ``pipeline.causal_inference`` importable
    from ``root``.  ``attention``: "ours" (this package's operators) or "reference" (the reference's own
    Triton / flash-attn path, needs a GPU)."""
    import torch
    if attention not in ("ours", "reference"):
        raise ValueError("attention must be 'ours' or 'reference'")
    root = Path(root)
    cuda = torch.cuda.is_available()
    _register_stand_ins(cuda)
    for name, sub in (("wan", "wan"), ("wan.modules", "wan/modules"), ("pipeline", "pipeline"), ("utils", "utils"),
                      ("demo_utils", "demo_utils")):
        if name in sys.modules and not hasattr(sys.modules[name], "__path__"):
            continue
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__path__ = [str(root / sub)]
            sys.modules[name] = mod
            parent, _, leaf = name.rpartition(".")
            if parent:
                setattr(sys.modules[parent], leaf, mod)
    if not cuda:
        # wan/modules/t5.py evaluates torch.cuda.current_device() in a class body
        _stub("wan.modules.t5", umt5_xxl=None)
    if attention == "ours":
        import self_forcing_b200 as sfb
        sfb.install_into_reference(replace_dense=replace_dense)


def build_generator(model: str = "1.3b", device="cuda", dtype=None, seed: int = 0, **overrides):
    """A ``WanDiffusionWrapper`` around a random-init ``CausalWanModel`` (its own ``init_weights``, plus a
    seeded normal head so that outputs are not identically zero), assembled without ``from_pretrained``."""
    import torch
    from torch import nn
    from utils.scheduler import FlowMatchScheduler
    from utils.wan_wrapper import WanDiffusionWrapper
    from utils.resolution import total_seq_len
    from wan.modules.causal_model import CausalWanModel

    dtype = dtype or torch.bfloat16
    shape = dict(MODEL_SHAPES[model]) if isinstance(model, str) else dict(model)
    shape.update(overrides)
    torch.manual_seed(seed)
    with torch.device(device):                       # initialise on the target device (14B on the host takes minutes)
        net = CausalWanModel(model_type="t2v", patch_size=(1, 2, 2), text_len=512, in_dim=16, freq_dim=256,
                             text_dim=4096, out_dim=16, qk_norm=True, cross_attn_norm=True, eps=1e-6, **shape)
        nn.init.normal_(net.head.head.weight, std=0.02)
    net = net.to(device=device, dtype=dtype).eval().requires_grad_(False)
    gen = object.__new__(WanDiffusionWrapper)
    nn.Module.__init__(gen)
    gen.model = net
    gen.uniform_timestep = False
    gen.scheduler = FlowMatchScheduler(shift=5.0, sigma_min=0.0, extra_one_step=True)
    gen.scheduler.set_timesteps(1000, training=True)
    gen.seq_len = total_seq_len
    gen.post_init()
    return gen


class RandomTextEncoder:
    """Stands in for WanTextEncoder: a seeded N(0,1) context of the encoder's output shape."""

    def __init__(self, device, dtype, seed: int = 1):
        self.device, self.dtype, self.seed = device, dtype, seed

    def __call__(self, text_prompts):
        import torch
        g = torch.Generator(device="cpu").manual_seed(self.seed)
        e = torch.randn(len(text_prompts), 512, 4096, generator=g)
        return {"prompt_embeds": e.to(device=self.device, dtype=self.dtype)}


class IdentityVAE:
    def decode_to_pixel(self, latents, use_cache=False):
        return latents


def build_pipeline(model: str = "1.3b", blocking: str = "framewise", device="cuda", dtype=None, num_iters: int = 1,
                   dense_init: bool = False, seed: int = 0, sequence_parallel: bool = False,
                   exchange: str = "all_to_all", **overrides):
    """``CausalInferencePipeline`` (pipeline/causal_inference.py:13-49) with the 4-step schedule of the
    reference's inference configs.  The Monarch environment is set before the model is constructed
    (it is read in ``CausalWanSelfAttention.__init__``)."""
    import torch
    for k in _ENV_KEYS:
        os.environ.pop(k, None)
    os.environ.update(BLOCKING_ENV[blocking])
    os.environ["MONARCH_ATTN_NUM_ITERS"] = str(int(num_iters))
    if dense_init:
        os.environ["USE_DENSE_INIT"] = "1"
    from pipeline.causal_inference import CausalInferencePipeline
    dtype = dtype or torch.bfloat16
    gen = build_generator(model, device=device, dtype=dtype, seed=seed, **overrides)
    if sequence_parallel:
        # one video over all ranks: tokens sharded outside attention, heads inside (weights replicated);
        # the reference's wrapper and pipeline stay as they are, the model object is wrapped
        import torch.distributed as dist
        from self_forcing_b200.sequence_parallel import (SequenceParallelCausalWan, SequenceParallelModelAdapter,
                                                         head_sharded_kv_cache)
        ft = 1 if BLOCKING_ENV[blocking].get("MONARCH_ATTN_FRAMEWISE") == "1" else 3
        blk = (ft, int(BLOCKING_ENV[blocking].get("MONARCH_ATTN_H_REDUCE", 1)),
               int(BLOCKING_ENV[blocking].get("MONARCH_ATTN_W_REDUCE", 1)))
        net = gen.model
        gen.model = SequenceParallelModelAdapter(net, SequenceParallelCausalWan(net, blk, num_iters=num_iters,
                                                                                   exchange=exchange))
    args = SimpleNamespace(denoising_step_list=[1000, 750, 500, 250], warp_denoising_step=True,
                           independent_first_frame=False, num_frame_per_block=3, context_noise=0)
    with contextlib.redirect_stdout(io.StringIO()):
        pipe = CausalInferencePipeline(args, device, generator=gen, text_encoder=RandomTextEncoder(device, dtype),
                                       vae=IdentityVAE())
    if sequence_parallel:
        from utils.resolution import total_seq_len

        def _initialize_kv_cache(batch_size, dtype, device, _pipe=pipe):
            _pipe.kv_cache1 = head_sharded_kv_cache(net, batch_size, total_seq_len, dist.get_world_size(), device, dtype)
        pipe._initialize_kv_cache = _initialize_kv_cache
    return pipe


_BLOCK_RE = re.compile(r"Block (\d+) generation time: ([0-9.]+) ms")
_DIFF_RE = re.compile(r"Diffusion generation time: ([0-9.]+) ms")


def run_rollout(pipe, batch: int = 1, frames: int = 21, seed: int = 2, device="cuda", dtype=None):
    """One ``inference(profile=True)`` call on seeded noise; the chunk times are the pipeline's own CUDA
    events, read from what it prints.  Returns (latents, {"block_ms": [...], "diffusion_ms": x})."""
    import torch
    dtype = dtype or torch.bfloat16
    g = torch.Generator(device="cpu").manual_seed(seed)
    noise = torch.randn(batch, frames, 16, 60, 104, generator=g).to(device=device, dtype=dtype)
    # the pipeline re-seeds the noise it adds between denoising steps from a list walked by a module-level
    # counter (pipeline/causal_inference.py:10-11, 213-214): start every rollout at its beginning
    mod = sys.modules.get(type(pipe).__module__)
    if mod is not None and hasattr(mod, "seed_count"):
        mod.seed_count = 0
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf), torch.no_grad():
        video, latents = pipe.inference(noise=noise, text_prompts=["synthetic"] * batch, return_latents=True,
                                        profile=torch.cuda.is_available())
    text = buf.getvalue()
    blocks = [float(m.group(2)) for m in _BLOCK_RE.finditer(text)]
    diff = _DIFF_RE.search(text)
    return latents, {"block_ms": blocks, "diffusion_ms": float(diff.group(1)) if diff else None}


def allocate_caches(gen, batch: int, device, dtype, cache_frames: int = 21):
    """Per-layer KV and cross-attention caches in the pipelines' layout
    (pipeline/causal_inference.py:288-321, pipeline/causal_diffusion_inference.py:272-330)."""
    import torch
    from utils.resolution import frame_height, frame_width
    net = gen.model
    heads, hd = net.num_heads, net.dim // net.num_heads
    n = cache_frames * frame_height * frame_width
    kv = [{"k": torch.zeros(batch, n, heads, hd, dtype=dtype, device=device),
           "v": torch.zeros(batch, n, heads, hd, dtype=dtype, device=device),
           "global_end_index": torch.tensor([0], dtype=torch.long, device=device),
           "local_end_index": torch.tensor([0], dtype=torch.long, device=device)} for _ in range(net.num_layers)]
    cross = [{"k": torch.zeros(batch, 512, heads, hd, dtype=dtype, device=device),
              "v": torch.zeros(batch, 512, heads, hd, dtype=dtype, device=device), "is_init": False}
             for _ in range(net.num_layers)]
    return kv, cross


def run_cfg_rollout(gen, frames: int = 6, solver_steps: int = 3, guidance_scale: float = 3.0, batch: int = 1,
                    seed: int = 5, device="cuda", dtype=None):
    """The call pattern of the reference's many-step sampler with classifier-free guidance
    (pipeline/causal_diffusion_inference.py:100-262) around the reference's own generator: two KV caches
    and two cross-attention caches (conditional / unconditional), per chunk ``solver_steps`` times a
    conditional and an unconditional forward at the same cache position, then one clean-context forward into
    each cache.  The solver itself (UniPC there) is replaced by a plain Euler step of the flow: it is scalar
    arithmetic on the latents and does not touch the attention path.  Returns (latents, kv_pos, kv_neg)."""
    import torch
    from utils.resolution import frame_height, frame_width
    dtype = dtype or torch.bfloat16
    g = torch.Generator(device="cpu").manual_seed(seed)
    noise = torch.randn(batch, frames, 16, 60, 104, generator=g).to(device=device, dtype=dtype)
    enc = RandomTextEncoder(device, dtype, seed=seed + 1)
    cond = enc(["synthetic"] * batch)
    uncond = RandomTextEncoder(device, dtype, seed=seed + 2)(["negative"] * batch)
    kv_pos, cross_pos = allocate_caches(gen, batch, device, dtype)
    kv_neg, cross_neg = allocate_caches(gen, batch, device, dtype)
    frame_tokens = frame_height * frame_width
    out = torch.zeros_like(noise)
    sigmas = torch.linspace(1.0, 0.0, solver_steps + 1)
    with torch.no_grad():
        for c0 in range(0, frames, 3):
            latents = noise[:, c0:c0 + 3]
            start = c0 * frame_tokens
            for i in range(solver_steps):
                t = torch.full([batch, 3], float(sigmas[i]) * 1000.0, device=device, dtype=torch.float32)
                f_c, _ = gen(noisy_image_or_video=latents, conditional_dict=cond, timestep=t, kv_cache=kv_pos,
                             crossattn_cache=cross_pos, current_start=start, cache_start=start)
                f_u, _ = gen(noisy_image_or_video=latents, conditional_dict=uncond, timestep=t, kv_cache=kv_neg,
                             crossattn_cache=cross_neg, current_start=start, cache_start=start)
                flow = f_u + guidance_scale * (f_c - f_u)
                latents = (latents.float() + (float(sigmas[i + 1]) - float(sigmas[i])) * flow.float()).to(dtype)
            out[:, c0:c0 + 3] = latents
            t0 = torch.zeros([batch, 3], device=device, dtype=torch.float32)
            gen(noisy_image_or_video=latents, conditional_dict=cond, timestep=t0, kv_cache=kv_pos,
                crossattn_cache=cross_pos, current_start=start, cache_start=start)
            gen(noisy_image_or_video=latents, conditional_dict=uncond, timestep=t0, kv_cache=kv_neg,
                crossattn_cache=cross_neg, current_start=start, cache_start=start)
    return out, kv_pos, kv_neg

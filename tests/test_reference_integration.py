"""This package inside the reference's own model code.

Needs the reference sources (``SF_REFERENCE_ROOT``, or the copy ``baseline/stage_reference.py`` stages
under ``baseline/_ref/``); every test here skips when they are absent.  The CPU tests check the drop-in
boundary itself: after ``install_into_reference()`` the reference's ``causal_model`` module binds this
package's functions, and their signatures equal the ones in the reference source.  The GPU tests run the
reference's ``CausalWanSelfAttention`` and its whole causal DiT on this package's kernels.
"""
import ast
import inspect
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "baseline"))
import reference_harness as rh  # noqa: E402

REF = rh.reference_root()
pytestmark = pytest.mark.skipif(REF is None, reason="reference sources not staged (baseline/stage_reference.py)")


@pytest.fixture(scope="module")
def causal_model():
    """wan.modules.causal_model imported from the reference with this package installed underneath; every
    module the import added is removed again afterwards so that other tests see a clean interpreter."""
    before = set(sys.modules)
    env = {k: os.environ.get(k) for k in rh._ENV_KEYS}
    rh.prepare_imports(REF, attention="ours")
    import wan.modules.causal_model as cm
    yield cm
    for name in set(sys.modules) - before:
        if name.split(".")[0] in ("wan", "utils", "pipeline", "demo_utils", "diffusers", "cuvs", "matplotlib", "ftfy",
                                  "loguru"):
            sys.modules.pop(name, None)
    for k, v in env.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


def _signature_from_source(path: Path, name: str):
    """(argument names, number of defaults) of a top-level function, read from the source text."""
    for node in ast.parse(path.read_text()).body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            a = node.args
            defaults = [eval(ast.unparse(d), {"torch": torch}) for d in a.defaults]     # literals and torch dtypes
            return [x.arg for x in a.posonlyargs + a.args], len(a.defaults), defaults
    raise AssertionError(f"{name} not found in {path}")


@pytest.mark.parametrize("rel,name,attr", [
    ("wan/modules/monarch_attn.py", "monarch_attn_with_kv_cache", "monarch_attn_with_kv_cache"),
    ("wan/modules/monarch_attn.py", "monarch_attn", "monarch_attn"),
    ("wan/modules/attention.py", "attention", "attention"),
    ("wan/modules/attention.py", "flash_attention", "flash_attention"),
    ("wan/modules/attn_patch.py", "full_attention_with_kv_cache", "full_attention_with_kv_cache"),
    ("wan/modules/causal_model.py", "causal_rope_apply", "causal_rope_apply"),
])
def test_signatures_equal_the_reference_source(rel, name, attr):
    import self_forcing_b200 as sfb
    names, n_def, defaults = _signature_from_source(REF / rel, name)
    sig = inspect.signature(getattr(sfb, attr))
    ours = [p for p in sig.parameters.values() if not p.name.startswith("_")]      # private keyword extras excluded
    assert [p.name for p in ours] == names
    ours_defaults = [p.default for p in ours if p.default is not inspect.Parameter.empty]
    assert len(ours_defaults) == n_def
    assert ours_defaults == defaults


def test_reference_module_binds_this_package(causal_model):
    import self_forcing_b200 as sfb
    cm = causal_model
    assert cm.monarch_attn_with_kv_cache is sfb.monarch_attn_with_kv_cache
    assert cm.monarch_attn is sfb.monarch_attn
    assert cm.attention is sfb.attention
    import wan.modules.model as wm
    assert wm.flash_attention is sfb.flash_attention          # cross-attention of the blocks
    # the file that was imported is the reference's, not a copy of ours
    assert Path(cm.__file__).resolve() == (REF / "wan/modules/causal_model.py").resolve()
    mod = cm.CausalWanSelfAttention(256, 2)
    assert mod.head_dim == 128 and isinstance(mod.norm_q, wm.WanRMSNorm)


def test_patched_forward_keeps_other_calls_on_the_original(causal_model):
    """patch_self_attention_forward on the real class: calls the fused path cannot serve (here: fp32 CPU
    tensors with stand-in operators) still go through the reference's own forward."""
    from self_forcing_b200.install import patch_self_attention_forward
    cm = causal_model
    cls = cm.CausalWanSelfAttention
    original = cls.forward
    seen = []
    saved = cm.monarch_attn_with_kv_cache

    def fake(q, kc, vc, nk, nv, s, e, *a, **k):
        seen.append((s, e, kc.shape[1]))
        return torch.zeros_like(q)
    try:
        cm.monarch_attn_with_kv_cache = fake
        patch_self_attention_forward(cls)
        assert cls.forward is not original and cls._sfm_original_forward is original
        os.environ["MONARCH_ATTN_FRAMEWISE"] = "1"
        mod = cls(256, 2)
        frame = 30 * 52
        kv = {"k": torch.zeros(1, 6 * frame, 2, 128), "v": torch.zeros(1, 6 * frame, 2, 128),
              "global_end_index": torch.tensor([0]), "local_end_index": torch.tensor([0])}
        freqs = torch.polar(torch.ones(1024, 64, dtype=torch.float64), torch.zeros(1024, 64, dtype=torch.float64))
        with torch.no_grad():
            for chunk in range(2):
                y = mod(torch.randn(1, 3 * frame, 256), torch.tensor([3 * frame]), torch.tensor([[3, 30, 52]]), freqs,
                        None, kv_cache=kv, current_start=chunk * 3 * frame)
        assert y.shape == (1, 3 * frame, 256)
        assert seen == [(0, 3 * frame, 3 * frame), (3 * frame, 6 * frame, 6 * frame)]
        assert int(kv["global_end_index"]) == 6 * frame and int(kv["local_end_index"]) == 6 * frame
    finally:
        cls.forward = original
        cm.monarch_attn_with_kv_cache = saved


# ------------------------------------------------------------------------------------------ GPU
def _rel_l2(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


@pytest.mark.gpu
@pytest.mark.parametrize("blocking", ["framewise", "reduce4xw2xh"])
def test_real_self_attention_module_on_gpu(causal_model, blocking):
    """The reference's CausalWanSelfAttention (dim 256, two heads) over a three-chunk rollout with rewrites:
    its own forward on this package's operators, against the patched forward (fused RMSNorm + RoPE + cache
    write, host-side indices).  Same weights, same inputs: outputs agree to bf16 rounding of the rotation
    (fp64 in the reference's RoPE, fp32 in the kernel), cache indices are equal."""
    from self_forcing_b200.install import patch_self_attention_forward
    cm = causal_model
    for k in rh._ENV_KEYS:
        os.environ.pop(k, None)
    os.environ.update(rh.BLOCKING_ENV[blocking])
    cls = cm.CausalWanSelfAttention
    original = cls.forward
    torch.manual_seed(3)
    mod = cls(256, 2).cuda().to(torch.bfloat16).eval()
    with torch.no_grad():
        mod.norm_q.weight.uniform_(0.5, 1.5)
        mod.norm_k.weight.uniform_(0.5, 1.5)
    frame = 30 * 52
    freqs = torch.cat([cm.rope_params(1024, 128 - 4 * (128 // 6)), cm.rope_params(1024, 2 * (128 // 6)),
                       cm.rope_params(1024, 2 * (128 // 6))], dim=1).cuda()
    grid = torch.tensor([[3, 30, 52]])
    xs = [torch.randn(1, 3 * frame, 256, device="cuda").to(torch.bfloat16) for _ in range(6)]

    def rollout():
        kv = {"k": torch.zeros(1, 9 * frame, 2, 128, device="cuda", dtype=torch.bfloat16),
              "v": torch.zeros(1, 9 * frame, 2, 128, device="cuda", dtype=torch.bfloat16),
              "global_end_index": torch.tensor([0], device="cuda"), "local_end_index": torch.tensor([0], device="cuda")}
        outs = []
        with torch.no_grad():
            for i, x in enumerate(xs):
                outs.append(mod(x, torch.tensor([3 * frame]), grid, freqs, None, kv_cache=kv,
                                current_start=(i // 2) * 3 * frame))
        torch.cuda.synchronize()
        return outs, kv
    ref_outs, ref_kv = rollout()
    try:
        patch_self_attention_forward(cls)
        got_outs, got_kv = rollout()
    finally:
        cls.forward = original
    for a, b in zip(got_outs, ref_outs):
        assert torch.isfinite(a).all()
        assert _rel_l2(a, b) <= 1e-2
    assert int(got_kv["global_end_index"]) == int(ref_kv["global_end_index"]) == 9 * frame
    assert int(got_kv["local_end_index"]) == int(ref_kv["local_end_index"]) == 9 * frame
    assert _rel_l2(got_kv["k"], ref_kv["k"]) <= 4e-3 and torch.equal(got_kv["v"], ref_kv["v"])


@pytest.mark.gpu
def test_whole_model_rollout_through_the_reference_pipeline(causal_model):
    """CausalInferencePipeline.inference (reference code, unmodified) over a two-block causal DiT at Wan-1.3B
    width, 6 latent frames: finite, non-trivial latents, every self-attention call served by this package's
    kernels, and the same latents again from the patched forward within bf16 noise."""
    from self_forcing_b200 import _lib
    from self_forcing_b200.install import patch_self_attention_forward
    cm = causal_model
    lib = _lib.load()
    pipe = rh.build_pipeline("1.3b", "framewise", device="cuda", num_layers=2)
    assert type(pipe).__module__ == "pipeline.causal_inference"
    n0 = lib.sfm_launch_count()
    lat, prof = rh.run_rollout(pipe, frames=6, device="cuda")
    assert lib.sfm_launch_count() - n0 >= 2 * 10 * 3            # 2 chunks x 5 forwards x 2 blocks x >= 3 kernels
    assert lat.shape == (1, 6, 16, 60, 104) and torch.isfinite(lat).all() and lat.float().std() > 0
    assert len(prof["block_ms"]) == 2 and prof["diffusion_ms"] > 0
    cls = cm.CausalWanSelfAttention
    original = cls.forward
    try:
        patch_self_attention_forward(cls)
        lat2, _ = rh.run_rollout(pipe, frames=6, device="cuda")
    finally:
        cls.forward = original
    assert _rel_l2(lat2, lat) <= 2e-2


@pytest.mark.gpu
def test_cfg_two_cache_rollout(causal_model):
    """Classifier-free guidance with two KV caches (the call pattern of the reference's many-step sampler):
    conditional and unconditional forwards alternate on the same stream at the same cache position, each into
    its own cache.  The reference's own forward on this package's operators and the patched forward must
    agree, and both caches must end at the same indices."""
    from self_forcing_b200.install import patch_self_attention_forward
    cm = causal_model
    for k in rh._ENV_KEYS:
        os.environ.pop(k, None)
    os.environ.update(rh.BLOCKING_ENV["framewise"])
    gen = rh.build_generator("1.3b", device="cuda", num_layers=2)
    lat, kv_pos, kv_neg = rh.run_cfg_rollout(gen, frames=6, solver_steps=3)
    cls = cm.CausalWanSelfAttention
    original = cls.forward
    try:
        patch_self_attention_forward(cls)
        lat2, kv_pos2, kv_neg2 = rh.run_cfg_rollout(gen, frames=6, solver_steps=3)
    finally:
        cls.forward = original
    torch.cuda.synchronize()
    assert torch.isfinite(lat).all() and lat.float().std() > 0
    assert _rel_l2(lat2, lat) <= 2e-2
    n = 6 * 30 * 52
    for a, b in ((kv_pos, kv_pos2), (kv_neg, kv_neg2)):
        for la, lb in zip(a, b):
            assert int(la["global_end_index"]) == int(lb["global_end_index"]) == n
            assert int(la["local_end_index"]) == int(lb["local_end_index"]) == n
            assert _rel_l2(lb["k"][:, :n], la["k"][:, :n]) <= 2e-2      # bf16 noise of the first block feeds the second
    # the two caches hold different keys (different text context flows into the later blocks)
    assert not torch.equal(kv_pos[1]["k"][:, :n], kv_neg[1]["k"][:, :n])

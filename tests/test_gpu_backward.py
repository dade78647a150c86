"""GPU parity tests of the Monarch attention backward kernels (through the C ABI) against autograd
through the CPU oracle's forward in fp32 on the same bf16-rounded inputs.

Tolerances: dq comes back in fp32 from fp32 arithmetic: relative L2 <= 2e-3; dk / dv are rounded to bf16 once:
relative L2 <= 1e-2 and max-abs <= 2e-2 of the largest reference magnitude (the forward's acceptance rule,
scaled to the gradient's range).
"""
import numpy as np
import pytest
import torch

import cases
from oracle import monarch_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sfb():
    import self_forcing_b200
    assert torch.cuda.is_available()
    return self_forcing_b200


def bf(x):
    return x.to(torch.bfloat16)


def grad_close(got, ref, rel_tol, what):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = ref.abs().max().clamp_min(1e-30).item()
    err = (got - ref).abs().max().item() / scale
    rel = ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert rel <= rel_tol and err <= 2e-2, f"{what}: rel-L2 {rel:.3e} max-abs/scale {err:.3e}"


def make_case(blocking, frames_q, groups_cached, B, H, seed):
    """Cache of `groups_cached` tied frame sets, the last `frames_q` of them written by this call."""
    ft, hr, wr, h, w = blocking
    rng = np.random.default_rng(seed)
    tied = ft * h * w
    n_q, n_kv = frames_q * tied, groups_cached * tied
    mk = lambda *s: bf(cases.randn(rng, *s))
    return dict(blocking=blocking, q=mk(B, n_q, H, 128), nk=mk(B, n_q, H, 128), nv=mk(B, n_q, H, 128),
                kbuf=mk(B, n_kv + tied, H, 128), vbuf=mk(B, n_kv + tied, H, 128), g=mk(B, n_q, H, 128),
                start=n_kv - n_q, end=n_kv, n_kv=n_kv, sm_scale=128 ** -0.5)


def oracle_grads(c):
    """Autograd through the oracle: gradients w.r.t. q, the cache content (Monarch order; zero where this call
    wrote) and new_k / new_v (natural order)."""
    q = c["q"].float().requires_grad_()
    nk, nv = c["nk"].float().requires_grad_(), c["nv"].float().requires_grad_()
    kb, vb = c["kbuf"].float().requires_grad_(), c["vbuf"].float().requires_grad_()
    kc, vc = kb.clone(), vb.clone()
    z = orc.monarch_attn_with_kv_cache(q, kc[:, :c["n_kv"]], vc[:, :c["n_kv"]], nk, nv, c["start"], c["end"],
                                       *c["blocking"], sm_scale=c["sm_scale"])
    (z * c["g"].float()).sum().backward()
    return dict(q=q.grad, nk=nk.grad, nv=nv.grad, kc=kb.grad[:, :c["n_kv"]], vc=vb.grad[:, :c["n_kv"]], z=z.detach())


def gpu_cache(sfb, c):
    dev = "cuda"
    kc, vc = c["kbuf"].to(dev).clone(), c["vbuf"].to(dev).clone()
    kv, vv = kc[:, :c["n_kv"]], vc[:, :c["n_kv"]]
    with torch.no_grad():
        z = sfb.monarch_attn_with_kv_cache(c["q"].to(dev), kv, vv, c["nk"].to(dev), c["nv"].to(dev), c["start"], c["end"],
                                           *c["blocking"], sm_scale=c["sm_scale"])
    return z, kv, vv


def direct_check(sfb, c, ref, budget=0):
    _, kv, vv = gpu_cache(sfb, c)
    dq, dk, dv = sfb.monarch_attn_with_kv_cache_backward(c["q"].cuda(), kv, vv, c["g"].cuda(), *c["blocking"],
                                                         sm_scale=c["sm_scale"], budget_bytes=budget)
    torch.cuda.synchronize()
    assert dq.dtype == torch.float32
    grad_close(dq, ref["q"], 1e-2, "dq")      # aL, Y and their gradients pass through bf16, as in the reference
    # reference cache gradients are zero in the written slots; the kernels return the gradient w.r.t. the cache
    # CONTENT there, which is the new keys' gradient in Monarch order
    ft, hr, wr, h, w = c["blocking"]
    full_k, full_v = ref["kc"].clone(), ref["vc"].clone()
    full_k[:, c["start"]:c["end"]] = orc.to_monarch_order(ref["nk"], ft, hr, wr, h, w).reshape(full_k[:, c["start"]:c["end"]].shape)
    full_v[:, c["start"]:c["end"]] = orc.to_monarch_order(ref["nv"], ft, hr, wr, h, w).reshape(full_v[:, c["start"]:c["end"]].shape)
    grad_close(dk, full_k, 1e-2, "dk")
    grad_close(dv, full_v, 1e-2, "dv")
    return dq, dk, dv


@pytest.mark.parametrize("ci", range(len(cases.SMALL_BLOCKINGS)))
def test_backward_small_blockings(sfb, ci):
    _, ft, hr, wr, h, w = cases.SMALL_BLOCKINGS[ci]
    c = make_case((ft, hr, wr, h, w), frames_q=2 if ft == 1 else 1, groups_cached=4 if ft == 1 else 2, B=2, H=2,
                  seed=8100 + ci)
    direct_check(sfb, c, oracle_grads(c))


@pytest.mark.parametrize("blocking,frames_q,cached", [((1, 1, 1, 30, 52), 1, 2), ((3, 1, 1, 30, 52), 1, 1),
                                                      ((1, 2, 1, 30, 52), 1, 2), ((1, 2, 4, 30, 52), 1, 2),
                                                      ((1, 1, 1, 45, 80), 1, 2), ((1, 1, 2, 8, 132), 2, 3)],
                         ids=["framewise", "tied3frame", "reduce2xh", "reduce4xw2xh", "wide45x80", "b2_66"])
def test_backward_real_block_sizes(sfb, blocking, frames_q, cached):
    """Block rows 30 / 90 / 15 / 45 (all three row-per-warp instantiations of the column kernel), block columns
    52 / 13 (odd) / 80 / 66 (both instantiations of the row kernel)."""
    c = make_case(blocking, frames_q, cached, B=1, H=2, seed=8200 + blocking[3] + blocking[0])
    direct_check(sfb, c, oracle_grads(c))


@pytest.mark.parametrize("blocking,frames_q,cached", [((1, 1, 1, 4, 24), 3, 4), ((1, 1, 1, 4, 40), 4, 5),
                                                      ((1, 1, 1, 5, 64), 3, 3), ((1, 1, 1, 30, 52), 3, 3),
                                                      ((1, 1, 1, 40, 24), 2, 4), ((3, 1, 1, 30, 52), 1, 2),
                                                      ((2, 1, 1, 33, 16), 2, 5)],
                         ids=["b2_24", "b2_40_two_tiles", "b2_64_two_tiles", "framewise_two_tiles",
                              "b1_40_two_chunks", "tied3frame_three_chunks_two_key_tiles", "b1_66_three_chunks"])
def test_backward_tile_widths_and_stacking(sfb, blocking, frames_q, cached):
    """Block columns 24 / 40 / 64 (the 32-, 48- and 64-wide instantiations of the tensor-core row-step backward;
    16 is covered by the small blockings) and three or four query groups, which stack into two tiles of query
    rows whose dK / dV shares are merged afterwards; block rows 40 / 66 / 90, i.e. two and three 32-row chunks
    in the column-step backward, over one to three key tiles."""
    c = make_case(blocking, frames_q, cached, B=1, H=2, seed=8250 + blocking[4])
    direct_check(sfb, c, oracle_grads(c))


def test_backward_row_kernels_agree(sfb, monkeypatch):
    """The tensor-core row-step backward against the fp32 one on the same intermediate gradients (the fp32 kernel
    rounds nothing but its inputs): both must sit within bf16 rounding of each other."""
    c = make_case((1, 1, 1, 6, 40), 3, 4, B=2, H=2, seed=8260)
    _, kv, vv = gpu_cache(sfb, c)
    args = (c["q"].cuda(), kv, vv, c["g"].cuda(), *c["blocking"])
    a = sfb.monarch_attn_with_kv_cache_backward(*args, sm_scale=c["sm_scale"])
    monkeypatch.setenv("SFM_BWD_ROW_FP32", "1")
    b = sfb.monarch_attn_with_kv_cache_backward(*args, sm_scale=c["sm_scale"])
    for x, y, what in zip(a, b, ("dq", "dk", "dv")):
        grad_close(x, y, 6e-3, what)


def test_backward_is_deterministic_and_slicing_is_invisible(sfb):
    c = make_case((1, 1, 1, 6, 8), 2, 4, B=2, H=3, seed=8300)
    ref = oracle_grads(c)
    a = direct_check(sfb, c, ref)
    b = direct_check(sfb, c, ref)
    one_pair = 2 * 8 * (4 * 6) * (2 * 128 + 2) * 4          # scratch of one (batch, head) pair: A b2 n_keys (2 D + 2) floats
    s = direct_check(sfb, c, ref, budget=2 * one_pair)      # three slices of two pairs
    for x, y, z in zip(a, b, s):
        assert torch.equal(x, y) and torch.equal(x, z)


def test_backward_group_range(sfb):
    """grad_only_new_kv at the C ABI: dK / dV of a range of groups equal that slice of the full result; dq does
    not depend on the range."""
    c = make_case((1, 1, 1, 6, 8), 2, 5, B=1, H=2, seed=8400)
    _, kv, vv = gpu_cache(sfb, c)
    args = (c["q"].cuda(), kv, vv, c["g"].cuda(), *c["blocking"])
    dq, dk, dv = sfb.monarch_attn_with_kv_cache_backward(*args, sm_scale=c["sm_scale"])
    dq2, dk2, dv2 = sfb.monarch_attn_with_kv_cache_backward(*args, sm_scale=c["sm_scale"], kv_groups=(3, 5))
    dq3, dk3, dv3 = sfb.monarch_attn_with_kv_cache_backward(*args, sm_scale=c["sm_scale"], kv_groups=(2, 2))
    assert torch.equal(dq, dq2) and torch.equal(dq, dq3)
    assert torch.equal(dk[:, 3 * 48:5 * 48], dk2) and torch.equal(dv[:, 3 * 48:5 * 48], dv2)
    assert dk3.shape[1] == 0 and dv3.shape[1] == 0


@pytest.mark.parametrize("only_new", [False, True])
def test_autograd_function(sfb, only_new):
    """monarch_attn_with_kv_cache under autograd: same forward result and cache content as without it;
    gradients of q, new_k, new_v (natural order) and of the cache (zero where the call wrote; absent with
    grad_only_new_kv)."""
    c = make_case((1, 2, 1, 6, 8), 2, 4, B=2, H=2, seed=8500)
    ref = oracle_grads(c)
    z0, kv0, _ = gpu_cache(sfb, c)
    dev = "cuda"
    q = c["q"].to(dev).requires_grad_()
    nk, nv = c["nk"].to(dev).requires_grad_(), c["nv"].to(dev).requires_grad_()
    kv = c["kbuf"].to(dev).clone()[:, :c["n_kv"]].requires_grad_(not only_new)
    vv = c["vbuf"].to(dev).clone()[:, :c["n_kv"]].requires_grad_(not only_new)
    z = sfb.monarch_attn_with_kv_cache(q, kv, vv, nk, nv, c["start"], c["end"], *c["blocking"], sm_scale=c["sm_scale"],
                                       grad_only_new_kv=only_new)
    assert torch.equal(z, z0) and torch.equal(kv.detach(), kv0)
    (z.float() * c["g"].to(dev).float()).sum().backward()
    torch.cuda.synchronize()
    grad_close(q.grad, ref["q"], 1e-2, "q.grad")
    grad_close(nk.grad, ref["nk"], 1e-2, "new_k.grad")
    grad_close(nv.grad, ref["nv"], 1e-2, "new_v.grad")
    if only_new:
        assert kv.grad is None and vv.grad is None
    else:
        # the reference's convention: gradient of the cache content after the write, the written slot holding
        # the new keys' / values' gradient in Monarch order
        ft, hr, wr, h, w = c["blocking"]
        s, e = c["start"], c["end"]
        full_k, full_v = ref["kc"].clone(), ref["vc"].clone()
        full_k[:, s:e] = orc.to_monarch_order(ref["nk"], ft, hr, wr, h, w).reshape(full_k[:, s:e].shape)
        full_v[:, s:e] = orc.to_monarch_order(ref["nv"], ft, hr, wr, h, w).reshape(full_v[:, s:e].shape)
        grad_close(kv.grad, full_k, 1e-2, "k_cache.grad")
        grad_close(vv.grad, full_v, 1e-2, "v_cache.grad")


@pytest.fixture(scope="module")
def pins():
    from conftest import ROOT
    return np.load(ROOT / "tests" / "golden" / "pins_golden.npz")


CS = cases.PIN_CHANNEL_STRIDE


@pytest.mark.parametrize("ci", range(len(cases.SMALL_BLOCKINGS)))
@pytest.mark.parametrize("only_new", [False, True])
def test_gradients_match_reference_fixtures(sfb, pins, ci, only_new):
    """The autograd path against gradients produced by the reference's own gradient oracle (autograd through
    its monarch_attn_with_kv_cache_ref, both grad_only_new_kv modes, as its run_kv_cache_test does)."""
    c = cases.grad_case(ci)
    dev = "cuda"
    q = bf(c["q"]).to(dev).requires_grad_()
    nk, nv = bf(c["nk"]).to(dev).requires_grad_(), bf(c["nv"]).to(dev).requires_grad_()
    kv = bf(c["kbuf"]).to(dev)[:, :c["n_kv"]].clone().requires_grad_(not only_new)
    vv = bf(c["vbuf"]).to(dev)[:, :c["n_kv"]].clone().requires_grad_(not only_new)
    z = sfb.monarch_attn_with_kv_cache(q, kv, vv, nk, nv, c["start"], c["end"], *c["blocking"], sm_scale=c["sm_scale"],
                                       grad_only_new_kv=only_new)
    z.backward(bf(c["g"]).to(dev))
    torch.cuda.synchronize()
    key = f"grad_{c['name']}_"
    ref = lambda n: torch.from_numpy(pins[key + n])
    err = (z.detach().float().cpu()[..., ::CS] - ref("z")).abs().max().item()
    assert err <= 2e-2, f"forward max-abs {err:.3e}"
    grad_close(q.grad[..., ::CS], ref("dq"), 1e-2, "q.grad")
    grad_close(nk.grad[..., ::CS], ref("dnk"), 1e-2, "new_k.grad")
    grad_close(nv.grad[..., ::CS], ref("dnv"), 1e-2, "new_v.grad")
    if only_new:
        assert kv.grad is None and vv.grad is None
    else:
        grad_close(kv.grad[..., ::CS], ref("dkc"), 1e-2, "k_cache.grad")
        grad_close(vv.grad[..., ::CS], ref("dvc"), 1e-2, "v_cache.grad")


@pytest.mark.parametrize("i", range(len(cases.CAUSAL_GRAD_CASES)))
def test_block_causal_gradients_match_reference_fixtures(sfb, pins, i):
    """monarch_attn with block_causal_size under autograd against autograd through the reference's
    monarch_attn_causal_ref."""
    c = cases.causal_grad_case(i)
    q, k, v = (bf(c[n]).cuda().requires_grad_() for n in ("q", "k", "v"))
    z = sfb.monarch_attn(q, k, v, *c["blocking"], sm_scale=c["sm_scale"], block_causal_size=c["block_causal"])
    z.backward(bf(c["g"]).cuda())
    torch.cuda.synchronize()
    key = f"causalgrad_{c['name']}_"
    for name, t in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
        grad_close(t[..., ::CS], torch.from_numpy(pins[key + name]), 1e-2, name)


def test_cache_rewrite_before_backward_is_an_error(sfb):
    """The saved cache is what the backward kernels read; overwriting it before backward must fail loudly (as
    the reference's in-place slice assignment does through autograd's version counters)."""
    c = cases.grad_case(0)
    dev = "cuda"
    q = bf(c["q"]).to(dev).requires_grad_()
    nk, nv = bf(c["nk"]).to(dev), bf(c["nv"]).to(dev)
    kv, vv = bf(c["kbuf"]).to(dev)[:, :c["n_kv"]].clone(), bf(c["vbuf"]).to(dev)[:, :c["n_kv"]].clone()
    z = sfb.monarch_attn_with_kv_cache(q, kv, vv, nk, nv, c["start"], c["end"], *c["blocking"])
    with torch.no_grad():
        sfb.monarch_attn_with_kv_cache(q.detach(), kv, vv, nk, nv, c["start"], c["end"], *c["blocking"])
    with pytest.raises(RuntimeError, match="modified by an inplace operation"):
        z.sum().backward()


@pytest.mark.parametrize("ci,causal_frames", [(0, None), (0, 2), (2, 1), (1, None), (3, 3)])
def test_nocache_autograd(sfb, ci, causal_frames):
    """monarch_attn under autograd, plain and block-causal: gradients of q, k, v in natural token order against
    autograd through the oracle."""
    _, ft, hr, wr, h, w = cases.SMALL_BLOCKINGS[ci]
    rng = np.random.default_rng(8600 + 10 * ci + (causal_frames or 0))
    n = 6 * ft * h * w
    B, H = 1, 2
    mk = lambda: bf(cases.randn(rng, B, n, H, 128))
    q, k, v, g = mk(), mk(), mk(), mk()
    bcs = None if causal_frames is None else causal_frames * ft * h * w
    q32, k32, v32 = (t.float().requires_grad_() for t in (q, k, v))
    z_ref = orc.monarch_attn(q32, k32, v32, ft, hr, wr, h, w, block_causal_size=bcs)
    (z_ref * g.float()).sum().backward()
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    z = sfb.monarch_attn(qg, kg, vg, ft, hr, wr, h, w, block_causal_size=bcs)
    with torch.no_grad():
        z_plain = sfb.monarch_attn(q.cuda(), k.cuda(), v.cuda(), ft, hr, wr, h, w, block_causal_size=bcs)
    assert torch.equal(z, z_plain)
    (z.float() * g.cuda().float()).sum().backward()
    torch.cuda.synchronize()
    grad_close(qg.grad, q32.grad, 1e-2, "q.grad")
    grad_close(kg.grad, k32.grad, 1e-2, "k.grad")
    grad_close(vg.grad, v32.grad, 1e-2, "v.grad")


def test_backward_properties_full_size(sfb):
    """Headline size (one 3-frame chunk against 7 cached chunks, 12 heads), where the oracle is too slow:
    the output is linear in V, so <dOut, out> = <dV, V> (checked with dOut = out, against the forward kernels'
    own output); doubling dOut doubles every gradient bit for bit; two runs agree bit for bit."""
    g = torch.Generator(device="cpu").manual_seed(8700)
    H, n_q, n_kv = 12, 4680, 7 * 4680
    mk = lambda n: torch.randn(1, n, H, 128, generator=g).to(torch.bfloat16).cuda()
    q, kc, vc = mk(n_q), mk(n_kv), mk(n_kv)
    blocking = (1, 1, 1, 30, 52)
    out = sfb.ops.monarch_attention_on_cache(q, kc, vc, *blocking)
    dq, dk, dv = sfb.monarch_attn_with_kv_cache_backward(q, kc, vc, out, *blocking)
    dq_b, dk_b, dv_b = sfb.monarch_attn_with_kv_cache_backward(q, kc, vc, out, *blocking)
    dq2, dk2, dv2 = sfb.monarch_attn_with_kv_cache_backward(q, kc, vc, out * 2, *blocking)
    torch.cuda.synchronize()
    assert torch.isfinite(dq).all() and torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()
    assert torch.equal(dq, dq_b) and torch.equal(dk, dk_b) and torch.equal(dv, dv_b)
    assert torch.equal(dq2, dq * 2) and torch.equal(dk2, dk * 2) and torch.equal(dv2, dv * 2)
    lhs = (out.double() ** 2).sum().item()
    rhs = (dv.double() * vc.double()).sum().item()
    assert abs(lhs - rhs) <= 1e-2 * lhs, (lhs, rhs)

"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle and the golden
fixtures.  Tolerance for bf16 results, from the acceptance rule of the task: max-abs <= 2e-2 and
relative L2 <= 1e-2 against an fp32 run of the reference arithmetic on the same (bf16-rounded)
inputs.  Integer / byte work (layout maps, cache writes without rotation) must be bit-exact.
"""
import numpy as np
import pytest
import torch

import cases
from oracle import monarch_oracle as orc

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
REL_L2 = 1e-2


@pytest.fixture(scope="module")
def sfb():
    import self_forcing_b200
    assert torch.cuda.is_available()
    return self_forcing_b200


def bf(x):
    return x.to(torch.bfloat16)


def check_close(got, ref, what=""):
    got = got.float().cpu()
    ref = ref.float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    err = (got - ref).abs().max().item()
    rel = ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert err <= MAX_ABS and rel <= REL_L2, f"{what}: max-abs {err:.3e} rel-L2 {rel:.3e}"
    return err, rel


def small_case(ci, iters, D=128, seed=None, B=2, H=2, chunks_cached=3):
    """Like cases.cache_case but at head_dim 128 (the only size the kernels are built for)."""
    name, ft, hr, wr, h, w = cases.SMALL_BLOCKINGS[ci]
    rng = np.random.default_rng(5000 + 10 * ci + iters if seed is None else seed)
    chunk = 3 * h * w
    n_buf, n_kv = (chunks_cached + 1) * chunk, chunks_cached * chunk
    mk = lambda *s: bf(cases.randn(rng, *s))
    return dict(name=name, blocking=(ft, hr, wr, h, w), q=mk(B, chunk, H, D), nk=mk(B, chunk, H, D),
                nv=mk(B, chunk, H, D), kbuf=mk(B, n_buf, H, D), vbuf=mk(B, n_buf, H, D),
                start=n_kv - chunk, end=n_kv, n_kv=n_kv, sm_scale=D ** -0.5)


def run_oracle_cache(c, iters=1):
    kc, vc = c["kbuf"].float().clone(), c["vbuf"].float().clone()
    n_kv = c["n_kv"]
    z = orc.monarch_attn_with_kv_cache(c["q"].float(), kc[:, :n_kv], vc[:, :n_kv], c["nk"].float(), c["nv"].float(),
                                       c["start"], c["end"], *c["blocking"], sm_scale=c["sm_scale"], num_iters=iters)
    return z, kc, vc


def run_gpu_cache(sfb, c, iters=1):
    dev = "cuda"
    kc, vc = c["kbuf"].to(dev).clone(), c["vbuf"].to(dev).clone()
    n_kv = c["n_kv"]
    z = sfb.monarch_attn_with_kv_cache(c["q"].to(dev), kc[:, :n_kv], vc[:, :n_kv], c["nk"].to(dev), c["nv"].to(dev),
                                       c["start"], c["end"], *c["blocking"], sm_scale=c["sm_scale"], num_iters=iters)
    torch.cuda.synchronize()
    return z, kc, vc


# ------------------------------------------------------------------------------- layout / rope
@pytest.mark.parametrize("ci", range(len(cases.SMALL_BLOCKINGS)))
def test_cache_write_bit_exact(sfb, ci):
    c = small_case(ci, 1)
    z_ref, kc_ref, vc_ref = run_oracle_cache(c)
    z, kc, vc = run_gpu_cache(sfb, c)
    assert torch.equal(kc.cpu().float(), kc_ref), "K cache after the in-place write differs"
    assert torch.equal(vc.cpu().float(), vc_ref), "V cache after the in-place write differs"


def test_cache_write_real_grid_bit_exact(sfb):
    """Permuted blocking on the real 30x52 grid, 12 heads: the written slot equals the oracle's map."""
    rng = np.random.default_rng(77)
    B, H, D, h, w = 1, 12, 128, 30, 52
    n = 3 * h * w
    nk, nv = bf(cases.randn(rng, B, n, H, D)), bf(cases.randn(rng, B, n, H, D))
    q = bf(cases.randn(rng, B, n, H, D))
    kc = torch.zeros(B, 2 * n, H, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    sfb.monarch_attn_with_kv_cache(q.cuda(), kc, vc, nk.cuda(), nv.cuda(), n, 2 * n, 1, 2, 4, h, w)
    _, mon2nat = orc.token_maps(n, 1, 2, 4, h, w)
    assert torch.equal(kc[:, n:].cpu(), nk[:, torch.from_numpy(mon2nat)])
    assert torch.equal(vc[:, n:].cpu(), nv[:, torch.from_numpy(mon2nat)])
    assert not kc[:, :n].any() and not vc[:, :n].any()


def ulp_mismatch(a, b, tiny=1e-3, tiny_abs=1e-6):
    """Count of elements differing, and max difference in bf16 ulps (via the int16 bit patterns).
    Results below `tiny` in magnitude come from cancelling terms of order one (a rotation in fp32
    here, fp64 in the reference) and are compared by absolute difference instead."""
    small = (b.float().abs() < tiny) & ((a.float() - b.float()).abs() <= tiny_abs)
    a = torch.where(small, b, a)
    ai = a.contiguous().view(torch.int16).to(torch.int32)
    bi = b.contiguous().view(torch.int16).to(torch.int32)
    # sign-magnitude -> monotonic integer
    ai = torch.where(ai < 0, -(ai & 0x7FFF), ai)
    bi = torch.where(bi < 0, -(bi & 0x7FFF), bi)
    d = (ai - bi).abs()
    return int((d > 0).sum()), int(d.max())


@pytest.mark.parametrize("sf", [0, 9])
def test_rope_standalone(sfb, golden, sf):
    x, grid = cases.rope_inputs()
    xb = bf(x)
    ref = orc.rope_apply(xb, grid, start_frame=sf)            # fp64 rotation, one rounding to bf16
    if sf == 9:
        assert np.array_equal(ref.float().numpy(), golden["rope_out_bf16_sf9"])
    grid_t = torch.tensor([list(grid)] * x.shape[0])
    got = sfb.causal_rope_apply(xb.cuda(), grid_t, None, start_frame=sf).cpu()
    n_diff, max_ulp = ulp_mismatch(got, ref)
    # fp32 rotation vs fp64: only rounding ties may move, by one ulp
    assert max_ulp <= 1 and n_diff <= 0.002 * got.numel(), (n_diff, max_ulp)
    # pass-through tail is exact
    assert torch.equal(got[:, 105:], xb[:, 105:])


@pytest.mark.parametrize("H", [1, 2, 3, 5])
def test_rope_fused_front_end(sfb, H):
    """RoPE + layout + cache write in one kernel == separate rotation followed by the plain op
    (head counts on both sides of the 64-thread mark: the rotation table is staged per CTA)."""
    rng = np.random.default_rng(11)
    B, D, h, w = 2, 128, 6, 8
    n = 3 * h * w
    q, k, v = (bf(cases.randn(rng, B, n, H, D)).cuda() for _ in range(3))
    kbuf = bf(cases.randn(rng, B, 3 * n, H, D)).cuda()
    vbuf = bf(cases.randn(rng, B, 3 * n, H, D)).cuda()
    grid_t = torch.tensor([[3, h, w]] * B)
    for ft, hr, wr in ((1, 1, 1), (1, 2, 4), (3, 1, 1)):
        k1, v1, k2, v2 = kbuf.clone(), vbuf.clone(), kbuf.clone(), vbuf.clone()
        z1 = sfb.rope_monarch_attn_with_kv_cache(q, k, v, k1[:, :2 * n], v1[:, :2 * n], n, 2 * n, 3, ft, hr, wr, h, w)
        rq = sfb.causal_rope_apply(q, grid_t, None, start_frame=3)
        rk = sfb.causal_rope_apply(k, grid_t, None, start_frame=3)
        z2 = sfb.monarch_attn_with_kv_cache(rq, k2[:, :2 * n], v2[:, :2 * n], rk, v, n, 2 * n, ft, hr, wr, h, w)
        assert torch.equal(k1, k2) and torch.equal(v1, v2)
        assert torch.equal(z1, z2)
        # and against the oracle's fp64 rotation
        ref_k = orc.rope_apply(k.cpu(), (3, h, w), start_frame=3)
        _, mon2nat = orc.token_maps(n, ft, hr, wr, h, w)
        n_diff, max_ulp = ulp_mismatch(k1[:, n:2 * n].cpu(), ref_k[:, torch.from_numpy(mon2nat)])
        assert max_ulp <= 1 and n_diff <= 0.002 * ref_k.numel()


# ------------------------------------------------------------------------------- Monarch, T = 1
@pytest.mark.parametrize("ci", range(len(cases.SMALL_BLOCKINGS)))
def test_monarch_small_blockings(sfb, ci):
    c = small_case(ci, 1)
    z_ref, _, _ = run_oracle_cache(c)
    z, _, _ = run_gpu_cache(sfb, c)
    check_close(z, z_ref, c["name"])


@pytest.mark.parametrize("blk", cases.REAL_BLOCKINGS)
def test_monarch_real_block_sizes_vs_golden(sfb, golden, blk):
    """30x52 grid, D=128, one head: compare with the fixture computed by the reference's own code
    (fp32 inputs there; the GPU sees them rounded to bf16, which the tolerance covers)."""
    name, ft, hr, wr = blk
    c = cases.real_case()
    kc, vc = bf(c["kbuf"]).cuda(), bf(c["vbuf"]).cuda()
    z = sfb.monarch_attn_with_kv_cache(bf(c["q"]).cuda(), kc, vc, bf(c["nk"]).cuda(), bf(c["nv"]).cuda(),
                                       c["start"], c["end"], ft, hr, wr, c["h"], c["w"])
    ref = torch.from_numpy(golden[f"real_{name}_z_sample"])
    check_close(z[0, ::37, 0, :], ref, name)


def test_monarch_baseline_config1_vs_golden(sfb, golden):
    c = cases.c1_case()
    kc = torch.zeros(1, c["chunk"], 12, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    z = sfb.monarch_attn_with_kv_cache(bf(c["q"]).cuda(), kc, vc, bf(c["k"]).cuda(), bf(c["v"]).cuda(), 0, c["chunk"],
                                       1, 1, 1, c["h"], c["w"])
    check_close(z[0, ::97, ::5, :], torch.from_numpy(golden["c1_T1_z_sample"]), "config 1, T=1")


@pytest.mark.parametrize("name,ft,hr,wr,k_chunks", [("framewise", 1, 1, 1, 7), ("tied3frame", 3, 1, 1, 4),
                                                      ("reduce2xh", 1, 2, 1, 3), ("reduce4xw2xh", 1, 2, 4, 2),
                                                      ("tied3frame", 3, 1, 1, 7), ("reduce2xh", 1, 2, 1, 7),
                                                      ("reduce4xw2xh", 1, 2, 4, 7), ("framewise", 1, 1, 1, 1)])
def test_monarch_rollout_shapes_vs_oracle(sfb, name, ft, hr, wr, k_chunks):
    """Wan-1.3B chunk (4680 queries) against k cached chunks, every blocking at the full cache length (k = 7,
    where the unit lists, the F splits and the bridge are largest); 2 of the heads are checked on the CPU."""
    rng = np.random.default_rng(900 + k_chunks)
    B, H, D, h, w = 1, 4, 128, 30, 52
    n = 3 * h * w
    n_kv = k_chunks * n
    mk = lambda *s: bf(cases.randn(rng, *s))
    q, nk, nv = mk(B, n, H, D), mk(B, n, H, D), mk(B, n, H, D)
    kbuf, vbuf = mk(B, 7 * n, H, D), mk(B, 7 * n, H, D)
    kc, vc = kbuf.cuda().clone(), vbuf.cuda().clone()
    z = sfb.monarch_attn_with_kv_cache(q.cuda(), kc[:, :n_kv], vc[:, :n_kv], nk.cuda(), nv.cuda(), n_kv - n, n_kv,
                                       ft, hr, wr, h, w)
    hs = [0, 3]
    kr, vr = kbuf[:, :, hs].float().clone(), vbuf[:, :, hs].float().clone()
    z_ref = orc.monarch_attn_with_kv_cache(q[:, :, hs].float(), kr[:, :n_kv], vr[:, :n_kv], nk[:, :, hs].float(),
                                           nv[:, :, hs].float(), n_kv - n, n_kv, ft, hr, wr, h, w)
    check_close(z[:, :, hs], z_ref, f"{name} k={k_chunks}")


def test_monarch_chunking_is_invisible(sfb, monkeypatch):
    """The bridge budget only changes how the work is cut into launches, never the result."""
    c = small_case(3, 1, B=2, H=3)
    z_a, _, _ = run_gpu_cache(sfb, c)
    monkeypatch.setenv("SFM_BRIDGE_MB", "1")
    z_b, _, _ = run_gpu_cache(sfb, c)
    assert torch.equal(z_a, z_b)


def test_monarch_properties_full_size(sfb):
    """Size-independent properties at the full benchmark size (12 heads, 32760 cached tokens):
    (1) bitwise run-to-run determinism, (2) a constant V comes back unchanged (all softmax
    weights sum to one), (3) heads are independent (a 1-head call equals that head of the
    12-head call)."""
    rng = np.random.default_rng(4242)
    B, H, D, h, w = 1, 12, 128, 30, 52
    n, n_kv = 3 * h * w, 7 * 3 * h * w
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(B, n, H, D, device="cuda", generator=g).bfloat16()
    kc = torch.randn(B, n_kv, H, D, device="cuda", generator=g).bfloat16()
    vc = torch.randn(B, n_kv, H, D, device="cuda", generator=g).bfloat16()
    nk, nv = kc[:, -n:].clone(), vc[:, -n:].clone()
    z1 = sfb.monarch_attn_with_kv_cache(q, kc, vc, nk, nv, n_kv - n, n_kv, 1, 1, 1, h, w)
    z2 = sfb.monarch_attn_with_kv_cache(q, kc, vc, nk, nv, n_kv - n, n_kv, 1, 1, 1, h, w)
    assert torch.equal(z1, z2)
    const = torch.linspace(-2, 2, D, device="cuda").bfloat16().expand(B, n_kv, H, D).contiguous()
    zc = sfb.monarch_attn_with_kv_cache(q, kc, const.clone(), nk, const[:, -n:].clone(), n_kv - n, n_kv, 1, 1, 1, h, w)
    assert (zc.float() - const[:, :n].float()).abs().max().item() <= 2e-2
    hsel = 5
    k1, v1 = kc[:, :, hsel:hsel + 1].contiguous(), vc[:, :, hsel:hsel + 1].contiguous()
    zh = sfb.monarch_attn_with_kv_cache(q[:, :, hsel:hsel + 1].contiguous(), k1, v1, k1[:, -n:].clone(),
                                        v1[:, -n:].clone(), n_kv - n, n_kv, 1, 1, 1, h, w)
    assert torch.equal(zh[:, :, 0], z1[:, :, hsel])


# ------------------------------------------------------------------------------- Monarch, T > 1
@pytest.mark.parametrize("ci", range(len(cases.SMALL_BLOCKINGS)))
@pytest.mark.parametrize("iters", [2, 5])
def test_monarch_iterative_small(sfb, ci, iters):
    c = small_case(ci, iters)
    z_ref, _, _ = run_oracle_cache(c, iters)
    z, _, _ = run_gpu_cache(sfb, c, iters)
    check_close(z, z_ref, f"{c['name']} T={iters}")


def test_monarch_baseline_config1_T20_vs_golden(sfb, golden):
    c = cases.c1_case()
    kc = torch.zeros(1, c["chunk"], 12, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    z = sfb.monarch_attn_with_kv_cache(bf(c["q"]).cuda(), kc, vc, bf(c["k"]).cuda(), bf(c["v"]).cuda(), 0, c["chunk"],
                                       1, 1, 1, c["h"], c["w"], num_iters=20)
    check_close(z[0, ::97, ::5, :], torch.from_numpy(golden["c1_T20_z_sample"]), "config 1, T=20")


# ------------------------------------------------------------------------------- no-cache entry point
@pytest.mark.parametrize("ci", range(4))
def test_monarch_nocache_and_block_causal(sfb, ci):
    name, ft, hr, wr, h, w = cases.SMALL_BLOCKINGS[ci]
    rng = np.random.default_rng(6000 + ci)
    B, H, D = 2, 2, 128
    n = 6 * h * w
    q, k, v = (bf(cases.randn(rng, B, n, H, D)) for _ in range(3))
    for iters in (1, 3):
        ref = orc.monarch_attn(q.float(), k.float(), v.float(), ft, hr, wr, h, w, num_iters=iters)
        got = sfb.monarch_attn(q.cuda(), k.cuda(), v.cuda(), ft, hr, wr, h, w, num_iters=iters)
        check_close(got, ref, f"{name} no-cache T={iters}")
    bc = 3 * h * w
    ref = orc.monarch_attn(q.float(), k.float(), v.float(), ft, hr, wr, h, w, block_causal_size=bc)
    got = sfb.monarch_attn(q.cuda(), k.cuda(), v.cuda(), ft, hr, wr, h, w, block_causal_size=bc)
    check_close(got, ref, f"{name} block-causal")


# ------------------------------------------------------------------------------- dense path
@pytest.mark.parametrize("n_q,n_kv", [(50, 170), (4680, 4680), (333, 1000)])
def test_dense_attention(sfb, n_q, n_kv):
    rng = np.random.default_rng(31 + n_q)
    B, H, D = 2, 3, 128
    q, k, v = bf(cases.randn(rng, B, n_q, H, D)), bf(cases.randn(rng, B, n_kv + 64, H, D)), bf(cases.randn(rng, B, n_kv + 64, H, D))
    kd, vd = k.cuda(), v.cuda()
    got = sfb.attention(q.cuda(), kd[:, :n_kv], vd[:, :n_kv])      # strided views, as the model passes them
    ref = orc.dense_attention(q.float(), k[:, :n_kv].float(), v[:, :n_kv].float())
    check_close(got, ref, f"dense {n_q}x{n_kv}")


@pytest.mark.parametrize("i", range(len(cases.DENSE_CASES)))
def test_dense_attention_vs_reference_fixture(sfb, i):
    """Against the reference's own attention() run through its SDPA branch in fp32 (pins_golden.npz)."""
    from conftest import ROOT
    pins = np.load(ROOT / "tests" / "golden" / "pins_golden.npz")
    c = cases.dense_case(i)
    kd, vd = bf(c["kbuf"]).cuda(), bf(c["vbuf"]).cuda()
    got = sfb.attention(bf(c["q"]).cuda(), kd[:, :c["n_kv"]], vd[:, :c["n_kv"]])
    check_close(got, torch.from_numpy(pins[f"dense_{i}_fp32"]), f"dense case {i}")


@pytest.mark.parametrize("gain", [0.02, 0.2, 1.0, 3.0])
def test_dense_attention_with_a_growing_maximum(sfb, gain):
    """Keys ordered so that every query's logits rise along the cache, by about 0.2, 2, 10 and 31 in log2 units per
    64 keys.  The slowest rise stays inside the rescale threshold of 8 for long stretches (half tiles taken in the
    speculative single pass against a reference that falls behind), the second passes it every few half tiles (the
    row sums refuse the speculative pass and the two-pass path rescales the accumulator), the last two at every
    half tile."""
    rng = np.random.default_rng(77)
    B, H, D, n_q, n_kv = 1, 2, 128, 256, 1500
    q = cases.randn(rng, B, n_q, H, D)
    direction = q.mean(dim=1, keepdim=True)
    direction = direction / direction.norm(dim=-1, keepdim=True)
    ramp = torch.linspace(0.0, 1.0, n_kv).view(1, n_kv, 1, 1)
    k = 0.3 * cases.randn(rng, B, n_kv, H, D) + gain * 400.0 * ramp * direction
    v = cases.randn(rng, B, n_kv, H, D)
    q = q + 4.0 * direction                                   # every query has a solid component along the ramp
    q, k, v = bf(q), bf(k), bf(v)
    got = sfb.attention(q.cuda(), k.cuda(), v.cuda())
    ref = orc.dense_attention(q.float(), k.float(), v.float())
    check_close(got, ref, f"dense, rising logits (gain {gain})")
    ops_mod = __import__("self_forcing_b200").ops
    ops_mod.check_device_status()


def test_dense_with_cache_write(sfb):
    rng = np.random.default_rng(8)
    B, H, D, n = 1, 2, 128, 96
    q, nk, nv = (bf(cases.randn(rng, B, n, H, D)) for _ in range(3))
    kbuf, vbuf = bf(cases.randn(rng, B, 3 * n, H, D)), bf(cases.randn(rng, B, 3 * n, H, D))
    kc, vc = kbuf.cuda().clone(), vbuf.cuda().clone()
    got = sfb.full_attention_with_kv_cache(q.cuda(), kc[:, :2 * n], vc[:, :2 * n], nk.cuda(), nv.cuda(), n, 2 * n)
    kr, vr = kbuf.clone(), vbuf.clone()
    kr[:, n:2 * n] = nk
    vr[:, n:2 * n] = nv
    assert torch.equal(kc.cpu(), kr) and torch.equal(vc.cpu(), vr)
    ref = orc.dense_attention(q.float(), kr[:, :2 * n].float(), vr[:, :2 * n].float())
    check_close(got, ref, "dense after cache write")


def test_errors_are_loud(sfb):
    q = torch.zeros(1, 1560, 1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):            # cache extent not a whole number of groups
        sfb.monarch_attn_with_kv_cache(q, torch.zeros(1, 1600, 1, 128, dtype=torch.bfloat16, device="cuda"),
                                       torch.zeros(1, 1600, 1, 128, dtype=torch.bfloat16, device="cuda"),
                                       q, q, 40, 1600, 1, 1, 1, 30, 52)
    with pytest.raises(TypeError):
        sfb.attention(q.float().half(), q.half(), q.half(), dtype=torch.float16)
    with pytest.raises(ValueError):
        sfb.attention(torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16, device="cuda"),
                      torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16, device="cuda"),
                      torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.gpu
def test_gather_scatter_shards_match_unsharded(sfb):
    """Head-sharded entry points, two ranks emulated on one GPU: rank r gathers its heads from both token
    shards and scatters its result rows into both output shards; together they must reproduce the
    unsharded call bit for bit (heads are independent in every kernel)."""
    import torch
    from self_forcing_b200 import ops
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(7)
    B, H, hh, ww, frames, world = 1, 4, 6, 8, 2, 2
    n = frames * hh * ww
    k_chunks = 3
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(dev)
    q, k, v = mk(B, n, H, 128), mk(B, n, H, 128), mk(B, n, H, 128)
    kc_full, vc_full = mk(B, k_chunks * n, H, 128), mk(B, k_chunks * n, H, 128)
    start, end, start_frame = (k_chunks - 1) * n, k_chunks * n, frames * (k_chunks - 1)
    kc_ref, vc_ref = kc_full.clone(), vc_full.clone()
    ref = sfb.rope_monarch_attn_with_kv_cache(q, k, v, kc_ref, vc_ref, start, end, start_frame, 1, 1, 1, hh, ww)
    sp, hp = n // world, H // world
    q_sh = [q[:, p * sp:(p + 1) * sp].contiguous() for p in range(world)]
    k_sh = [k[:, p * sp:(p + 1) * sp].contiguous() for p in range(world)]
    v_sh = [v[:, p * sp:(p + 1) * sp].contiguous() for p in range(world)]
    out_sh = [torch.zeros(B, sp, H, 128, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    for r in range(world):
        kc = kc_full[:, :, r * hp:(r + 1) * hp].contiguous()
        vc = vc_full[:, :, r * hp:(r + 1) * hp].contiguous()
        ops.rope_monarch_attn_with_kv_cache_sharded([t.data_ptr() for t in q_sh], [t.data_ptr() for t in k_sh],
                                                    [t.data_ptr() for t in v_sh], [t.data_ptr() for t in out_sh], r,
                                                    (B, sp, H, 128), kc, vc, start, end, start_frame, 1, 1, 1, hh, ww)
        torch.cuda.synchronize()
        assert torch.equal(kc, kc_ref[:, :, r * hp:(r + 1) * hp])
        assert torch.equal(vc, vc_ref[:, :, r * hp:(r + 1) * hp])
    got = torch.cat(out_sh, dim=1)
    assert torch.equal(got, ref)


# ------------------------------------------------------------------------------- layer level
@pytest.mark.gpu
@pytest.mark.parametrize("H", [2, 12])
def test_norm_rope_cache_write_vs_oracle(sfb, H):
    """Full-width RMSNorm of q and k + RoPE + Monarch-order cache write in one kernel against the oracle
    chain rms_norm (reference WanRMSNorm) -> fp64 rotation -> permutation.  bf16 results may differ by one
    ulp where the fp32 mean of squares sums in another order; v is copied bit for bit."""
    rng = np.random.default_rng(77 + H)
    B, h, w = 2, 6, 8
    n = 3 * h * w
    q, k, v = (bf(cases.randn(rng, B, n, H, 128) * 1.7) for _ in range(3))
    wq = bf(torch.from_numpy(rng.uniform(0.5, 1.5, size=H * 128).astype(np.float32)))
    wk = bf(torch.from_numpy(rng.uniform(0.5, 1.5, size=H * 128).astype(np.float32)))
    eps = 1e-6
    kc = torch.zeros(B, 2 * n, H, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q_rot = sfb.norm_rope_cache_write(q.cuda(), k.cuda(), v.cuda(), kc, vc, n, 3, 1, 2, 4, h, w,
                                      norm_q_weight=wq.cuda(), norm_k_weight=wk.cuda(), eps=eps)
    torch.cuda.synchronize()
    nq = orc.rms_norm(q.reshape(B, n, H * 128), wq, eps).reshape(B, n, H, 128)
    nk = orc.rms_norm(k.reshape(B, n, H * 128), wk, eps).reshape(B, n, H, 128)
    ref_q = orc.rope_apply(nq, (3, h, w), start_frame=3)
    ref_k = orc.rope_apply(nk, (3, h, w), start_frame=3)
    _, mon2nat = orc.token_maps(n, 1, 2, 4, h, w)
    perm = torch.from_numpy(mon2nat)
    for got, ref in ((q_rot.cpu(), ref_q), (kc[:, n:].cpu(), ref_k[:, perm])):
        n_diff, max_ulp = ulp_mismatch(got, ref)
        assert max_ulp <= 2 and n_diff <= 0.01 * ref.numel(), (n_diff, max_ulp)
    assert torch.equal(vc[:, n:].cpu(), v[:, perm])
    assert not kc[:, :n].any() and not vc[:, :n].any()


def _oracle_layer_call(state, q, k, v, current_start, grid, cfg, wq, wk):
    """CPU restatement of the cache branch of CausalWanSelfAttention.forward (causal_model.py:900-1103)
    from oracle pieces, on fp32 copies of bf16-rounded cache contents."""
    frames, gh, gw = grid
    B, n, H, D = q.shape
    ft = 1 if cfg.use_framewise else 3
    frame = gh * gw
    r = orc.cache_indices(current_start, n, state["g_end"], state["l_end"], state["k"].shape[1], cfg.max_attention_size,
                          local_attn_size=cfg.local_attn_size, sink_tokens=cfg.sink_size * frame)
    if r["roll"] is not None:
        dst, src, cnt = r["roll"]
        for t in (state["k"], state["v"]):
            t[:, dst:dst + cnt] = t[:, src:src + cnt].clone()
    nq = orc.rms_norm(q.reshape(B, n, H * D), wq, cfg.eps).reshape(B, n, H, D)
    nk = orc.rms_norm(k.reshape(B, n, H * D), wk, cfg.eps).reshape(B, n, H, D)
    rq = orc.rope_apply(nq, grid, start_frame=current_start // frame)
    rk = orc.rope_apply(nk, grid, start_frame=current_start // frame)
    ck = state["k"][:, r["cache_start"]:r["cache_start"] + r["local_end"]]
    cv = state["v"][:, r["cache_start"]:r["cache_start"] + r["local_end"]]
    is_init = cfg.use_dense_init and ck.shape[1] == 3 * frame
    if cfg.disable_monarch or is_init:
        ck[:, r["local_start"]:r["local_end"]] = rk.float()
        cv[:, r["local_start"]:r["local_end"]] = v.float()
        out = orc.dense_attention(rq.float(), ck, cv)
    else:
        out = orc.monarch_attn_with_kv_cache(rq.float(), ck, cv, rk.float(), v.float(), r["local_start"], r["local_end"],
                                             ft, cfg.h_reduce, cfg.w_reduce, gh, gw, num_iters=cfg.num_iters)
    state["g_end"], state["l_end"] = r["store_global_end"], r["store_local_end"]
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["plain", "window_sink", "window10_sink2", "window7_dense", "dense_init", "regular"])
def test_layer_rollout_matches_oracle(sfb, mode):
    """Several chunks through self_attention_kv (each chunk denoised twice, as the few-step sampler does)
    against the oracle's restatement of the reference layer, including the sliding window with a sink frame,
    the dense first chunk and the all-dense configuration; the caches must agree too."""
    rng = np.random.default_rng({"plain": 1, "window_sink": 2, "dense_init": 3, "regular": 4, "window10_sink2": 5,
                                 "window7_dense": 6}[mode])
    B, H, gh, gw = 1, 2, 6, 8
    frame, n = gh * gw, 3 * gh * gw
    cfg = sfb.LayerConfig(use_framewise=True)
    cache_frames = 12
    if mode == "window_sink":                      # evicts a whole chunk each time (shift inside the write kernel)
        cfg.local_attn_size, cfg.sink_size, cache_frames = 9, 1, 9
    if mode == "window10_sink2":                   # window not a multiple of the chunk: the first eviction is shorter
        cfg.local_attn_size, cfg.sink_size, cache_frames = 10, 2, 10
    if mode == "window7_dense":                    # natural-order (dense) cache with eviction
        cfg.local_attn_size, cfg.sink_size, cache_frames, cfg.disable_monarch = 7, 0, 7, True
    if mode == "dense_init":
        cfg.use_dense_init = True
    if mode == "regular":
        cfg.disable_monarch = True
    cfg.max_attention_size = cache_frames * frame
    cache = sfb.KVCache.allocate(B, cache_frames * frame, H, "cuda")
    state = {"k": torch.zeros(B, cache_frames * frame, H, 128), "v": torch.zeros(B, cache_frames * frame, H, 128),
             "g_end": 0, "l_end": 0}
    wq = bf(torch.from_numpy(rng.uniform(0.7, 1.3, size=H * 128).astype(np.float32)))
    wk = bf(torch.from_numpy(rng.uniform(0.7, 1.3, size=H * 128).astype(np.float32)))
    n_chunks = 6 if mode.startswith("window") else 4
    for chunk in range(n_chunks):
        for rep in range(2):
            q, k, v = (bf(cases.randn(rng, B, n, H, 128)) for _ in range(3))
            got = sfb.self_attention_kv(q.cuda(), k.cuda(), v.cuda(), cache, chunk * n, (3, gh, gw), cfg,
                                        norm_q_weight=wq.cuda(), norm_k_weight=wk.cuda())
            torch.cuda.synchronize()
            ref = _oracle_layer_call(state, q, k, v, chunk * n, (3, gh, gw), cfg, wq, wk)
            check_close(got, ref, f"{mode} chunk {chunk} pass {rep}")
            assert (cache.global_end, cache.local_end) == (state["g_end"], state["l_end"])
            # cache contents: rotated keys within bf16 rounding of the oracle's, values identical
            used = state["l_end"]
            assert torch.equal(cache.v[:, :used].cpu().float(), state["v"][:, :used])
            dk = (cache.k[:, :used].cpu().float() - bf(state["k"][:, :used]).float()).abs().max().item()
            assert dk <= 0.05, dk
            # keep the two caches in lock step (the oracle's keys are fp32, ours bf16)
            state["k"][:, :used] = cache.k[:, :used].cpu().float()


@pytest.mark.gpu
def test_patched_forward_on_a_lookalike_module(sfb):
    """patch_self_attention_forward on a module with the attributes of the reference's
    CausalWanSelfAttention (the reference itself cannot be imported where the GPU tests run): the patched
    forward must equal projections -> oracle layer -> output projection, follow a cache reset done the
    pipeline's way (new index tensors in the dict), and leave the dict's device indices up to date."""
    from self_forcing_b200.install import patch_self_attention_forward
    torch.manual_seed(3)
    dim, H, gh, gw = 256, 2, 6, 8
    frame, n = gh * gw, 3 * gh * gw

    class Norm(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.rand(dim) + 0.5)

    class Attn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.num_heads, self.head_dim, self.eps = H, dim // H, 1e-6
            self.use_framewise, self.h_reduce, self.w_reduce, self.num_iters = True, 1, 1, 1
            self.disable_monarch, self.use_dense_init = False, True
            self.local_attn_size, self.sink_size, self.max_attention_size = -1, 0, 12 * frame
            self.topk, self.use_svg, self.use_radial_attn = None, False, False
            self.q, self.k, self.v, self.o = (torch.nn.Linear(dim, dim) for _ in range(4))
            self.norm_q, self.norm_k = Norm(), Norm()

        def forward(self, *a, **k):
            raise AssertionError("the original forward must not be reached on the cache path")

    patch_self_attention_forward(Attn)
    m = Attn().cuda().to(torch.bfloat16)
    kv = {"k": torch.zeros(1, 12 * frame, H, 128, dtype=torch.bfloat16, device="cuda"),
          "v": torch.zeros(1, 12 * frame, H, 128, dtype=torch.bfloat16, device="cuda"),
          "global_end_index": torch.tensor([0], device="cuda"), "local_end_index": torch.tensor([0], device="cuda")}
    grid_sizes = torch.tensor([[3, gh, gw]])
    cfg = sfb.LayerConfig(use_framewise=True, use_dense_init=True, max_attention_size=12 * frame)
    for video in range(2):
        state = {"k": torch.zeros(1, 12 * frame, H, 128), "v": torch.zeros(1, 12 * frame, H, 128), "g_end": 0, "l_end": 0}
        for chunk in range(3):
            x = torch.randn(1, n, dim).to(torch.bfloat16).cuda()
            got = m(x, None, grid_sizes, None, None, kv_cache=kv, current_start=chunk * n)
            torch.cuda.synchronize()
            q = m.q(x).view(1, n, H, 128).cpu()
            k = m.k(x).view(1, n, H, 128).cpu()
            v = m.v(x).view(1, n, H, 128).cpu()
            ref = _oracle_layer_call(state, q, k, v, chunk * n, (3, gh, gw), cfg, m.norm_q.weight.detach().cpu(),
                                     m.norm_k.weight.detach().cpu())
            ref_out = m.o(bf(ref).cuda().flatten(2))
            err = (got.float() - ref_out.float()).abs().max().item()
            assert err <= 3e-2, (video, chunk, err)
            assert kv["global_end_index"].item() == state["g_end"] and kv["local_end_index"].item() == state["l_end"]
            state["k"][:, :state["l_end"]] = kv["k"][:, :state["l_end"]].cpu().float()
        # the pipeline's reset: new index tensors, same k / v buffers
        kv["global_end_index"] = torch.tensor([0], device="cuda")
        kv["local_end_index"] = torch.tensor([0], device="cuda")


# ------------------------------------------------------------------------------- seeded shape sweep
def _sweep_configs():
    """Seeded mix of shapes the other tests do not pair up: odd head counts, two videos with a cache batch
    stride longer than the view, query chunks of 3 to 6 frames, 1 to 5 cached chunks, grids whose block rows
    and columns land on every padding case of the kernels (b2 from 2 to 48, b1 from 3 to 36)."""
    import random
    rnd = random.Random(2024)
    grids = [(6, 8), (4, 12), (12, 16), (8, 48), (5, 7), (10, 26)]
    out = []
    for _ in range(18):
        h, w = rnd.choice(grids)
        ft = rnd.choice([1, 3])
        hr = rnd.choice([d for d in (1, 2, 3, 4, 5) if h % d == 0])
        wr = rnd.choice([d for d in (1, 2, 4, 13) if w % d == 0])
        frames_q = 3 * rnd.choice([1, 2])
        cached = rnd.randint(1, 5)
        out.append(dict(h=h, w=w, ft=ft, hr=hr, wr=wr, frames_q=frames_q, cached=cached, B=rnd.choice([1, 2]),
                        H=rnd.choice([1, 2, 3, 5]), T=rnd.choice([1, 1, 1, 2]), seed=rnd.randrange(1 << 30)))
    # wide grids: block columns above 64 (two-stage K / V ring and the chunked row softmax of the row step)
    for (h, w, hr, wr, ft, B, H, cached, fq) in [(4, 80, 1, 1, 1, 1, 2, 2, 3), (3, 128, 1, 1, 1, 2, 1, 1, 3),
                                                 (6, 72, 2, 1, 1, 1, 3, 3, 6), (2, 104, 1, 1, 3, 1, 2, 2, 3),
                                                 (4, 96, 4, 1, 1, 1, 1, 4, 3), (5, 66, 1, 1, 1, 1, 2, 1, 6)]:
        out.append(dict(h=h, w=w, ft=ft, hr=hr, wr=wr, frames_q=fq, cached=cached, B=B, H=H, T=1,
                        seed=rnd.randrange(1 << 30)))
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", _sweep_configs(), ids=lambda c: "h{h}w{w}_ft{ft}hr{hr}wr{wr}_q{frames_q}c{cached}_B{B}H{H}T{T}".format(**c))
def test_monarch_seeded_shape_sweep(sfb, cfg):
    rng = np.random.default_rng(cfg["seed"])
    h, w, B, H = cfg["h"], cfg["w"], cfg["B"], cfg["H"]
    frame = h * w
    n_q = cfg["frames_q"] * frame
    n_kv = cfg["cached"] * 3 * frame + n_q
    n_buf = n_kv + 3 * frame                                  # the view is shorter than the buffer
    mk = lambda *s: bf(cases.randn(rng, *s))
    q, nk, nv = mk(B, n_q, H, 128), mk(B, n_q, H, 128), mk(B, n_q, H, 128)
    kbuf, vbuf = mk(B, n_buf, H, 128), mk(B, n_buf, H, 128)
    blocking = (cfg["ft"], cfg["hr"], cfg["wr"], h, w)
    kc, vc = kbuf.float().clone(), vbuf.float().clone()
    ref = orc.monarch_attn_with_kv_cache(q.float(), kc[:, :n_kv], vc[:, :n_kv], nk.float(), nv.float(), n_kv - n_q, n_kv,
                                         *blocking, num_iters=cfg["T"])
    kg, vg = kbuf.cuda().clone(), vbuf.cuda().clone()
    got = sfb.monarch_attn_with_kv_cache(q.cuda(), kg[:, :n_kv], vg[:, :n_kv], nk.cuda(), nv.cuda(), n_kv - n_q, n_kv,
                                         *blocking, num_iters=cfg["T"])
    torch.cuda.synchronize()
    check_close(got, ref, str(cfg))
    assert torch.equal(kg.cpu().float(), kc) and torch.equal(vg.cpu().float(), vc)


@pytest.mark.gpu
def test_status_watch_without_synchronising(sfb, monkeypatch):
    """Without SFM_CHECK_STATUS the Python layer mirrors the device status word to pinned memory every few
    calls and looks at the mirror on each call: healthy calls leave it at zero, a non-zero word left by a
    (here simulated) failed call makes the next call raise, and check_device_status() is the synchronous form."""
    from self_forcing_b200 import ops
    monkeypatch.delenv("SFM_CHECK_STATUS", raising=False)
    monkeypatch.setattr(ops, "_WATCH_EVERY", 2)
    c = small_case(0, 1)
    for _ in range(5):
        z, _, _ = run_gpu_cache(sfb, c)
    torch.cuda.synchronize()
    dev = torch.cuda.current_device()
    assert int(ops._status_mirror[dev][0][0]) == 0
    ops.check_device_status()
    ops._status_mirror[dev][0][0] = 31                   # what a softmax warp's timed-out wait would leave
    with pytest.raises(RuntimeError, match="device status 31"):
        run_gpu_cache(sfb, c)
    z2, _, _ = run_gpu_cache(sfb, c)                     # the report clears the mirror
    torch.cuda.synchronize()
    assert torch.equal(z, z2)


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_reports(sfb):
    """A device-side wait that nothing satisfies: the library's self-test kernel allocates tensor memory, waits a
    few thousand polls on an mbarrier nobody arrives at, gives up, stores its code in the workspace's status word,
    releases the tensor memory and returns.  The host then sees SFM_ERR_DEVICE_STATUS through the same reader the
    attention calls use, the context is still usable, and the next attention call on that workspace clears the
    word and is bit-equal to one made before."""
    from self_forcing_b200 import _lib, ops
    lib = _lib.load()
    c = small_case(0, 1)
    ref, _, _ = run_gpu_cache(sfb, c)
    torch.cuda.synchronize()
    dev = torch.cuda.current_device()
    ws = ops._workspaces[(dev, int(ops._stream().value or 0), "monarch")]
    assert lib.sfm_workspace_status(ops._ptr(ws), ops._stream()) == 0
    _lib.check(lib.sfm_selftest_bounded_wait(ops._ptr(ws), 4096, 77, ops._stream()), "sfm_selftest_bounded_wait")
    assert int(ws[:4].view(torch.int32)[0]) == 77
    assert lib.sfm_workspace_status(ops._ptr(ws), ops._stream()) == -7          # SFM_ERR_DEVICE_STATUS
    with pytest.raises(RuntimeError):
        ops.check_device_status()
    again, _, _ = run_gpu_cache(sfb, c)
    torch.cuda.synchronize()
    assert lib.sfm_workspace_status(ops._ptr(ws), ops._stream()) == 0
    assert torch.equal(ref, again)
    assert lib.sfm_selftest_bounded_wait(ops._ptr(ws), 0, 77, ops._stream()) == -2       # argument checks
    assert lib.sfm_selftest_bounded_wait(None, 16, 77, ops._stream()) == -1


@pytest.mark.gpu
def test_two_streams_use_separate_workspaces(sfb):
    """Calls queued on different streams may overlap on the GPU: each stream gets its own scratch, and both
    results equal the single-stream one."""
    from self_forcing_b200 import ops
    c = small_case(1, 1, H=3)
    ref, _, _ = run_gpu_cache(sfb, c)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for s in (s1, s2, s1, s2):
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            outs.append(run_gpu_cache(sfb, c)[0])
    torch.cuda.synchronize()
    keys = {k for k in ops._workspaces if k[1] in (s1.cuda_stream, s2.cuda_stream)}
    assert len(keys) == 2
    for o in outs:
        assert torch.equal(o, ref)


@pytest.mark.gpu
def test_recycled_workspace_does_not_raise_a_false_status(sfb):
    """A workspace that holds garbage (recycled allocator memory) must not read as a failed call: every path,
    the iterative one included, clears the status word before its first launch."""
    import ctypes as C
    from self_forcing_b200 import _lib
    lib = _lib.load()
    c = small_case(0, 2)
    B, n_q, H, D = c["q"].shape
    ft, hr, wr, h, w = c["blocking"]
    n_kv = c["n_kv"]
    kc, vc = c["kbuf"].cuda()[:, :n_kv].contiguous(), c["vbuf"].cuda()[:, :n_kv].contiguous()
    q = c["q"].cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: C.c_void_p(t.data_ptr())
    for iters in (2, 1):
        nbytes = lib.sfm_monarch_workspace_bytes(B, H, D, n_q, n_kv, ft, hr, wr, h, w, iters, 0)
        ws = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device="cuda")
        out = torch.empty_like(q)
        rc = lib.sfm_monarch_fwd(ptr(q), n_q * H * D, ptr(kc), ptr(vc), n_kv * H * D, ptr(out), ptr(ws), nbytes, B, H, D,
                                 n_q, n_kv, ft, hr, wr, h, w, D ** -0.5, iters, 0, stream)
        assert rc == 0
        assert lib.sfm_workspace_status(ptr(ws), stream) == 0
        ref = sfb.ops.monarch_attention_on_cache(q, kc, vc, ft, hr, wr, h, w, num_iters=iters)
        assert torch.equal(out, ref)


@pytest.mark.gpu
def test_dense_status_word_is_read_and_cleared(sfb):
    """check_device_status covers the dense kernels' status word: healthy calls leave it at zero."""
    import ctypes as C
    from self_forcing_b200 import _lib, ops
    lib = _lib.load()
    q = torch.randn(1, 256, 2, 128, device="cuda").bfloat16()
    sfb.attention(q, q, q)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.sfm_dense_status(stream) == 0
    ops.check_device_status()


@pytest.mark.gpu
@pytest.mark.parametrize("parts", [2, 8])
def test_norm_rope_token_slices_equal_the_whole_chunk(sfb, parts):
    """Sequence-parallel front end: RMSNorm + RoPE applied slice by slice (each slice knowing its first token's
    position in the chunk's grid) equals the one-pass kernel on the whole chunk bit for bit, with slices that cut
    through frames and rows."""
    from self_forcing_b200 import ops
    rng = np.random.default_rng(12)
    B, H, gh, gw = 2, 3, 6, 8
    n = 3 * gh * gw                                            # 144 tokens: 72 / 18 per slice
    q, k, v = (bf(cases.randn(rng, B, n, H, 128)).cuda() for _ in range(3))
    wq = bf(torch.from_numpy(rng.uniform(0.7, 1.3, size=H * 128).astype(np.float32))).cuda()
    wk = bf(torch.from_numpy(rng.uniform(0.7, 1.3, size=H * 128).astype(np.float32))).cuda()
    kc, vc = torch.zeros_like(k), torch.zeros_like(v)
    q_ref = ops.norm_rope_cache_write(q, k, v, kc, vc, 0, 5, 1, 1, 1, gh, gw, norm_q_weight=wq, norm_k_weight=wk,
                                      monarch_order=False)
    sp = n // parts
    for r in range(parts):
        sl = slice(r * sp, (r + 1) * sp)
        qo, ko, vo = (torch.empty(B, sp, H, 128, dtype=torch.bfloat16, device="cuda") for _ in range(3))
        ops.norm_rope_token_slice(q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous(), qo, ko, vo,
                                  r * sp, 5, gh, gw, norm_q_weight=wq, norm_k_weight=wk)
        torch.cuda.synchronize()
        assert torch.equal(qo, q_ref[:, sl]) and torch.equal(ko, kc[:, sl]) and torch.equal(vo, vc[:, sl])

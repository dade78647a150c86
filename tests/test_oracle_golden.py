"""The CPU oracle against every fixture produced from the reference's own functions."""
import numpy as np
import pytest
import torch

import cases
from oracle import monarch_oracle as orc

TOL = dict(rtol=2e-4, atol=2e-5)      # fp32 vs fp32, different summation order


@pytest.mark.parametrize("case", cases.MAP_CASES)
def test_maps_bit_exact(golden, case):
    ft, hr, wr, h, w, n = case
    key = f"map_{ft}_{hr}_{wr}_{h}_{w}_{n}"
    nat2mon, mon2nat = orc.token_maps(n, ft, hr, wr, h, w)
    assert np.array_equal(mon2nat, golden[key + "_mon2nat"].astype(np.int64))
    assert np.array_equal(nat2mon[mon2nat], np.arange(n))
    assert tuple(golden[key + "_dims"]) == orc.block_dims(n, ft, hr, wr, h, w)


def test_map_formula_matches_closed_form():
    ft, hr, wr, h, w, n = 3, 2, 4, 30, 52, 9360
    hh, ww = h // hr, w // wr
    nat2mon, _ = orc.token_maps(n, ft, hr, wr, h, w)
    idx = np.arange(n)
    j = idx % ww; t = idx // ww
    e = t % wr; t //= wr
    i = t % hh; t //= hh
    c = t % hr; t //= hr
    f = t % ft; a = t // ft
    mon = ((((a * hr + c) * wr + e) * ft + f) * hh + i) * ww + j
    assert np.array_equal(mon, nat2mon)


def test_rope_table(golden):
    cos, sin, split = orc.rope_table(128, 1024)
    assert split == (22, 21, 21)
    # fp64 tables; the reference builds them with torch.polar, a few ulp apart at most
    np.testing.assert_allclose(cos[:64].numpy(), golden["rope_freqs_re"], rtol=0, atol=1e-14)
    np.testing.assert_allclose(sin[:64].numpy(), golden["rope_freqs_im"], rtol=0, atol=1e-14)


@pytest.mark.parametrize("sf", [0, 9])
def test_rope_apply(golden, sf):
    x, grid = cases.rope_inputs()
    y = orc.rope_apply(x, grid, start_frame=sf)
    np.testing.assert_allclose(y.numpy(), golden[f"rope_out_sf{sf}"], rtol=0, atol=1e-6)


def test_rope_apply_bf16(golden):
    x, grid = cases.rope_inputs()
    y = orc.rope_apply(x.to(torch.bfloat16), grid, start_frame=9)
    assert y.dtype == torch.bfloat16
    assert np.array_equal(y.float().numpy(), golden["rope_out_bf16_sf9"])


@pytest.mark.parametrize("ci", range(len(cases.SMALL_BLOCKINGS)))
@pytest.mark.parametrize("iters", cases.SMALL_ITERS)
def test_cache_path(golden, ci, iters):
    c = cases.cache_case(ci, iters)
    kc, vc = c["kbuf"].clone(), c["vbuf"].clone()
    n_kv = c["n_kv"]
    z = orc.monarch_attn_with_kv_cache(c["q"], kc[:, :n_kv], vc[:, :n_kv], c["nk"], c["nv"],
                                       c["start"], c["end"], *c["blocking"], sm_scale=c["sm_scale"],
                                       num_iters=iters)
    key = f"cache_{c['name']}_T{iters}"
    np.testing.assert_allclose(z.numpy(), golden[key + "_z"], **TOL)
    s, e = c["start"], c["end"]
    assert torch.equal(kc[:, :s], c["kbuf"][:, :s]) and torch.equal(kc[:, e:], c["kbuf"][:, e:])
    assert torch.equal(vc[:, :s], c["vbuf"][:, :s]) and torch.equal(vc[:, e:], c["vbuf"][:, e:])
    if iters == 1:
        assert np.array_equal(kc[:, s:e].numpy(), golden[key + "_kc_written"])
        assert np.array_equal(vc[:, s:e].numpy(), golden[key + "_vc_written"])


@pytest.mark.parametrize("ci", range(4))
def test_nocache_path(golden, ci):
    c = cases.nocache_case(ci)
    for iters in cases.NOCACHE_ITERS:
        z = orc.monarch_attn(c["q"], c["k"], c["v"], *c["blocking"], sm_scale=c["sm_scale"], num_iters=iters)
        np.testing.assert_allclose(z.numpy(), golden[f"nocache_{c['name']}_T{iters}_z"], **TOL)
    z = orc.monarch_attn(c["q"], c["k"], c["v"], *c["blocking"], sm_scale=c["sm_scale"],
                         block_causal_size=c["block_causal"])
    np.testing.assert_allclose(z.numpy(), golden[f"nocache_{c['name']}_causal_z"], **TOL)


@pytest.mark.parametrize("blk", cases.REAL_BLOCKINGS)
def test_real_block_sizes(golden, blk):
    name, ft, hr, wr = blk
    c = cases.real_case()
    kc, vc = c["kbuf"].clone(), c["vbuf"].clone()
    z = orc.monarch_attn_with_kv_cache(c["q"], kc, vc, c["nk"], c["nv"], c["start"], c["end"],
                                       ft, hr, wr, c["h"], c["w"], sm_scale=c["sm_scale"])
    np.testing.assert_allclose(z[0, ::37, 0, :].numpy(), golden[f"real_{name}_z_sample"], **TOL)
    ref_sum = golden[f"real_{name}_z_sum"]
    assert abs(z.double().sum().item() - ref_sum[0]) <= 1e-4 * ref_sum[1]
    assert abs(z.double().abs().sum().item() - ref_sum[1]) <= 1e-5 * ref_sum[1]


def test_baseline_config1_T1(golden):
    c = cases.c1_case()
    kc, vc = torch.zeros_like(c["k"]), torch.zeros_like(c["v"])
    z = orc.monarch_attn_with_kv_cache(c["q"], kc, vc, c["k"], c["v"], 0, c["chunk"], 1, 1, 1,
                                       c["h"], c["w"], sm_scale=c["sm_scale"])
    np.testing.assert_allclose(z[0, ::97, ::5, :].numpy(), golden["c1_T1_z_sample"], **TOL)
    ref_sum = golden["c1_T1_z_sum"]
    assert abs(z.double().abs().sum().item() - ref_sum[1]) <= 1e-5 * ref_sum[1]


def test_dense_matches_sdpa():
    rng = np.random.default_rng(7)
    q, k, v = cases.randn(rng, 2, 50, 3, 32), cases.randn(rng, 2, 170, 3, 32), cases.randn(rng, 2, 170, 3, 32)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
    np.testing.assert_allclose(orc.dense_attention(q, k, v).numpy(), ref.numpy(), rtol=1e-4, atol=1e-5)


def test_cache_indices_rollout():
    """Chunk-wise rollout without a sliding window: 5 forwards per chunk rewrite the same slot."""
    g_end = l_end = 0
    for chunk in range(7):
        for _ in range(5):
            r = orc.cache_indices(chunk * 4680, 4680, g_end, l_end, 32760, 32760)
            assert r["roll"] is None and r["cache_start"] == 0
            assert (r["local_start"], r["local_end"]) == (chunk * 4680, (chunk + 1) * 4680)
            g_end, l_end = r["store_global_end"], r["store_local_end"]


def test_cache_indices_sliding_window():
    frame = 1560
    size = 9 * frame          # local_attn_size = 9 frames, 1 sink frame
    g_end = l_end = 0
    for chunk in range(5):
        r = orc.cache_indices(chunk * 3 * frame, 3 * frame, g_end, l_end, size, size,
                              local_attn_size=9, sink_tokens=frame)
        if chunk < 3:
            assert r["roll"] is None
        else:
            assert r["roll"] == (frame, frame + 3 * frame, 9 * frame - 3 * frame - frame)
            assert r["local_end"] == size and r["local_start"] == size - 3 * frame
        g_end, l_end = r["store_global_end"], r["store_local_end"]


def test_rms_norm_matches_reference_class(golden):
    """oracle.rms_norm against outputs of the reference's own WanRMSNorm (fp32 and bf16 module)."""
    x, w, eps = cases.rmsnorm_inputs()
    np.testing.assert_allclose(orc.rms_norm(x, w, eps).numpy(), golden["rmsnorm_fp32"], rtol=1e-6, atol=1e-6)
    got = orc.rms_norm(x.to(torch.bfloat16), w.to(torch.bfloat16), eps).float().numpy()
    assert np.array_equal(got, golden["rmsnorm_bf16"])

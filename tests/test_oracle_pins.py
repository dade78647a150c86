"""The CPU oracle and the host-side bookkeeping against the second fixture file (pins_golden.npz):
gradients from the reference's own gradient oracle, its dense attention, and the index arithmetic of its
CausalWanSelfAttention.forward recorded call by call (tests/golden/make_golden.py says how each was made)."""
import numpy as np
import pytest
import torch

import cases
from oracle import monarch_oracle as orc

TOL = dict(rtol=1e-3, atol=1e-4)      # fp32 vs fp32 through two different autograd graphs (values of order 0.1 - 1)
CS = cases.PIN_CHANNEL_STRIDE
FRAME = 30 * 52


@pytest.fixture(scope="module")
def pins():
    from conftest import ROOT
    return np.load(ROOT / "tests" / "golden" / "pins_golden.npz")


def oracle_cache_grads(c):
    """Gradients through the oracle in the reference's convention: the cache gradient is the one taken after
    the in-place write, i.e. over the written slot it is the new keys' gradient in Monarch order."""
    q = c["q"].clone().requires_grad_()
    nk, nv = c["nk"].clone().requires_grad_(), c["nv"].clone().requires_grad_()
    kb, vb = c["kbuf"].clone().requires_grad_(), c["vbuf"].clone().requires_grad_()
    kc, vc = kb.clone(), vb.clone()
    z = orc.monarch_attn_with_kv_cache(q, kc[:, :c["n_kv"]], vc[:, :c["n_kv"]], nk, nv, c["start"], c["end"],
                                       *c["blocking"], sm_scale=c["sm_scale"])
    z.backward(c["g"])
    dkc, dvc = kb.grad[:, :c["n_kv"]].clone(), vb.grad[:, :c["n_kv"]].clone()
    s, e = c["start"], c["end"]
    assert not dkc[:, s:e].any() and not dvc[:, s:e].any()
    dkc[:, s:e] = orc.to_monarch_order(nk.grad, *c["blocking"]).reshape(dkc[:, s:e].shape)
    dvc[:, s:e] = orc.to_monarch_order(nv.grad, *c["blocking"]).reshape(dvc[:, s:e].shape)
    return dict(z=z.detach(), dq=q.grad, dnk=nk.grad, dnv=nv.grad, dkc=dkc, dvc=dvc)


@pytest.mark.parametrize("ci", range(len(cases.SMALL_BLOCKINGS)))
def test_oracle_gradients_match_reference(pins, ci):
    c = cases.grad_case(ci)
    got = oracle_cache_grads(c)
    for name, val in got.items():
        ref = pins[f"grad_{c['name']}_{name}"]
        np.testing.assert_allclose(val[..., ::CS].numpy(), ref, err_msg=name, **TOL)


@pytest.mark.parametrize("i", range(len(cases.CAUSAL_GRAD_CASES)))
def test_oracle_block_causal_gradients_match_reference(pins, i):
    c = cases.causal_grad_case(i)
    q, k, v = (c[n].clone().requires_grad_() for n in ("q", "k", "v"))
    z = orc.monarch_attn(q, k, v, *c["blocking"], sm_scale=c["sm_scale"], block_causal_size=c["block_causal"])
    z.backward(c["g"])
    for name, t in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
        np.testing.assert_allclose(t[..., ::CS].numpy(), pins[f"causalgrad_{c['name']}_{name}"], err_msg=name, **TOL)


@pytest.mark.parametrize("i", range(len(cases.DENSE_CASES)))
def test_oracle_dense_matches_reference_attention(pins, i):
    """The dense oracle against the reference's attention() run through its own SDPA branch in fp32; the
    same call with the function's default bf16 cast stays within the bf16 acceptance rule of the fp32 run."""
    c = cases.dense_case(i)
    k, v = c["kbuf"][:, :c["n_kv"]], c["vbuf"][:, :c["n_kv"]]
    ref = pins[f"dense_{i}_fp32"]
    np.testing.assert_allclose(orc.dense_attention(c["q"], k, v).numpy(), ref, rtol=2e-4, atol=2e-5)
    low = torch.from_numpy(pins[f"dense_{i}_bf16_bits"]).view(torch.bfloat16).float().numpy()
    assert np.abs(low - ref).max() <= 2e-2
    assert np.linalg.norm(low - ref) / np.linalg.norm(ref) <= 1e-2


def replay(sc, step_fn):
    """Replays one recorded rollout with an integer model of the cache: `step_fn` returns
    (roll, cache_start, local_start, local_end, store_global_end, store_local_end) for each call."""
    n_cache = sc["cache_frames"] * FRAME
    ids = -(np.arange(n_cache, dtype=np.int64) + 1)
    g_end = l_end = 0
    rows, id_rows = [], []
    for chunk, repeats in sc["calls"]:
        for _ in range(repeats):
            cur = chunk * 3 * FRAME
            roll, c0, ls, le, sg, sl = step_fn(cur, 3 * FRAME, g_end, l_end, n_cache)
            if roll is not None:
                dst, src, cnt = roll
                ids[dst:dst + cnt] = ids[src:src + cnt].copy()
            ids[c0 + ls:c0 + le] = cur + np.arange(3 * FRAME) + 1
            rows.append([cur, g_end, l_end, c0, le, ls, le, sg, sl])
            id_rows.append(ids[::cases.BOOKKEEPING_ID_STRIDE].copy())
            g_end, l_end = sg, sl
    return np.array(rows), np.stack(id_rows)


@pytest.mark.parametrize("name", list(cases.BOOKKEEPING_SCENARIOS))
@pytest.mark.parametrize("which", ["product", "oracle"])
def test_cache_bookkeeping_matches_reference_module(pins, name, which):
    """plan_cache_step (product) and cache_indices (oracle) against what the reference module did: the view
    it handed to the attention operator, the slot written, the stored end indices and, through the token ids,
    the eviction shift."""
    sc = cases.BOOKKEEPING_SCENARIOS[name]
    max_att = 21 * FRAME if sc["local_attn_size"] == -1 else sc["local_attn_size"] * FRAME
    sink = sc["sink_size"] * FRAME
    if which == "product":
        from self_forcing_b200.layer import plan_cache_step

        def step_fn(cur, n, g, l, size):
            s = plan_cache_step(cur, n, g, l, size, max_att, sc["local_attn_size"], sink)
            return s.roll, s.cache_start, s.local_start, s.local_end, s.store_global_end, s.store_local_end
    else:
        def step_fn(cur, n, g, l, size):
            r = orc.cache_indices(cur, n, g, l, size, max_att, sc["local_attn_size"], sink)
            return (r["roll"], r["cache_start"], r["local_start"], r["local_end"], r["store_global_end"],
                    r["store_local_end"])
    rows, ids = replay(sc, step_fn)
    ref = pins[f"book_{name}_calls"]
    # recorded columns: current_start, global_end before, local_end before, branch, view offset, view length,
    # slot start, slot end, stored global_end, stored local_end
    assert np.array_equal(rows[:, :3], ref[:, :3])
    assert np.array_equal(rows[:, 3:], ref[:, 4:]), "view / slot / stored indices differ"
    assert np.array_equal(ids, pins[f"book_{name}_ids"].astype(np.int64)), "cache contents (eviction) differ"
    if sc.get("dense_init"):
        # dense branch exactly while the view is a single chunk
        assert np.array_equal(ref[:, 3] == 1, ref[:, 5] == 3 * FRAME)
    else:
        assert not ref[:, 3].any()

"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, and its
host-only entry points (maps, rotary table, planning, argument validation) agree with the oracle."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import cases
from oracle import monarch_oracle as orc

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def sfb():
    import self_forcing_b200
    return self_forcing_b200


def declared_symbols():
    text = (ROOT / "include" / "sfmonarch.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sfm_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_exported_and_bound(sfb):
    from self_forcing_b200 import _lib
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in sfmonarch.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)
    assert lib.sfm_version() >= 100
    assert lib.sfm_error_string(-2).decode().startswith("sizes")


@pytest.mark.parametrize("case", cases.MAP_CASES)
def test_maps_bit_exact(sfb, golden, case):
    ft, hr, wr, h, w, n = case
    nat2mon, mon2nat = sfb.build_maps(n, ft, hr, wr, h, w)
    key = f"map_{ft}_{hr}_{wr}_{h}_{w}_{n}"
    assert np.array_equal(mon2nat, golden[key + "_mon2nat"])
    o_nat2mon, o_mon2nat = orc.token_maps(n, ft, hr, wr, h, w)
    assert np.array_equal(nat2mon, o_nat2mon) and np.array_equal(mon2nat, o_mon2nat)


def test_maps_reject_bad_shapes(sfb):
    with pytest.raises(ValueError):
        sfb.build_maps(100, 1, 1, 1, 30, 52)      # not a whole frame
    with pytest.raises(ValueError):
        sfb.build_maps(1560, 1, 4, 1, 30, 52)     # 4 does not divide 30


def test_rope_table_matches_oracle(sfb):
    from self_forcing_b200 import _lib
    host = np.empty((1024, 64, 2), dtype=np.float32)
    assert _lib.load().sfm_rope_table(host.ctypes.data_as(C.c_void_p), 128, 1024, 10000.0) == 0
    cos, sin, _ = orc.rope_table(128, 1024)
    assert np.array_equal(host[..., 0], cos.numpy().astype(np.float32))
    assert np.array_equal(host[..., 1], sin.numpy().astype(np.float32))


def test_workspace_planning(sfb):
    # framewise, 7 chunks cached: the bridge of one head is 3*52 columns x 630 keys x 516 bytes
    per_head = 3 * 52 * 630 * (2 * 128 * 2 + 4)
    got = sfb.workspace_bytes(1, 12, 4680, 32760, 1, 1, 1, 30, 52, bridge_budget_bytes=per_head + 4096)
    assert per_head <= got <= per_head + 8192
    got2 = sfb.workspace_bytes(1, 12, 4680, 32760, 1, 1, 1, 30, 52, bridge_budget_bytes=3 * per_head)
    assert 3 * per_head <= got2 <= 3 * per_head + 8192
    # a budget below one query group still plans one group per chunk
    small = sfb.workspace_bytes(1, 12, 4680, 32760, 1, 1, 1, 30, 52, bridge_budget_bytes=1 << 20)
    assert per_head // 3 <= small <= per_head // 3 + 8192
    # invalid sizes plan to zero bytes
    assert sfb.workspace_bytes(1, 12, 4680, 32761, 1, 1, 1, 30, 52) == 0
    assert sfb.workspace_bytes(1, 12, 4000, 32760, 1, 1, 1, 30, 52) == 0


def test_ops_refuse_cpu_tensors(sfb):
    import torch
    q = torch.zeros(1, 1560, 1, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        sfb.monarch_attn_with_kv_cache(q, q.clone(), q.clone(), q, q, 0, 1560, 1, 1, 1, 30, 52)
    with pytest.raises(RuntimeError):
        sfb.attention(q, q, q)


def test_entry_points_validate_arguments_without_a_gpu(sfb):
    """Argument checks run before any CUDA call, so they can be exercised on a CPU-only box."""
    from self_forcing_b200 import _lib
    lib = _lib.load()
    null = C.c_void_p(0)
    one = C.c_void_p(256)
    assert lib.sfm_dense_fwd(null, 0, null, null, 0, null, 1, 1, 128, 16, 16, 1.0, null) == -1
    assert lib.sfm_dense_fwd(one, 0, one, one, 0, one, 1, 1, 64, 16, 16, 1.0, null) == -3
    assert lib.sfm_dense_fwd(C.c_void_p(260), 0, one, one, 0, one, 1, 1, 128, 16, 16, 1.0, null) == -4
    assert lib.sfm_monarch_fwd(one, 0, one, one, 0, one, one, 0, 1, 1, 128, 1560, 1560, 1, 1, 1, 30, 52,
                               1.0, 1, 0, null) == -5
    assert lib.sfm_monarch_fwd(one, 0, one, one, 0, one, one, 1 << 30, 1, 1, 128, 1000, 1560, 1, 1, 1, 30, 52,
                               1.0, 1, 0, null) == -2
    assert lib.sfm_rope_cache_write(null, one, one, null, one, one, 0, null, 1, 100, 1, 128, 0, 1, 1, 1, 30, 52,
                                    0, 1, null) == -2
    # fused RMSNorm front end: both weights and q are required
    assert lib.sfm_norm_rope_cache_write(one, one, one, null, one, 1e-6, one, one, one, 0, null, 1, 1560, 1, 128, 0,
                                         1, 1, 1, 30, 52, 0, 1, null) == -1
    assert lib.sfm_norm_rope_cache_write(null, one, one, one, one, 1e-6, one, one, one, 0, null, 1, 1560, 1, 128, 0,
                                         1, 1, 1, 30, 52, 0, 1, null) == -1
    # backward: null gradient, workspace too small, group range outside the cache, block rows above 128
    big = 1 << 40
    assert lib.sfm_monarch_bwd(one, 0, one, one, 0, null, one, one, one, one, big, 1, 1, 128, 1560, 3120, 1, 1, 1,
                               30, 52, 1.0, 0, 2, 0, 0, null) == -1
    assert lib.sfm_monarch_bwd(one, 0, one, one, 0, one, one, one, one, one, 0, 1, 1, 128, 1560, 3120, 1, 1, 1,
                               30, 52, 1.0, 0, 2, 0, 0, null) == -5
    assert lib.sfm_monarch_bwd(one, 0, one, one, 0, one, one, one, one, one, big, 1, 1, 128, 1560, 3120, 1, 1, 1,
                               30, 52, 1.0, 1, 3, 0, 0, null) == -2
    assert lib.sfm_monarch_bwd(one, 0, one, one, 0, one, one, null, null, one, big, 1, 1, 128, 1560, 3120, 1, 1, 1,
                               30, 52, 1.0, 0, 2, 0, 0, null) == -1
    # block-causal needs n_q == n_kv
    assert lib.sfm_monarch_bwd(one, 0, one, one, 0, one, one, one, one, one, big, 1, 1, 128, 1560, 3120, 1, 1, 1,
                               30, 52, 1.0, 0, 2, 1, 0, null) == -2
    assert lib.sfm_monarch_bwd_workspace_bytes(1, 1, 128, 5 * 30 * 52, 5 * 30 * 52, 5, 1, 1, 30, 52, 0) == 0
    per_bh = 1 * 52 * (2 * 30) * (2 * 128 + 2) * 4           # aL, Y, cL, dcL of one (batch, head) pair
    dq2 = 1 * 1560 * 2 * 128 * 4                              # second dQ buffer, whole call
    # on top of the fp32 kernels' scratch: what the tensor-core path lays out differently (a scratch output, delta and
    # log-sum-exp rows, and one fp32 copy of dK / dV per tile of query groups as far as the bf16 bridge leaves no room)
    def extras(nbh):
        return 1560 * 2 * (128 * 2 + 4) + 2 * nbh * 3120 * 128 * 4 + (1 << 16)
    assert 0 <= lib.sfm_monarch_bwd_workspace_bytes(1, 2, 128, 1560, 3120, 1, 1, 1, 30, 52, 0) - 2 * per_bh - dq2 <= extras(2)
    assert 0 <= lib.sfm_monarch_bwd_workspace_bytes(1, 2, 128, 1560, 3120, 1, 1, 1, 30, 52, per_bh) - per_bh - dq2 <= extras(1)
    # head-sharded entry points: rank / world range, shard pointers, divisibility of the chunk
    ptrs = (C.c_void_p * 2)(256, 512)
    holes = (C.c_void_p * 2)(256, 0)
    assert lib.sfm_rope_cache_write_gather(ptrs, ptrs, ptrs, 9, 0, one, one, one, 0, null, 1, 1560, 1, 128, 0,
                                           1, 1, 1, 30, 52, 0, 1, null) == -2
    assert lib.sfm_rope_cache_write_gather(ptrs, ptrs, ptrs, 2, 2, one, one, one, 0, null, 1, 1560, 1, 128, 0,
                                           1, 1, 1, 30, 52, 0, 1, null) == -2
    assert lib.sfm_rope_cache_write_gather(ptrs, holes, ptrs, 2, 0, one, one, one, 0, null, 1, 1560, 1, 128, 0,
                                           1, 1, 1, 30, 52, 0, 1, null) == -1
    assert lib.sfm_rope_cache_write_gather(ptrs, ptrs, ptrs, 2, 0, one, one, one, 0, null, 1, 1561, 1, 128, 0,
                                           1, 1, 1, 30, 52, 0, 1, null) == -2
    assert lib.sfm_monarch_fwd_scatter(one, 0, one, one, 0, holes, 2, 0, one, 1 << 30, 1, 1, 128, 1560, 1560,
                                       1, 1, 1, 30, 52, 1.0, 0, null) == -1
    assert lib.sfm_monarch_fwd_scatter(one, 0, one, one, 0, ptrs, 2, 5, one, 1 << 30, 1, 1, 128, 1560, 1560,
                                       1, 1, 1, 30, 52, 1.0, 0, null) == -2
    # block rows above 128 (tied3frame at 480p: 90 is fine; 3 x 60 = 180 is not) cannot scatter
    assert lib.sfm_monarch_fwd_scatter(one, 0, one, one, 0, ptrs, 2, 0, one, 1 << 34, 1, 1, 128, 3 * 60 * 52,
                                       3 * 60 * 52, 3, 1, 1, 60, 52, 1.0, 0, null) == -3


def test_plan_cache_step_equals_oracle(sfb):
    """The product's cache bookkeeping against the oracle's restatement of causal_model.py:907-938,
    over a random walk of rollouts with and without a sliding window (integers: exact)."""
    from oracle import monarch_oracle as orc
    import random
    rnd = random.Random(5)
    frame = 1560
    for trial in range(200):
        window = rnd.choice([-1, 6, 9, 12, 21])
        sink = rnd.choice([0, 1, 3]) if window != -1 else 0
        size = 21 * frame if window == -1 else window * frame
        max_att = size if rnd.random() < 0.7 else rnd.choice([6, 9]) * frame
        g_end = l_end = 0
        chunk = 0
        for _ in range(rnd.randint(1, 14)):
            repeat = rnd.random() < 0.5 and chunk > 0       # re-denoise the same chunk: same current_start
            if not repeat:
                chunk += 1
            cur = (chunk - 1) * 3 * frame
            a = orc.cache_indices(cur, 3 * frame, g_end, l_end, size, max_att, local_attn_size=window,
                                  sink_tokens=sink * frame)
            b = sfb.plan_cache_step(cur, 3 * frame, g_end, l_end, size, max_att, local_attn_size=window,
                                    sink_tokens=sink * frame)
            assert (b.roll, b.cache_start, b.local_start, b.local_end, b.store_global_end, b.store_local_end) == \
                   (a["roll"], a["cache_start"], a["local_start"], a["local_end"], a["store_global_end"],
                    a["store_local_end"])
            g_end, l_end = b.store_global_end, b.store_local_end
            if window == -1 and chunk >= 7:
                break


def test_cache_roll_in_place_equals_copy_through_temporary(sfb):
    """KVCache._roll shifts in place, piece by piece; the reference clones the source range first
    (causal_model.py:917-926).  Same result for every overlap pattern."""
    import torch
    for dst, src, count in [(48, 192, 240), (0, 144, 288), (48, 96, 300), (5, 6, 100), (0, 300, 100), (7, 7, 50)]:
        k = torch.arange(2 * 600 * 128, dtype=torch.float32).reshape(2, 600, 1, 128).to(torch.bfloat16)
        v = k.clone() + 1
        ref_k, ref_v = k.clone(), v.clone()
        ref_k[:, dst:dst + count] = k[:, src:src + count].clone()
        ref_v[:, dst:dst + count] = v[:, src:src + count].clone()
        c = sfb.KVCache(k, v)
        c._roll((dst, src, count))
        assert torch.equal(c.k, ref_k) and torch.equal(c.v, ref_v), (dst, src, count)


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs without a GPU (the CPU oracle port on the host cores) and prints one
    JSON line with the keys the bench contract asks of the reference arm."""
    import json
    import subprocess
    import sys
    root = Path(__file__).resolve().parents[1]
    out = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=str(root))
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["higher_is_better"] is True and line["n_gpus"] == 1
    for key in ("metric", "value", "unit", "steps", "warmup", "ms_per_step", "scaling", "vs_baseline", "dtype", "data",
                "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert "workload" in line["config"] and "model" not in line["config"]

"""Generate the golden fixtures in this directory from the reference's own code.

Run once, in a container that has the reference checkout (default
``/root/reference``; override with ``SF_REFERENCE_ROOT``):

    python tests/golden/make_golden.py

The reference module ``wan/modules/monarch_attn.py`` cannot be imported without
a CUDA driver (it asserts on a Triton target at import time), so its
pure-PyTorch functions are pulled out of the file with ``ast`` and executed on
the CPU in fp32 with ``torch`` and ``einops.rearrange`` in scope.  No reference
source text is written into this repository: only numeric inputs and outputs.

Inputs come from ``numpy.random.default_rng(seed)`` so that tests can rebuild
the large ones from the seed instead of storing them.
"""
from __future__ import annotations

import ast
import math
import os
import sys
import textwrap
from pathlib import Path

import numpy as np
import torch
from einops import rearrange

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402
REF = Path(os.environ.get("SF_REFERENCE_ROOT", "/root/reference"))


def _extract(path: Path, names):
    src = path.read_text()
    tree = ast.parse(src)
    wanted = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    missing = set(names) - {n.name for n in wanted}
    if missing:
        raise RuntimeError(f"not found in {path}: {missing}")
    ns = {"torch": torch, "nn": torch.nn, "rearrange": rearrange, "math": math}
    code = ast.Module(body=wanted, type_ignores=[])
    exec(compile(code, str(path), "exec"), ns)
    return ns


def load_reference():
    ns = _extract(REF / "wan/modules/monarch_attn.py",
                  ["_get_rearrange_fns", "monarch_attn_slow", "monarch_attn_ref_op",
                   "monarch_attn_with_kv_cache_ref", "monarch_attn_causal_ref"])
    ns_model = _extract(REF / "wan/modules/model.py", ["rope_params", "WanRMSNorm"])
    ns_causal = _extract(REF / "wan/modules/causal_model.py", ["causal_rope_apply"])
    return ns, ns_model, ns_causal


def ref_slow_with_cache(ns, q, kc, vc, nk, nv, s, e, ft, hr, wr, h, w, sm_scale, iters):
    """The num_iters != 1 branch of the reference's cache entry point
    (monarch_attn.py:1788-1795), composed from the extracted functions."""
    b, _, nh, d = q.shape
    fn, ret = ns["_get_rearrange_fns"](q, ft, hr, wr, h, w)
    qb = fn(q).contiguous()
    nk = fn(nk).reshape(b, -1, nh, d)
    nv = fn(nv).reshape(b, -1, nh, d)
    kc[:, s:e] = nk
    vc[:, s:e] = nv
    b1, b2 = qb.shape[2], qb.shape[3]
    kb = kc.reshape(b, -1, b1, b2, nh, d)
    vb = vc.reshape(b, -1, b1, b2, nh, d)
    return ret(ns["monarch_attn_slow"](qb, kb, vb, sm_scale, num_iters=iters))


def ref_nocache(ns, q, k, v, ft, hr, wr, h, w, sm_scale, iters):
    fn, ret = ns["_get_rearrange_fns"](q, ft, hr, wr, h, w)
    qb, kb, vb = fn(q).contiguous(), fn(k).contiguous(), fn(v).contiguous()
    if iters == 1:
        return ret(ns["monarch_attn_ref_op"](qb, kb, vb, sm_scale))
    return ret(ns["monarch_attn_slow"](qb, kb, vb, sm_scale, num_iters=iters))


def main():
    torch.set_num_threads(os.cpu_count() or 1)
    ns, ns_model, ns_causal = load_reference()
    out = {}

    # ---- 1. integer maps -------------------------------------------------
    for (ft, hr, wr, h, w, n) in cases.MAP_CASES:
        x = torch.arange(n, dtype=torch.float64).view(1, n, 1, 1)
        fn, ret = ns["_get_rearrange_fns"](x, ft, hr, wr, h, w)
        blk = fn(x)
        g, b1, b2 = blk.shape[1:4]
        mon2nat = blk.reshape(-1).to(torch.int64).numpy()
        back = ret(blk).reshape(-1).to(torch.int64).numpy()
        assert (back == np.arange(n)).all()
        key = f"map_{ft}_{hr}_{wr}_{h}_{w}_{n}"
        out[key + "_mon2nat"] = mon2nat.astype(np.int32)
        out[key + "_dims"] = np.array([g, b1, b2], dtype=np.int32)

    # ---- 2. RoPE ----------------------------------------------------------
    d = 128
    freqs = torch.cat([ns_model["rope_params"](1024, d - 4 * (d // 6)),
                       ns_model["rope_params"](1024, 2 * (d // 6)),
                       ns_model["rope_params"](1024, 2 * (d // 6))], dim=1)
    out["rope_freqs_re"] = freqs.real[:64].numpy()      # fp64 [64, 64]
    out["rope_freqs_im"] = freqs.imag[:64].numpy()
    x, g3 = cases.rope_inputs()
    grid = torch.tensor([list(g3), list(g3)])
    for sf in (0, 9):
        out[f"rope_out_sf{sf}"] = ns_causal["causal_rope_apply"](x, grid, freqs, start_frame=sf).numpy()
    xb = x.to(torch.bfloat16)
    out["rope_out_bf16_sf9"] = ns_causal["causal_rope_apply"](xb, grid, freqs, start_frame=9).float().numpy().astype(np.float32)

    # ---- 3. small Monarch cases, cache path -------------------------------
    for ci in range(len(cases.SMALL_BLOCKINGS)):
        for iters in cases.SMALL_ITERS:
            c = cases.cache_case(ci, iters)
            ft, hr, wr, h, w = c["blocking"]
            s, e, n_kv = c["start"], c["end"], c["n_kv"]
            kc, vc = c["kbuf"].clone(), c["vbuf"].clone()
            if iters == 1:
                z = ns["monarch_attn_with_kv_cache_ref"](c["q"], kc[:, :n_kv], vc[:, :n_kv], c["nk"], c["nv"],
                                                         s, e, ft, hr, wr, h, w, c["sm_scale"],
                                                         grad_only_new_kv=True)
            else:
                z = ref_slow_with_cache(ns, c["q"], kc[:, :n_kv], vc[:, :n_kv], c["nk"], c["nv"], s, e,
                                        ft, hr, wr, h, w, c["sm_scale"], iters)
            key = f"cache_{c['name']}_T{iters}"
            out[key + "_z"] = z.numpy()
            # side effect: only [s, e) may change; keep that slice (exact values)
            assert torch.equal(kc[:, :s], c["kbuf"][:, :s]) and torch.equal(kc[:, e:], c["kbuf"][:, e:])
            assert torch.equal(vc[:, :s], c["vbuf"][:, :s]) and torch.equal(vc[:, e:], c["vbuf"][:, e:])
            if iters == 1:
                out[key + "_kc_written"] = kc[:, s:e].numpy()
                out[key + "_vc_written"] = vc[:, s:e].numpy()

    # ---- 4. no-cache entry point, plain and block causal -------------------
    for ci in range(4):
        c = cases.nocache_case(ci)
        ft, hr, wr, h, w = c["blocking"]
        for iters in cases.NOCACHE_ITERS:
            out[f"nocache_{c['name']}_T{iters}_z"] = ref_nocache(ns, c["q"], c["k"], c["v"], ft, hr, wr, h, w,
                                                                 c["sm_scale"], iters).numpy()
        out[f"nocache_{c['name']}_causal_z"] = ns["monarch_attn_causal_ref"](
            c["q"], c["k"], c["v"], ft, hr, wr, h, w, c["block_causal"], c["sm_scale"]).numpy()

    # ---- 5. one head of the real block sizes (30x52, D=128) ----------------
    c = cases.real_case()
    for name, ft, hr, wr in cases.REAL_BLOCKINGS:
        kc, vc = c["kbuf"].clone(), c["vbuf"].clone()
        z = ns["monarch_attn_with_kv_cache_ref"](c["q"], kc, vc, c["nk"], c["nv"], c["start"], c["end"],
                                                 ft, hr, wr, c["h"], c["w"], c["sm_scale"],
                                                 grad_only_new_kv=True)
        out[f"real_{name}_z_sample"] = z[0, ::37, 0, :].numpy()
        out[f"real_{name}_z_sum"] = np.array([z.double().sum().item(), z.double().abs().sum().item()])

    # ---- 6. BASELINE config 1: 12 heads, first chunk, empty cache ----------
    c = cases.c1_case()
    n = c["chunk"]
    for iters in (1, 20):
        kc = torch.zeros_like(c["k"]); vc = torch.zeros_like(c["v"])
        if iters == 1:
            z = ns["monarch_attn_with_kv_cache_ref"](c["q"], kc, vc, c["k"], c["v"], 0, n, 1, 1, 1,
                                                     c["h"], c["w"], c["sm_scale"], grad_only_new_kv=True)
        else:
            z = ref_slow_with_cache(ns, c["q"], kc, vc, c["k"], c["v"], 0, n, 1, 1, 1, c["h"], c["w"],
                                    c["sm_scale"], iters)
        out[f"c1_T{iters}_z_sample"] = z[0, ::97, ::5, :].numpy()
        out[f"c1_T{iters}_z_sum"] = np.array([z.double().sum().item(), z.double().abs().sum().item()])

    # ---- 7. full-width RMS normalisation of q / k (WanRMSNorm, model.py:462-478) ----------
    x, wgt, eps = cases.rmsnorm_inputs()
    norm = ns_model["WanRMSNorm"](x.shape[-1], eps=eps)
    with torch.no_grad():
        norm.weight.copy_(wgt)
        out["rmsnorm_fp32"] = norm(x).numpy()
        norm_b = norm.to(torch.bfloat16)
        out["rmsnorm_bf16"] = norm_b(x.to(torch.bfloat16)).float().numpy()

    np.savez_compressed(HERE / "monarch_golden.npz", **out)
    sz = (HERE / "monarch_golden.npz").stat().st_size
    print(f"wrote {len(out)} arrays, {sz/1e6:.2f} MB")


if __name__ == "__main__":
    sys.exit(main())

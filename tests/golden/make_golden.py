"""Generate the golden fixtures in this directory from the reference's own code.

Run once, in a container that has the reference checkout, with ``SF_REFERENCE_ROOT`` pointing at it:

    SF_REFERENCE_ROOT=/path/to/Self-Forcing python tests/golden/make_golden.py [--only-pins]

Two files are written: ``monarch_golden.npz`` (layout maps, RoPE, RMSNorm, forward results) and
``pins_golden.npz`` (gradients, dense attention, KV-cache bookkeeping); ``--only-pins`` regenerates the
second one alone.

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
if not os.environ.get("SF_REFERENCE_ROOT"):
    sys.exit("set SF_REFERENCE_ROOT to a checkout of the reference project")
REF = Path(os.environ["SF_REFERENCE_ROOT"])
ROOT = HERE.parent.parent


def _extract(path: Path, names, extra=None):
    src = path.read_text()
    tree = ast.parse(src)
    wanted = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    missing = set(names) - {n.name for n in wanted}
    if missing:
        raise RuntimeError(f"not found in {path}: {missing}")
    ns = {"torch": torch, "nn": torch.nn, "rearrange": rearrange, "math": math}
    ns.update(extra or {})
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


# =============================================================================================
# pins_golden.npz
# =============================================================================================
def gradient_pins(ns, out):
    """Gradients from the reference's own gradient oracle: autograd through monarch_attn_with_kv_cache_ref
    (monarch_attn.py:1860-1878), used the way run_kv_cache_test does (:1880-1932): q, new_k, new_v are
    leaves; the cache tensors are not, and with grad_only_new_kv=False their retained gradient (taken
    after the in-place write, so it covers the written slot too) is the cache gradient."""
    for ci in range(len(cases.SMALL_BLOCKINGS)):
        c = cases.grad_case(ci)
        ft, hr, wr, h, w = c["blocking"]
        res = {}
        for only_new in (False, True):
            q = c["q"].clone().requires_grad_(True)
            nk, nv = c["nk"].clone().requires_grad_(True), c["nv"].clone().requires_grad_(True)
            kc, vc = c["kbuf"][:, :c["n_kv"]].clone(), c["vbuf"][:, :c["n_kv"]].clone()
            z = ns["monarch_attn_with_kv_cache_ref"](q, kc, vc, nk, nv, c["start"], c["end"], ft, hr, wr, h, w,
                                                     c["sm_scale"], grad_only_new_kv=only_new)
            z.backward(c["g"])
            res[only_new] = dict(z=z.detach(), dq=q.grad, dnk=nk.grad, dnv=nv.grad,
                                 dkc=None if only_new else kc.grad, dvc=None if only_new else vc.grad)
        for name in ("z", "dq", "dnk", "dnv"):          # the mode only decides which gradients exist
            assert torch.equal(res[False][name], res[True][name])
        key = f"grad_{c['name']}"
        for name, val in res[False].items():
            out[f"{key}_{name}"] = val[..., ::cases.PIN_CHANNEL_STRIDE].numpy()
    for i in range(len(cases.CAUSAL_GRAD_CASES)):
        c = cases.causal_grad_case(i)
        ft, hr, wr, h, w = c["blocking"]
        q, k, v = (c[n].clone().requires_grad_(True) for n in ("q", "k", "v"))
        z = ns["monarch_attn_causal_ref"](q, k, v, ft, hr, wr, h, w, c["block_causal"], c["sm_scale"])
        z.backward(c["g"])
        key = f"causalgrad_{c['name']}"
        cs = cases.PIN_CHANNEL_STRIDE
        out[key + "_dq"] = q.grad[..., ::cs].numpy()
        out[key + "_dk"], out[key + "_dv"] = k.grad[..., ::cs].numpy(), v.grad[..., ::cs].numpy()


def dense_pins(out):
    """The reference's dense attention() with its flash-attn branch switched off, i.e. its own SDPA
    fallback (attention.py:177-187): once in fp32 (the parity target) and once with the default
    dtype=bfloat16 cast the function applies (recorded for information)."""
    import warnings
    ns = _extract(REF / "wan/modules/attention.py", ["attention"],
                  extra={"FLASH_ATTN_2_AVAILABLE": False, "FLASH_ATTN_3_AVAILABLE": False, "warnings": warnings})
    for i in range(len(cases.DENSE_CASES)):
        c = cases.dense_case(i)
        k, v = c["kbuf"][:, :c["n_kv"]], c["vbuf"][:, :c["n_kv"]]
        out[f"dense_{i}_fp32"] = ns["attention"](c["q"], k, v, dtype=torch.float32).numpy()
        out[f"dense_{i}_bf16_bits"] = ns["attention"](c["q"], k, v).contiguous().view(torch.int16).numpy()


def bookkeeping_pins(out):
    """Replays rollouts through the reference's CausalWanSelfAttention.forward (cache branch,
    causal_model.py:900-1103) on the CPU.  The attention operators are replaced by stand-ins that perform
    the cache write the real ones do and return zeros; what is recorded is pure index arithmetic: per
    call the view the operator was given (offset into the cache and length), the slot it wrote, the two
    end indices the module stored afterwards, and which token sits where in the cache (token ids kept
    in one element of every cache row, so that the eviction shift is captured as the module performs it)."""
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_harness as rh
    rh.prepare_imports(REF, attention="ours")
    import wan.modules.causal_model as cm

    frame = 30 * 52
    rec = {}

    def view_of(cache_k, view):
        row = cache_k.stride(1) * cache_k.element_size()
        off = (view.data_ptr() - cache_k.data_ptr())
        assert off % row == 0
        return off // row, view.shape[1]

    def fake_monarch(q, k_cache, v_cache, new_k, new_v, start_idx, end_idx, *a, **kw):
        k_cache[:, start_idx:end_idx] = new_k
        v_cache[:, start_idx:end_idx] = new_v
        rec.update(branch=0, view=view_of(rec["cache_k"], k_cache), slot=(int(start_idx), int(end_idx)))
        return torch.zeros_like(q)

    def fake_attention(q, k, v, *a, **kw):
        rec.update(branch=1, view=view_of(rec["cache_k"], k), slot=None)
        return torch.zeros_like(q)

    cm.monarch_attn_with_kv_cache = fake_monarch
    cm.attention = fake_attention
    stride = cases.BOOKKEEPING_ID_STRIDE
    for name, sc in cases.BOOKKEEPING_SCENARIOS.items():
        for k in ("MONARCH_ATTN_FRAMEWISE", "USE_DENSE_INIT"):
            os.environ.pop(k, None)
        os.environ["MONARCH_ATTN_FRAMEWISE"] = "1"
        if sc.get("dense_init"):
            os.environ["USE_DENSE_INIT"] = "1"
        torch.manual_seed(7)
        mod = cm.CausalWanSelfAttention(256, 2, local_attn_size=sc["local_attn_size"], sink_size=sc["sink_size"])
        n_cache = sc["cache_frames"] * frame
        kv = {"k": torch.zeros(1, n_cache, 2, 128), "v": torch.zeros(1, n_cache, 2, 128),
              "global_end_index": torch.tensor([0], dtype=torch.long),
              "local_end_index": torch.tensor([0], dtype=torch.long)}
        kv["k"][0, :, 0, 0] = -(torch.arange(n_cache, dtype=torch.float32) + 1)      # "never written" ids
        grid = torch.tensor([[3, 30, 52]], dtype=torch.long)
        freqs = torch.polar(torch.ones(1024, 64, dtype=torch.float64), torch.zeros(1024, 64, dtype=torch.float64))
        rows = []
        ids_rows = []
        with torch.no_grad():
            for chunk, repeats in sc["calls"]:
                for _ in range(repeats):
                    current_start = chunk * 3 * frame
                    x = torch.randn(1, 3 * frame, 256)
                    before = (int(kv["global_end_index"]), int(kv["local_end_index"]))
                    rec.clear()
                    rec["cache_k"] = kv["k"]
                    mod(x, torch.tensor([3 * frame]), grid, freqs, None, kv_cache=kv, current_start=current_start)
                    col = kv["k"][0, :, 0, 0]
                    fresh = (col != col.round()).nonzero().flatten()      # rows holding projected keys = the slot
                    assert fresh.numel() == 3 * frame and int(fresh[-1] - fresh[0]) == 3 * frame - 1
                    col[fresh] = current_start + torch.arange(3 * frame, dtype=torch.float32) + 1
                    v0, vlen = rec["view"]
                    s0 = int(fresh[0]) - v0
                    if rec["slot"] is not None:
                        assert rec["slot"] == (s0, s0 + 3 * frame)
                    rows.append([current_start, before[0], before[1], rec["branch"], v0, vlen, s0, s0 + 3 * frame,
                                 int(kv["global_end_index"]), int(kv["local_end_index"])])
                    ids_rows.append(col[::stride].to(torch.int64).numpy().copy())
        out[f"book_{name}_calls"] = np.array(rows, dtype=np.int64)
        out[f"book_{name}_ids"] = np.stack(ids_rows).astype(np.int32)


def make_pins():
    ns, _, _ = load_reference()
    out = {}
    gradient_pins(ns, out)
    dense_pins(out)
    bookkeeping_pins(out)
    np.savez_compressed(HERE / "pins_golden.npz", **out)
    sz = (HERE / "pins_golden.npz").stat().st_size
    print(f"pins: wrote {len(out)} arrays, {sz/1e6:.2f} MB")


if __name__ == "__main__":
    torch.set_num_threads(os.cpu_count() or 1)
    if "--only-pins" not in sys.argv:
        main()
    make_pins()

"""Attention operators with the reference's call signatures, backed by libsfmonarch.so.

Every function here launches hand-written sm_100a kernels through the C ABI on the current
CUDA stream.  Inputs must be CUDA bf16 tensors with head_dim 128; anything else raises (there
is no eager / CPU fallback).  Scratch memory is a buffer per (GPU, stream) that grows on demand, is
reused by later calls queued on that stream and can be dropped with release_workspaces().
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import _lib

_workspaces: Dict[Tuple[int, int, str], torch.Tensor] = {}
_rope_tables: Dict[tuple, torch.Tensor] = {}
_status_mirror: Dict[int, list] = {}


# ------------------------------------------------------------------------------------- helpers
def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _require(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")
    if t.dim() != 4 or t.shape[-1] != 128:
        raise ValueError(f"{name} must be [B, N, H, 128], got {tuple(t.shape)}")


def _token_major(t: torch.Tensor) -> bool:
    """[B, N, H, D] with dense (N, H, D) strides; the batch stride is free."""
    _, n, h, d = t.shape
    return t.stride(3) == 1 and t.stride(2) == d and (n == 1 or t.stride(1) == h * d)


def _as_token_major(t: torch.Tensor) -> torch.Tensor:
    return t if _token_major(t) else t.contiguous()


def _batch_stride(t: torch.Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 else t.shape[1] * t.shape[2] * t.shape[3]


_MAX_WORKSPACES = 8


def _workspace(device: torch.device, nbytes: int, tag: str = "monarch") -> torch.Tensor:
    """Scratch for the row-step results, cached per (GPU, stream, kind): calls queued on one stream run in
    order and may share it, calls on different streams may overlap and must not.  A buffer only grows (up to
    the bridge budget, 1 GiB by default, plus the call's fixed part); at most _MAX_WORKSPACES buffers are kept,
    the least recently used one is dropped beyond that (a buffer was allocated on the stream that uses it, so
    PyTorch's allocator hands its memory out again in that stream's order only), and release_workspaces()
    drops them all."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), int(_stream().value or 0), tag)
    ws = _workspaces.pop(key, None)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
    _workspaces[key] = ws                          # re-inserted last: dict order is the LRU order
    while len(_workspaces) > _MAX_WORKSPACES:
        _workspaces.pop(next(iter(_workspaces)))       # freed in the order of the stream it was allocated on
    return ws


def release_workspaces() -> None:
    """Drops every cached scratch buffer (they come back on demand)."""
    _workspaces.clear()


_WATCH_EVERY = 32


def _watch_status(ws: torch.Tensor) -> None:
    """Keeps device-side failures loud without synchronising.  Every _WATCH_EVERY-th call on a GPU copies
    the workspace's status word to pinned host memory on the call's stream (a small device-to-host copy
    costs several microseconds of stream time, too much for every call); every call first looks at what
    the last such copy delivered.  A kernel that gave up on a bounded wait sets the word, every later
    launch on that workspace leaves a set word alone only until the next call clears it, so a persistent
    fault is reported within _WATCH_EVERY calls and a transient one may pass unseen: the synchronous
    check (SFM_CHECK_STATUS=1, or check_device_status()) is the strict form."""
    key = ws.device.index if ws.device.index is not None else torch.cuda.current_device()
    state = _status_mirror.get(key)
    if state is None:
        state = [torch.zeros(1, dtype=torch.int32).pin_memory(), 0]
        _status_mirror[key] = state
    host = state[0]
    code = int(host[0])
    if code != 0:
        host[0] = 0
        raise RuntimeError(f"an earlier Monarch attention call on this GPU recorded device status {code} "
                           "(a kernel gave up on a bounded wait); its output is not valid")
    state[1] += 1
    if state[1] % _WATCH_EVERY == 0:
        host.copy_(ws[:4].view(torch.int32), non_blocking=True)


def check_device_status(device=None) -> None:
    """Synchronous form: waits for the work queued on the current stream and raises if the last Monarch
    attention call queued on it (on ``device``) left a non-zero status word."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    lib = _lib.load()
    with torch.cuda.device(dev):
        for kind in ("monarch", "monarch_bwd"):      # the workspaces of the current stream
            ws = _workspaces.get((index, int(_stream().value or 0), kind))
            if ws is not None:
                _lib.check(lib.sfm_workspace_status(_ptr(ws), _stream()), f"sfm_workspace_status ({kind})")
        _lib.check(lib.sfm_dense_status(_stream()), "sfm_dense_status")


def _rope_table_from_freqs(freqs: Optional[torch.Tensor], device: torch.device) -> torch.Tensor:
    """Device table [1024, 64, 2] fp32 = (cos, sin).  Built from the model's complex128
    ``freqs`` buffer when given (causal_model.py:1352-1357), else by the library."""
    if freqs is None:
        key = ("lib", device)
        tab = _rope_tables.get(key)
        if tab is None:
            host = np.empty((1024, 64, 2), dtype=np.float32)
            _lib.check(_lib.load().sfm_rope_table(host.ctypes.data_as(C.c_void_p), 128, 1024, 10000.0),
                       "sfm_rope_table")
            tab = torch.from_numpy(host).to(device)
            _rope_tables[key] = tab
        return tab
    key = (freqs.data_ptr(), tuple(freqs.shape), device)
    tab = _rope_tables.get(key)
    if tab is None:
        if freqs.dim() != 2 or freqs.shape[1] != 64 or freqs.shape[0] < 1024 or not freqs.is_complex():
            raise ValueError("freqs must be a complex [>=1024, 64] table")
        tab = torch.view_as_real(freqs[:1024].to(torch.complex128)).to(torch.float32).contiguous().to(device)
        _rope_tables[key] = tab
    return tab


def _mark_written(*tensors) -> None:
    """The kernels write the caches through raw pointers, which autograd cannot see.  Bumping the version
    counters makes a later backward that saved one of these tensors fail loudly, as it does after the
    reference's slice assignment (monarch_attn.py:1230-1231), instead of using overwritten keys."""
    for t in tensors:
        if not t.is_inference():                   # inference tensors carry no version counter
            torch.autograd.graph.increment_version(t)


def workspace_bytes(B, H, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, num_iters=1, bridge_budget_bytes=0) -> int:
    return int(_lib.load().sfm_monarch_workspace_bytes(B, H, 128, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w,
                                                       num_iters, bridge_budget_bytes))


def build_maps(n_tokens, f_tied, h_reduce, w_reduce, h, w):
    """(nat2mon, mon2nat) int32 arrays: the token permutation of
    _get_rearrange_fns (monarch_attn.py:1696-1703)."""
    a = np.empty(n_tokens, dtype=np.int32)
    b = np.empty(n_tokens, dtype=np.int32)
    _lib.check(_lib.load().sfm_build_maps(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), n_tokens,
                                          f_tied, h_reduce, w_reduce, h, w), "sfm_build_maps")
    return a, b


def _cache_view_ok(c: torch.Tensor, name: str) -> None:
    _require(c, name)
    if not _token_major(c):
        raise ValueError(f"{name} must keep dense (token, head, dim) strides: it is written in place")


def _monarch_fwd(q, k_cache, v_cache, f_tied, h_reduce, w_reduce, h, w, sm_scale, num_iters):
    B, n_q, H, D = q.shape
    n_kv = k_cache.shape[1]
    lib = _lib.load()
    nbytes = lib.sfm_monarch_workspace_bytes(B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, num_iters, 0)
    if nbytes == 0:
        # let the entry point produce the precise error
        nbytes = 256
    ws = _workspace(q.device, nbytes)
    out = torch.empty((B, n_q, H, D), dtype=q.dtype, device=q.device)
    rc = lib.sfm_monarch_fwd(_ptr(q), _batch_stride(q), _ptr(k_cache), _ptr(v_cache), _batch_stride(k_cache),
                             _ptr(out), _ptr(ws), ws.numel(), B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w,
                             float(sm_scale), int(num_iters), 0, _stream())
    _lib.check(rc, "sfm_monarch_fwd")
    if os.environ.get("SFM_CHECK_STATUS") == "1":      # debugging aid: synchronises the stream
        _lib.check(lib.sfm_workspace_status(_ptr(ws), _stream()), "sfm_workspace_status")
    else:
        _watch_status(ws)
    return out


def monarch_attn_with_kv_cache_backward(q, k_cache, v_cache, grad_out, f_tied, h_reduce, w_reduce, h, w, sm_scale=None,
                                        kv_groups: Optional[Tuple[int, int]] = None, budget_bytes: int = 0,
                                        causal_groups: int = 0):
    """Gradients of ``monarch_attn_with_kv_cache`` (single pass) for a gradient ``grad_out`` of its output.

    q, grad_out: [B, n_q, H, 128] bf16, natural token order; k_cache / v_cache: the cache view the forward
    call attended, [B, n_kv, H, 128] bf16 in Monarch order.  ``kv_groups`` = (begin, end) limits dK / dV to
    those cached groups (one group = b1 * b2 tokens, a frame for the framewise blocking); None = all.
    Returns (dq fp32 [B, n_q, H, 128] natural order, dk, dv bf16 [B, groups * b1 * b2, H, 128] Monarch
    order).  The call runs in slices of (batch, head) pairs whose fp32 scratch stays under ``budget_bytes``
    (0 = 2 GiB).  ``causal_groups`` > 0 applies the block-causal mask of ``monarch_attn`` (query group a sees
    the groups below (a // causal_groups + 1) * causal_groups).  Stands in for _attention_with_cache.backward (monarch_attn.py:1325-1470)."""
    for t, name in ((q, "q"), (grad_out, "grad_out")):
        _require(t, name)
    _cache_view_ok(k_cache, "k_cache")
    _cache_view_ok(v_cache, "v_cache")
    if k_cache.stride() != v_cache.stride() or k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must share shape and strides")
    if grad_out.shape != q.shape:
        raise ValueError("grad_out must have q's shape")
    B, n_q, H, D = q.shape
    n_kv = k_cache.shape[1]
    if sm_scale is None:
        sm_scale = D ** -0.5
    q = _as_token_major(q)
    grad_out = grad_out.contiguous()
    lib = _lib.load()
    nbytes = lib.sfm_monarch_bwd_workspace_bytes(B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, budget_bytes)
    ws = _workspace(q.device, max(int(nbytes), 256), "monarch_bwd")
    group = (f_tied * h * w) // (h_reduce * w_reduce)
    g0, g1 = (0, n_kv // group) if kv_groups is None else (int(kv_groups[0]), int(kv_groups[1]))
    dq = torch.empty((B, n_q, H, D), dtype=torch.float32, device=q.device)
    dk = torch.empty((B, max(g1 - g0, 0) * group, H, D), dtype=q.dtype, device=q.device)
    dv = torch.empty_like(dk)
    rc = lib.sfm_monarch_bwd(_ptr(q), _batch_stride(q), _ptr(k_cache), _ptr(v_cache), _batch_stride(k_cache),
                             _ptr(grad_out), _ptr(dq), _ptr(dk) if dk.numel() else None,
                             _ptr(dv) if dv.numel() else None, _ptr(ws), ws.numel(), B, H, D, n_q, n_kv, f_tied,
                             h_reduce, w_reduce, h, w, float(sm_scale), g0, g1, int(causal_groups), budget_bytes,
                             _stream())
    _lib.check(rc, "sfm_monarch_bwd")
    if os.environ.get("SFM_CHECK_STATUS") == "1":      # debugging aid: synchronises the stream
        _lib.check(lib.sfm_workspace_status(_ptr(ws), _stream()), "sfm_workspace_status")
    else:
        _watch_status(ws)
    return dq, dk, dv


class _MonarchWithKVCacheFn(torch.autograd.Function):
    """Cache write + Monarch attention with the backward kernels behind it.  Differentiable inputs: q,
    new_k, new_v (natural order) and, unless grad_only_new_kv, the cache tensors."""

    @staticmethod
    def forward(ctx, q, new_k, new_v, k_cache, v_cache, start_idx, end_idx, blocking, sm_scale, grad_only_new_kv):
        f_tied, h_reduce, w_reduce, h, w = blocking
        out = monarch_attn_with_kv_cache(q.detach(), k_cache.detach(), v_cache.detach(), new_k.detach(), new_v.detach(),
                                         start_idx, end_idx, f_tied, h_reduce, w_reduce, h, w, sm_scale, 1,
                                         _no_grad=True)
        ctx.save_for_backward(q, k_cache, v_cache)
        ctx.args = (int(start_idx), int(end_idx), blocking, sm_scale, bool(grad_only_new_kv))
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k_cache, v_cache = ctx.saved_tensors
        start, end, blocking, sm_scale, only_new = ctx.args
        f_tied, h_reduce, w_reduce, h, w = blocking
        group = (f_tied * h * w) // (h_reduce * w_reduce)
        n_kv = k_cache.shape[1]
        want_cache = not only_new and (ctx.needs_input_grad[3] or ctx.needs_input_grad[4])
        g0, g1 = (0, n_kv // group) if want_cache else (start // group, -(-end // group))
        dq, dk, dv = monarch_attn_with_kv_cache_backward(q, k_cache, v_cache, grad_out.to(q.dtype), f_tied, h_reduce,
                                                         w_reduce, h, w, sm_scale, (g0, g1))
        lo = start - g0 * group
        nat2mon, _ = build_maps(end - start, f_tied, h_reduce, w_reduce, h, w)
        idx = torch.from_numpy(nat2mon.astype(np.int64)).to(q.device)
        d_new_k = dk[:, lo:lo + end - start].index_select(1, idx)
        d_new_v = dv[:, lo:lo + end - start].index_select(1, idx)
        # The reference hands back the gradient with respect to the cache CONTENT after its in-place write,
        # written slot included (monarch_attn.py:1462-1470; its PyTorch restatement retains the gradient of
        # the cache after the write, :1869-1872), so the same is returned here.
        d_kc, d_vc = (dk, dv) if want_cache else (None, None)
        return dq, d_new_k, d_new_v, d_kc, d_vc, None, None, None, None, None


class _MonarchNoCacheFn(torch.autograd.Function):
    """monarch_attn (no cache, optionally block-causal) with the backward kernels behind it."""

    @staticmethod
    def forward(ctx, q, k, v, blocking, sm_scale, block_causal_size):
        out, k_mon, v_mon, causal_groups = _monarch_attn_fwd(q.detach(), k.detach(), v.detach(), *blocking, sm_scale,
                                                             block_causal_size, 1)
        ctx.save_for_backward(q, k_mon, v_mon)
        ctx.args = (blocking, sm_scale, causal_groups)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k_mon, v_mon = ctx.saved_tensors
        blocking, sm_scale, causal_groups = ctx.args
        dq, dk, dv = monarch_attn_with_kv_cache_backward(q, k_mon, v_mon, grad_out.to(q.dtype), *blocking, sm_scale,
                                                         causal_groups=causal_groups)
        nat2mon, _ = build_maps(k_mon.shape[1], *blocking)
        idx = torch.from_numpy(nat2mon.astype(np.int64)).to(q.device)
        return dq, dk.index_select(1, idx), dv.index_select(1, idx), None, None, None


# ------------------------------------------------------------------------------------- public
def monarch_attn_with_kv_cache(q, k_cache, v_cache, new_k, new_v, start_idx, end_idx, f_tied, h_reduce, w_reduce,
                               h, w, sm_scale=None, num_iters=1, grad_only_new_kv=False, _no_grad=False):
    """Same contract as the reference's monarch_attn_with_kv_cache (monarch_attn.py:1778-1796):
    new_k / new_v are written, in Monarch block order, into k_cache / v_cache[:, start_idx:end_idx]
    IN PLACE, then q attends the whole cache view.  q, new_k, new_v: [B, n, H, 128] bf16 (already
    rotated); caches [B, n_kv, H, 128] bf16, possibly a [:, :n_kv] view of a longer buffer.  Returns
    [B, n_q, H, 128].  When autograd is recording and an input requires a gradient the call goes
    through an autograd function whose backward runs the backward kernels (single pass only);
    grad_only_new_kv then limits dK / dV to the slots this call wrote.  As in the reference, the cache
    gradient is the one with respect to the cache content after the write (the written slot carries the new
    keys' gradient in Monarch order), and writing the cache again before backward is an error."""
    if (not _no_grad and torch.is_grad_enabled()
            and any(t.requires_grad for t in (q, new_k, new_v, k_cache, v_cache))):
        if num_iters != 1:
            raise NotImplementedError("the backward pass exists for num_iters == 1 only")
        return _MonarchWithKVCacheFn.apply(q, new_k, new_v, k_cache, v_cache, start_idx, end_idx,
                                           (f_tied, h_reduce, w_reduce, h, w), sm_scale, grad_only_new_kv)
    for t, name in ((q, "q"), (new_k, "new_k"), (new_v, "new_v")):
        _require(t, name)
    _cache_view_ok(k_cache, "k_cache")
    _cache_view_ok(v_cache, "v_cache")
    if k_cache.stride() != v_cache.stride() or k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must share shape and strides")
    B, n_q, H, D = q.shape
    n_new = new_k.shape[1]
    if end_idx - start_idx != n_new or new_v.shape != new_k.shape or end_idx > k_cache.shape[1] or start_idx < 0:
        raise ValueError("start_idx/end_idx do not match new_k / the cache extent")
    if sm_scale is None:
        sm_scale = D ** -0.5
    q = _as_token_major(q)
    new_k = new_k.contiguous()
    new_v = new_v.contiguous()
    rc = _lib.load().sfm_rope_cache_write(_ptr(None), _ptr(new_k), _ptr(new_v), _ptr(None), _ptr(k_cache),
                                          _ptr(v_cache), _batch_stride(k_cache), _ptr(None), B, n_new, H, D,
                                          int(start_idx), f_tied, h_reduce, w_reduce, h, w, 0, 1, _stream())
    _lib.check(rc, "sfm_rope_cache_write")
    _mark_written(k_cache, v_cache)
    return _monarch_fwd(q, k_cache, v_cache, f_tied, h_reduce, w_reduce, h, w, sm_scale, num_iters)


def norm_rope_cache_write(q, k, v, k_cache, v_cache, start_idx, start_frame, f_tied, h_reduce, w_reduce, h, w,
                          freqs=None, norm_q_weight=None, norm_k_weight=None, eps=1e-6, monarch_order=True, roll=None):
    """One kernel: optional full-width RMSNorm of q and k (WanRMSNorm, model.py:462-478, as applied in
    qkv_fn, causal_model.py:801-807), 3-axis RoPE with frame offset (causal_model.py:687-715), and the
    in-place write of k, v into cache tokens [start_idx, start_idx + n) in Monarch order (or natural
    order for the dense branch).  ``roll`` = (dst, shift) folds the sliding window's eviction into the same
    launch: the cached tokens [dst + shift, start_idx + shift) first move left by ``shift``
    (causal_model.py:912-926).  Returns the normalised, rotated q."""
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _require(t, name)
    _cache_view_ok(k_cache, "k_cache")
    _cache_view_ok(v_cache, "v_cache")
    B, n, H, D = q.shape
    if k.shape != q.shape or v.shape != q.shape or start_idx + n > k_cache.shape[1]:
        raise ValueError("q, k, v shapes or the cache extent do not match")
    tab = _rope_table_from_freqs(freqs, q.device)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    q_rot = torch.empty_like(q)
    lib = _lib.load()
    if (norm_q_weight is None) != (norm_k_weight is None):
        raise ValueError("give both norm weights or neither")
    wq = wk = None
    if norm_q_weight is not None:
        wq = norm_q_weight.detach().to(device=q.device, dtype=torch.bfloat16).contiguous()
        wk = norm_k_weight.detach().to(device=q.device, dtype=torch.bfloat16).contiguous()
        if wq.numel() != H * D or wk.numel() != H * D:
            raise ValueError("norm weights must have H*D elements")
    if roll is not None:
        dst, shift = int(roll[0]), int(roll[1])
        if start_idx + shift > k_cache.shape[1]:
            raise ValueError("the eviction shift reads past the cache view")
        rc = lib.sfm_rope_cache_write_roll(_ptr(q), _ptr(k), _ptr(v), _ptr(wq), _ptr(wk), float(eps), _ptr(q_rot),
                                           _ptr(k_cache), _ptr(v_cache), _batch_stride(k_cache), _ptr(tab), B, n, H, D,
                                           int(start_idx), dst, shift, f_tied, h_reduce, w_reduce, h, w,
                                           int(start_frame), 1 if monarch_order else 0, _stream())
        _lib.check(rc, "sfm_rope_cache_write_roll")
    elif norm_q_weight is not None:
        rc = lib.sfm_norm_rope_cache_write(_ptr(q), _ptr(k), _ptr(v), _ptr(wq), _ptr(wk), float(eps), _ptr(q_rot),
                                           _ptr(k_cache), _ptr(v_cache), _batch_stride(k_cache), _ptr(tab), B, n, H, D,
                                           int(start_idx), f_tied, h_reduce, w_reduce, h, w, int(start_frame),
                                           1 if monarch_order else 0, _stream())
        _lib.check(rc, "sfm_norm_rope_cache_write")
    else:
        rc = lib.sfm_rope_cache_write(_ptr(q), _ptr(k), _ptr(v), _ptr(q_rot), _ptr(k_cache), _ptr(v_cache),
                                      _batch_stride(k_cache), _ptr(tab), B, n, H, D, int(start_idx), f_tied, h_reduce,
                                      w_reduce, h, w, int(start_frame), 1 if monarch_order else 0, _stream())
        _lib.check(rc, "sfm_rope_cache_write")
    _mark_written(k_cache, v_cache)
    return q_rot


def rope_monarch_attn_with_kv_cache(q, k, v, k_cache, v_cache, start_idx, end_idx, start_frame, f_tied, h_reduce,
                                    w_reduce, h, w, freqs=None, sm_scale=None, num_iters=1):
    """Fused front end: q, k are the UN-rotated projections.  One kernel applies the 3-axis RoPE
    (frame positions start at start_frame), keeps rotated q, and writes rotated k and v into the
    cache slot in Monarch order; then the Monarch forward runs.  Equivalent to
    causal_rope_apply(q), causal_rope_apply(k) followed by monarch_attn_with_kv_cache
    (causal_model.py:902-905, 1085-1100)."""
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _require(t, name)
    _cache_view_ok(k_cache, "k_cache")
    _cache_view_ok(v_cache, "v_cache")
    B, n_q, H, D = q.shape
    if end_idx - start_idx != n_q or k.shape != q.shape or v.shape != q.shape or end_idx > k_cache.shape[1]:
        raise ValueError("start_idx/end_idx do not match the chunk / the cache extent")
    if sm_scale is None:
        sm_scale = D ** -0.5
    tab = _rope_table_from_freqs(freqs, q.device)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    q_rot = torch.empty_like(q)
    rc = _lib.load().sfm_rope_cache_write(_ptr(q), _ptr(k), _ptr(v), _ptr(q_rot), _ptr(k_cache), _ptr(v_cache),
                                          _batch_stride(k_cache), _ptr(tab), B, n_q, H, D, int(start_idx), f_tied,
                                          h_reduce, w_reduce, h, w, int(start_frame), 1, _stream())
    _lib.check(rc, "sfm_rope_cache_write")
    _mark_written(k_cache, v_cache)
    return _monarch_fwd(q_rot, k_cache, v_cache, f_tied, h_reduce, w_reduce, h, w, sm_scale, num_iters)


def _ptr_array(ptrs):
    arr = (C.c_void_p * len(ptrs))(*[C.c_void_p(int(p)) for p in ptrs])
    return arr


def norm_rope_token_slice(q, k, v, q_out, k_out, v_out, token0, start_frame, h, w, freqs=None, norm_q_weight=None,
                          norm_k_weight=None, eps=1e-6):
    """RMSNorm (optional) + RoPE of a token slice of a chunk whose first token is ``token0`` of the chunk's grid:
    q_out, k_out <- rotated (normalised) q, k; v_out <- v; all [B, n, H, 128] natural order.  One kernel; the
    outputs may be symmetric-memory buffers that the peers' gather kernels read."""
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (q_out, "q_out"), (k_out, "k_out"), (v_out, "v_out")):
        _require(t, name)
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    B, n, H, D = q.shape
    if any(t.shape != q.shape for t in (k, v, q_out, k_out, v_out)):
        raise ValueError("all six tensors must share one shape")
    if (norm_q_weight is None) != (norm_k_weight is None):
        raise ValueError("give both norm weights or neither")
    wq = wk = None
    if norm_q_weight is not None:
        wq = norm_q_weight.detach().to(device=q.device, dtype=torch.bfloat16).contiguous()
        wk = norm_k_weight.detach().to(device=q.device, dtype=torch.bfloat16).contiguous()
    tab = _rope_table_from_freqs(freqs, q.device)
    rc = _lib.load().sfm_norm_rope_token_slice(_ptr(q), _ptr(k), _ptr(v), _ptr(wq), _ptr(wk), float(eps), _ptr(q_out),
                                               _ptr(k_out), _ptr(v_out), _ptr(tab), B, n, H, D, int(token0), int(h),
                                               int(w), int(start_frame), _stream())
    _lib.check(rc, "sfm_norm_rope_token_slice")


def rope_monarch_attn_with_kv_cache_sharded(q_shards, k_shards, v_shards, out_shards, rank, shard_shape, k_cache,
                                            v_cache, start_idx, end_idx, start_frame, f_tied, h_reduce, w_reduce,
                                            h, w, freqs=None, sm_scale=None, rotate=True):
    """Head-sharded form of rope_monarch_attn_with_kv_cache for P GPUs of one box.

    ``q_shards[p]``, ``k_shards[p]``, ``v_shards[p]``, ``out_shards[p]`` are device addresses (ints),
    valid on THIS GPU, of GPU p's token shard ``shard_shape = (B, n/P, H_total, 128)`` (bf16,
    contiguous); ``k_cache`` / ``v_cache`` hold this rank's ``H_total/P`` heads.  The gather of the
    inputs and the scatter of the result are done by the kernels over peer memory; the caller
    puts a barrier before (shards complete) and after (rows landed) the call.  ``rotate=False``: the shards
    hold q, k that are rotated already (norm_rope_token_slice).  Returns nothing: the result is in the out shards."""
    world = len(q_shards)
    B, sp, h_total, D = shard_shape
    if h_total % world:
        raise ValueError("heads must divide evenly over the ranks")
    H = h_total // world
    n_q = sp * world
    _cache_view_ok(k_cache, "k_cache")
    _cache_view_ok(v_cache, "v_cache")
    if end_idx - start_idx != n_q or end_idx > k_cache.shape[1] or k_cache.shape[2] != H:
        raise ValueError("start_idx/end_idx or the cache's head count do not match the shards")
    if sm_scale is None:
        sm_scale = D ** -0.5
    lib = _lib.load()
    tab = _rope_table_from_freqs(freqs, k_cache.device) if rotate else None     # shards already rotated: gather only
    q_rot = torch.empty((B, n_q, H, D), dtype=torch.bfloat16, device=k_cache.device)
    rc = lib.sfm_rope_cache_write_gather(_ptr_array(q_shards), _ptr_array(k_shards), _ptr_array(v_shards), world,
                                         int(rank), _ptr(q_rot), _ptr(k_cache), _ptr(v_cache), _batch_stride(k_cache),
                                         _ptr(tab), B, n_q, H, D, int(start_idx), f_tied, h_reduce, w_reduce, h, w,
                                         int(start_frame), 1, _stream())
    _lib.check(rc, "sfm_rope_cache_write_gather")
    _mark_written(k_cache, v_cache)
    n_kv = end_idx
    kc, vc = k_cache[:, :n_kv], v_cache[:, :n_kv]
    nbytes = lib.sfm_monarch_workspace_bytes(B, H, D, n_q, n_kv, f_tied, h_reduce, w_reduce, h, w, 1, 0) or 256
    ws = _workspace(k_cache.device, nbytes)
    rc = lib.sfm_monarch_fwd_scatter(_ptr(q_rot), _batch_stride(q_rot), _ptr(kc), _ptr(vc), _batch_stride(kc),
                                     _ptr_array(out_shards), world, int(rank), _ptr(ws), ws.numel(), B, H, D, n_q,
                                     n_kv, f_tied, h_reduce, w_reduce, h, w, float(sm_scale), 0, _stream())
    _lib.check(rc, "sfm_monarch_fwd_scatter")
    if os.environ.get("SFM_CHECK_STATUS") == "1":
        _lib.check(lib.sfm_workspace_status(_ptr(ws), _stream()), "sfm_workspace_status")


def monarch_attn(q, k, v, f_tied, h_reduce, w_reduce, h, w, sm_scale=None, block_causal_size=None, num_iters=1):
    """Same contract as the reference's monarch_attn (monarch_attn.py:1753-1776): no cache;
    with block_causal_size, causal over blocks of that many tokens.  Under autograd (an input requires a
    gradient) the single-pass variant goes through an autograd function backed by the backward kernels."""
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v)):
        if num_iters != 1:
            raise NotImplementedError("the backward pass exists for num_iters == 1 only")
        return _MonarchNoCacheFn.apply(q, k, v, (f_tied, h_reduce, w_reduce, h, w), sm_scale, block_causal_size)
    return _monarch_attn_fwd(q, k, v, f_tied, h_reduce, w_reduce, h, w, sm_scale, block_causal_size, num_iters)[0]


def _monarch_attn_fwd(q, k, v, f_tied, h_reduce, w_reduce, h, w, sm_scale, block_causal_size, num_iters):
    """Forward of monarch_attn; returns (out, k_mon, v_mon, causal_groups): the keys / values in Monarch block
    order are what the backward kernels read."""
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _require(t, name)
    B, N, H, D = q.shape
    if k.shape != q.shape and block_causal_size is not None:
        raise ValueError("block-causal Monarch needs kv length equal to q length")
    if sm_scale is None:
        sm_scale = D ** -0.5
    lib = _lib.load()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    n_kv = k.shape[1]
    causal_groups = 0
    if block_causal_size is not None:
        b1 = f_tied * (h // h_reduce)
        b2 = w // w_reduce
        if N % block_causal_size or block_causal_size % (b1 * b2):
            raise ValueError("block_causal_size must divide the sequence and align with Monarch blocks")
        if num_iters != 1:
            raise ValueError("causal currently only supported for num_iters=1")
        causal_groups = block_causal_size // (b1 * b2)
    if n_kv != N:
        k_mon = torch.empty_like(k)
        v_mon = torch.empty_like(v)
        rc = lib.sfm_rope_cache_write(_ptr(None), _ptr(k), _ptr(v), _ptr(None), _ptr(k_mon), _ptr(v_mon),
                                      n_kv * H * D, _ptr(None), B, n_kv, H, D, 0, f_tied, h_reduce, w_reduce, h, w,
                                      0, 1, _stream())
        _lib.check(rc, "sfm_rope_cache_write")
        return _monarch_fwd(q, k_mon, v_mon, f_tied, h_reduce, w_reduce, h, w, sm_scale, num_iters), k_mon, v_mon, 0
    nbytes = lib.sfm_monarch_workspace_bytes(B, H, D, N, N, f_tied, h_reduce, w_reduce, h, w, num_iters, 0) or 256
    ws = _workspace(q.device, nbytes)
    out = torch.empty_like(q)
    k_mon = torch.empty_like(k)
    v_mon = torch.empty_like(v)
    rc = lib.sfm_monarch_nocache_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(k_mon), _ptr(v_mon), _ptr(out), _ptr(ws),
                                     ws.numel(), B, H, D, N, f_tied, h_reduce, w_reduce, h, w, float(sm_scale),
                                     causal_groups, int(num_iters), 0, _stream())
    _lib.check(rc, "sfm_monarch_nocache_fwd")
    return out, k_mon, v_mon, causal_groups


def flash_attention(q, k, v, q_lens=None, k_lens=None, dropout_p=0., softmax_scale=None, q_scale=None,
                    causal=False, window_size=(-1, -1), deterministic=False, dtype=torch.bfloat16, version=None):
    """Dense softmax attention with the reference's flash_attention signature
    (wan/modules/attention.py:34-138).  Only what the causal rollout uses is supported: full
    lengths, no dropout, no mask, no window."""
    del deterministic, version
    if q_lens is not None or k_lens is not None:
        raise NotImplementedError("variable lengths are not used by the KV-cache rollout")
    if causal or dropout_p != 0. or tuple(window_size) != (-1, -1):
        raise NotImplementedError("only unmasked, dropout-free dense attention is implemented")
    out_dtype = q.dtype
    if q.dtype != torch.bfloat16:
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _require(t, name)
    if q_scale is not None:
        q = q * q_scale
    B, n_q, H, D = q.shape
    if softmax_scale is None:
        softmax_scale = D ** -0.5
    q = _as_token_major(q)
    k = _as_token_major(k)
    v = _as_token_major(v)
    if _batch_stride(k) != _batch_stride(v):
        v = v.contiguous()
        k = k.contiguous()
    out = torch.empty((B, n_q, H, D), dtype=torch.bfloat16, device=q.device)
    rc = _lib.load().sfm_dense_fwd(_ptr(q), _batch_stride(q), _ptr(k), _ptr(v), _batch_stride(k), _ptr(out), B, H, D,
                                   n_q, k.shape[1], float(softmax_scale), _stream())
    _lib.check(rc, "sfm_dense_fwd")
    if os.environ.get("SFM_CHECK_STATUS") == "1":      # debugging aid: synchronises the stream
        _lib.check(_lib.load().sfm_dense_status(_stream()), "sfm_dense_status")
    return out.type(out_dtype)


def attention(q, k, v, q_lens=None, k_lens=None, dropout_p=0., softmax_scale=None, q_scale=None, causal=False,
              window_size=(-1, -1), deterministic=False, dtype=torch.bfloat16, fa_version=None):
    """Same signature as the reference's attention (wan/modules/attention.py:141-187)."""
    return flash_attention(q=q, k=k, v=v, q_lens=q_lens, k_lens=k_lens, dropout_p=dropout_p,
                           softmax_scale=softmax_scale, q_scale=q_scale, causal=causal, window_size=window_size,
                           deterministic=deterministic, dtype=dtype, version=fa_version)


def full_attention_with_kv_cache(q, k_cache, v_cache, new_k, new_v, start_idx, end_idx, sm_scale=None,
                                 grad_only_new_kv=False):
    """Dense attention after an in-place, natural-order cache write
    (wan/modules/attn_patch.py:416; the dense branch of causal_model.py:961-967)."""
    del grad_only_new_kv
    for t, name in ((q, "q"), (new_k, "new_k"), (new_v, "new_v")):
        _require(t, name)
    _cache_view_ok(k_cache, "k_cache")
    _cache_view_ok(v_cache, "v_cache")
    B, n_q, H, D = q.shape
    n_new = new_k.shape[1]
    if end_idx - start_idx != n_new or end_idx > k_cache.shape[1]:
        raise ValueError("start_idx/end_idx do not match new_k / the cache extent")
    new_k, new_v = new_k.contiguous(), new_v.contiguous()
    rc = _lib.load().sfm_rope_cache_write(_ptr(None), _ptr(new_k), _ptr(new_v), _ptr(None), _ptr(k_cache),
                                          _ptr(v_cache), _batch_stride(k_cache), _ptr(None), B, n_new, H, D,
                                          int(start_idx), 1, 1, 1, 1, 1, 0, 0, _stream())
    _lib.check(rc, "sfm_rope_cache_write")
    _mark_written(k_cache, v_cache)
    return attention(q, k_cache, v_cache, softmax_scale=sm_scale)


def dense_attention_on_cache(q, k_view, v_view, sm_scale=None):
    """Dense attention of already rotated q against a cache view that already holds the new tokens."""
    _cache_view_ok(k_view, "k_cache")
    _cache_view_ok(v_view, "v_cache")
    return attention(q, k_view, v_view, softmax_scale=sm_scale)


def monarch_attention_on_cache(q, k_view, v_view, f_tied, h_reduce, w_reduce, h, w, sm_scale=None, num_iters=1):
    """Monarch attention of already rotated q against a cache view (Monarch order) that already holds
    the new tokens: the part of monarch_attn_with_kv_cache after its cache write."""
    _require(q, "q")
    _cache_view_ok(k_view, "k_cache")
    _cache_view_ok(v_view, "v_cache")
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    return _monarch_fwd(_as_token_major(q), k_view, v_view, f_tied, h_reduce, w_reduce, h, w, sm_scale, num_iters)


def causal_rope_apply(x, grid_sizes, freqs, start_frame=0):
    """Same contract as the reference's causal_rope_apply (causal_model.py:687-715) for a batch
    whose samples share one (frames, rows, cols) grid: rotate the first frames*rows*cols tokens,
    pass the rest through; result in x's dtype."""
    _require(x, "x")
    if isinstance(grid_sizes, torch.Tensor):
        grid_sizes = grid_sizes.tolist()
    grids = {tuple(int(v) for v in g) for g in grid_sizes}
    if len(grids) != 1:
        raise NotImplementedError("all samples must share one token grid")
    f, h, w = next(iter(grids))
    B, L, H, D = x.shape
    tab = _rope_table_from_freqs(freqs, x.device)
    x = x.contiguous()
    out = torch.empty_like(x)
    rc = _lib.load().sfm_rope_apply(_ptr(x), _ptr(out), _ptr(tab), B, L, H, D, f, h, w, int(start_frame), _stream())
    _lib.check(rc, "sfm_rope_apply")
    return out

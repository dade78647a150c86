"""CPU oracle for the Monarch self-attention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch/NumPy on the CPU, the arithmetic of the
reference's pure-PyTorch Monarch attention path.  It exists to check the CUDA
kernels; nothing in the product package imports it.  Only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may call it.

Parity status: PINNED.  The reference stores no golden vectors, so the pins are
outputs of the reference's own functions (extracted from its source and run in
fp32 on the CPU) committed as fixtures under ``tests/golden/`` together with the
script that produced them; ``tests/test_oracle_golden.py`` checks this file
against every one of them.

Reference functions followed (paths inside the reference project):

* token <-> (group, row, column) maps ....... wan/modules/monarch_attn.py:1696-1703
* one-iteration Monarch attention ........... wan/modules/monarch_attn.py:1801-1830
* multi-iteration ("slow") Monarch .......... wan/modules/monarch_attn.py:1705-1751
* KV-cache entry point and its side effect .. wan/modules/monarch_attn.py:1778-1796
* no-cache entry point (block causal) ....... wan/modules/monarch_attn.py:1753-1776, 1832-1858
* 3-axis rotary embedding ................... wan/modules/causal_model.py:687-715,
                                              wan/modules/model.py:421-428,
                                              wan/modules/causal_model.py:1352-1357
* KV-cache index bookkeeping ................ wan/modules/causal_model.py:900-938
* dense attention (SDPA fallback semantics) . wan/modules/attention.py:177-187
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

__all__ = [
    "block_dims", "token_maps", "to_monarch_order", "from_monarch_order",
    "rope_table", "rope_apply", "monarch_core", "monarch_attn_with_kv_cache",
    "monarch_attn", "dense_attention", "cache_indices",
]


# --------------------------------------------------------------------------- #
# integer layout maps  (wan/modules/monarch_attn.py:1696-1703)
# --------------------------------------------------------------------------- #
def block_dims(n_tokens: int, f_tied: int, h_reduce: int, w_reduce: int, h: int, w: int):
    """Return (groups, b1, b2) for ``n_tokens`` tokens of an h x w token grid."""
    if h % h_reduce or w % w_reduce:
        raise ValueError("h_reduce / w_reduce must divide the token grid")
    per_group_frames = f_tied * h * w
    if n_tokens % per_group_frames:
        raise ValueError("token count is not a whole number of tied frame groups")
    b1 = f_tied * (h // h_reduce)
    b2 = w // w_reduce
    groups = (n_tokens // per_group_frames) * h_reduce * w_reduce
    return groups, b1, b2


def token_maps(n_tokens: int, f_tied: int, h_reduce: int, w_reduce: int, h: int, w: int
               ) -> Tuple[np.ndarray, np.ndarray]:
    """Integer permutation between natural token order and Monarch block order.

    natural index   n = (((((a*f_tied+f)*h_reduce+c)*hh+i)*w_reduce+e)*ww+j)
    Monarch index   m = ((((a*h_reduce+c)*w_reduce+e)*f_tied+f)*hh+i)*ww+j
    with hh = h/h_reduce and ww = w/w_reduce, i.e. group = (a,c,e), row = (f,i),
    column = j.  Returns ``(nat2mon, mon2nat)`` as int64 arrays: the token at
    natural position n sits at Monarch position nat2mon[n]; mon2nat is the inverse.
    """
    block_dims(n_tokens, f_tied, h_reduce, w_reduce, h, w)
    hh, ww = h // h_reduce, w // w_reduce
    n_a = n_tokens // (f_tied * h * w)
    nat = np.arange(n_tokens, dtype=np.int64).reshape(n_a, f_tied, h_reduce, hh, w_reduce, ww)
    # axes: a f c i e j  ->  a c e f i j
    mon2nat = np.ascontiguousarray(nat.transpose(0, 2, 4, 1, 3, 5)).reshape(-1)
    nat2mon = np.empty_like(mon2nat)
    nat2mon[mon2nat] = np.arange(n_tokens, dtype=np.int64)
    return nat2mon, mon2nat


def to_monarch_order(x: torch.Tensor, f_tied, h_reduce, w_reduce, h, w) -> torch.Tensor:
    """[B, N, H, D] natural order -> [B, G, b1, b2, H, D]."""
    b, n, nh, d = x.shape
    g, b1, b2 = block_dims(n, f_tied, h_reduce, w_reduce, h, w)
    _, mon2nat = token_maps(n, f_tied, h_reduce, w_reduce, h, w)
    return x[:, torch.from_numpy(mon2nat)].reshape(b, g, b1, b2, nh, d)


def from_monarch_order(x: torch.Tensor, f_tied, h_reduce, w_reduce, h, w) -> torch.Tensor:
    """[B, G, b1, b2, H, D] -> [B, N, H, D] natural order."""
    b, g, b1, b2, nh, d = x.shape
    n = g * b1 * b2
    nat2mon, _ = token_maps(n, f_tied, h_reduce, w_reduce, h, w)
    return x.reshape(b, n, nh, d)[:, torch.from_numpy(nat2mon)]


# --------------------------------------------------------------------------- #
# rotary embedding  (model.py:421-428, causal_model.py:1352-1357, :687-715)
# --------------------------------------------------------------------------- #
def rope_table(head_dim: int = 128, max_len: int = 1024, theta: float = 10000.0
               ) -> Tuple[torch.Tensor, torch.Tensor, Tuple[int, int, int]]:
    """fp64 angle tables for the three axes.

    The head's ``head_dim/2`` complex pairs are split (frame, row, column) as
    ``c - 2*(c//3), c//3, c//3`` pairs with c = head_dim/2 (22/21/21 for 128).
    Axis ``x`` with ``p`` pairs uses angle ``pos * theta**(-(2m)/(2p))`` for
    m = 0..p-1.  Returns (cos, sin) of shape [max_len, c] (the three axes
    concatenated along the last dim) and the pair split.
    """
    c = head_dim // 2
    split = (c - 2 * (c // 3), c // 3, c // 3)
    pos = torch.arange(max_len, dtype=torch.float64)
    cols = []
    for p in split:
        dim_axis = 2 * p
        inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64),
                              torch.arange(0, dim_axis, 2, dtype=torch.float64) / dim_axis)
        cols.append(torch.outer(pos, inv))
    ang = torch.cat(cols, dim=1)
    return torch.cos(ang), torch.sin(ang), split


def rope_apply(x: torch.Tensor, grid: Tuple[int, int, int], start_frame: int = 0,
               theta: float = 10000.0) -> torch.Tensor:
    """Rotate x [B, L, H, D] for a (frames, rows, cols) token grid.

    Pairs are adjacent elements (x[2m], x[2m+1]); frame position is offset by
    ``start_frame``; the rotation is done in fp64 and cast back to x.dtype.
    Tokens beyond frames*rows*cols are passed through unchanged.
    """
    bsz, L, nh, d = x.shape
    f, hh, ww = grid
    seq = f * hh * ww
    cos, sin, split = rope_table(d, 1024, theta)
    p0, p1, p2 = split
    fi = torch.arange(f).view(f, 1, 1).expand(f, hh, ww).reshape(-1) + start_frame
    ri = torch.arange(hh).view(1, hh, 1).expand(f, hh, ww).reshape(-1)
    ci = torch.arange(ww).view(1, 1, ww).expand(f, hh, ww).reshape(-1)
    cs = torch.cat([cos[fi, :p0], cos[ri, p0:p0 + p1], cos[ci, p0 + p1:]], dim=1)  # [seq, c]
    sn = torch.cat([sin[fi, :p0], sin[ri, p0:p0 + p1], sin[ci, p0 + p1:]], dim=1)
    xr = x[:, :seq].to(torch.float64).reshape(bsz, seq, nh, d // 2, 2)
    re, im = xr[..., 0], xr[..., 1]
    cs = cs.view(1, seq, 1, d // 2)
    sn = sn.view(1, seq, 1, d // 2)
    out = torch.stack([re * cs - im * sn, re * sn + im * cs], dim=-1).reshape(bsz, seq, nh, d)
    out = out.to(x.dtype)
    if L > seq:
        out = torch.cat([out, x[:, seq:]], dim=1)
    return out


# --------------------------------------------------------------------------- #
# Monarch attention core on block-ordered tensors
# --------------------------------------------------------------------------- #
def _r_step(q_like, inv_c, K, V):
    """Row-block softmax step for one (batch, head).

    q_like [A, F, b1, b2, D]  (the "aR" operand: per query group a, kv group f,
                               row k, column j), inv_c [A, F, b1, b2] multiplier,
    K, V  [F, b1, b2, D].
    Returns aL [A,F,b1(k),b2(j),D], cL [A,F,b1,b2], Y (or None) like aL.
    """
    z = torch.matmul(q_like, K.unsqueeze(0).transpose(-1, -2))          # [A,F,k,j,l]
    z = z * inv_c.unsqueeze(-1)
    z = z - z.amax(dim=-1, keepdim=True)
    lse = torch.logsumexp(z, dim=-1, keepdim=True)
    R = torch.exp(z - lse)
    cL = (R * (z - lse)).sum(dim=-1)                                    # sum R ln R
    aL = torch.matmul(R, K.unsqueeze(0))                                # [A,F,k,j,D]
    Y = torch.matmul(R, V.unsqueeze(0)) if V is not None else None
    return aL, cL, Y


def _l_softmax(Q, aL, cL):
    """Column-block softmax over all (f, k) for every (a, j, i).

    Q [A, b1(i), b2(j), D], aL [A,F,b1(k),b2(j),D], cL [A,F,b1(k),b2(j)].
    Returns L [A, b2(j), b1(i), F*b1] (normalised).
    """
    A, F, b1, b2, D = aL.shape
    keys = aL.permute(0, 3, 1, 2, 4).reshape(A, b2, F * b1, D)         # [A,j,(f,k),D]
    bias = cL.permute(0, 3, 1, 2).reshape(A, b2, 1, F * b1)
    qj = Q.permute(0, 2, 1, 3)                                          # [A,j,i,D]
    logits = torch.matmul(qj, keys.transpose(-1, -2)) - bias            # [A,j,i,(f,k)]
    return torch.softmax(logits, dim=-1)


def monarch_core(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, sm_scale: float,
                 num_iters: int = 1) -> torch.Tensor:
    """Monarch attention on block-ordered inputs.

    Q [B, A, b1, b2, H, D]; K, V [B, F, b1, b2, H, D]; returns [B, A, b1, b2, H, D]
    in Q's dtype (arithmetic in Q's dtype; use fp32/fp64 inputs for an oracle).
    Both Q and K are multiplied by sqrt(sm_scale).  With ``num_iters == 1`` this
    is monarch_attn_ref_op (monarch_attn.py:1801-1830); otherwise it follows
    monarch_attn_slow (monarch_attn.py:1705-1751) including its
    ``min(1/(cR+1e-6), 1e4)`` multiplier, which that path also applies on its
    single pass when ``num_iters == 1`` is routed to it (``slow_form=True``).
    """
    return _monarch_core(Q, K, V, sm_scale, num_iters, slow_form=(num_iters != 1))


def _monarch_core(Q, K, V, sm_scale, num_iters, slow_form):
    B, A, b1, b2, H, D = Q.shape
    F = K.shape[1]
    rs = sm_scale ** 0.5
    out = torch.empty_like(Q)
    for b in range(B):
        for hd in range(H):
            q = Q[b, :, :, :, hd, :] * rs                               # [A,i,j,D]
            k = K[b, :, :, :, hd, :] * rs                               # [F,k,l,D]
            v = V[b, :, :, :, hd, :]
            aR = q.unsqueeze(1).expand(A, F, b1, b2, D)                 # row k uses Q[a,k,j]
            cR = torch.ones(A, F, b1, b2, dtype=q.dtype)
            for _ in range(num_iters - 1):
                inv = (1.0 / (cR + 1e-6)).clamp_max(1e4)
                aL, cL, _ = _r_step(aR, inv, k, None)
                L = _l_softmax(q, aL, cL).reshape(A, b2, b1, F, b1)     # [A,j,i,f,k]
                # aR[a,f,k,j,:] = sum_i L[a,j,i,f,k] Q[a,i,j,:] ; cR = sum_i L
                aR = torch.einsum("ajifk,aijd->afkjd", L, q)
                cR = L.sum(dim=2).permute(0, 2, 3, 1)                   # [A,f,k,j]
            if slow_form:
                inv = (1.0 / (cR + 1e-6)).clamp_max(1e4)
            else:
                inv = torch.ones_like(cR)
            aL, cL, Y = _r_step(aR, inv, k, v)
            L = _l_softmax(q, aL, cL)                                   # [A,j,i,(f,k)]
            vals = Y.permute(0, 3, 1, 2, 4).reshape(A, b2, F * b1, D)   # [A,j,(f,k),D]
            o = torch.matmul(L, vals)                                   # [A,j,i,D]
            out[b, :, :, :, hd, :] = o.permute(0, 2, 1, 3)
    return out


# --------------------------------------------------------------------------- #
# public entry points, mirroring the reference signatures
# --------------------------------------------------------------------------- #
def monarch_attn_with_kv_cache(q, k_cache, v_cache, new_k, new_v, start_idx, end_idx,
                               f_tied, h_reduce, w_reduce, h, w, sm_scale=None,
                               num_iters=1, grad_only_new_kv=False):
    """monarch_attn.py:1778-1796.  Writes new_k/new_v (in Monarch order) into
    k_cache/v_cache[:, start_idx:end_idx] IN PLACE, then attends q against the
    whole cache view.  q, new_k, new_v: [B, n, H, D] natural order; caches
    [B, n_kv, H, D] (possibly a strided view).  Returns [B, n_q, H, D]."""
    del grad_only_new_kv
    b, n_q, nh, d = q.shape
    if sm_scale is None:
        sm_scale = d ** -0.5
    Qb = to_monarch_order(q, f_tied, h_reduce, w_reduce, h, w)
    _, b1, b2 = Qb.shape[1:4]
    nk = to_monarch_order(new_k, f_tied, h_reduce, w_reduce, h, w).reshape(b, -1, nh, d)
    nv = to_monarch_order(new_v, f_tied, h_reduce, w_reduce, h, w).reshape(b, -1, nh, d)
    k_cache[:, start_idx:end_idx] = nk
    v_cache[:, start_idx:end_idx] = nv
    n_kv = k_cache.shape[1]
    if n_kv % (b1 * b2):
        raise ValueError("cache extent is not a whole number of Monarch groups")
    Kb = k_cache.reshape(b, n_kv // (b1 * b2), b1, b2, nh, d)
    Vb = v_cache.reshape(b, n_kv // (b1 * b2), b1, b2, nh, d)
    z = monarch_core(Qb, Kb, Vb, sm_scale, num_iters)
    return from_monarch_order(z, f_tied, h_reduce, w_reduce, h, w)


def monarch_attn(q, k, v, f_tied, h_reduce, w_reduce, h, w, sm_scale=None,
                 block_causal_size=None, num_iters=1):
    """monarch_attn.py:1753-1776 (no cache).  With ``block_causal_size`` the
    query groups of causal block c attend the kv groups of blocks 0..c
    (monarch_attn.py:1832-1858)."""
    b, n_q, nh, d = q.shape
    if sm_scale is None:
        sm_scale = d ** -0.5
    Qb = to_monarch_order(q, f_tied, h_reduce, w_reduce, h, w)
    Kb = to_monarch_order(k, f_tied, h_reduce, w_reduce, h, w)
    Vb = to_monarch_order(v, f_tied, h_reduce, w_reduce, h, w)
    b1, b2 = Qb.shape[2], Qb.shape[3]
    if block_causal_size is None:
        z = monarch_core(Qb, Kb, Vb, sm_scale, num_iters)
    else:
        if n_q % block_causal_size or k.shape[1] != n_q or block_causal_size % (b1 * b2):
            raise ValueError("bad block_causal_size")
        if num_iters != 1:
            raise ValueError("block-causal Monarch supports num_iters == 1 only")
        gpb = block_causal_size // (b1 * b2)
        parts = []
        for g0 in range(0, Qb.shape[1], gpb):
            parts.append(monarch_core(Qb[:, g0:g0 + gpb], Kb[:, :g0 + gpb], Vb[:, :g0 + gpb],
                                      sm_scale, 1))
        z = torch.cat(parts, dim=1)
    return from_monarch_order(z, f_tied, h_reduce, w_reduce, h, w)


def dense_attention(q, k, v, softmax_scale=None):
    """softmax(q k^T * scale) v over the whole key range, no mask.
    q [B, Lq, H, D]; k, v [B, Lk, H, D]; returns [B, Lq, H, D] in q's dtype."""
    d = q.shape[-1]
    if softmax_scale is None:
        softmax_scale = d ** -0.5
    qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
    s = torch.matmul(qh, kh.transpose(-1, -2)) * softmax_scale
    return torch.matmul(torch.softmax(s, dim=-1), vh).transpose(1, 2).contiguous()


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """WanRMSNorm.forward (wan/modules/model.py:470-478): normalise in fp32 over the last (full model
    width) dimension, round back to the input dtype, then multiply by the weight."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y.type_as(x) * weight


def cache_indices(current_start: int, num_new: int, global_end: int, local_end: int,
                  cache_size: int, max_attention_size: int, local_attn_size: int = -1,
                  sink_tokens: int = 0):
    """KV-cache bookkeeping of causal_model.py:907-938 as pure integer arithmetic.

    Returns a dict with: roll (None, or (dst_start, src_start, count) of the token
    range shifted left before the write), cache_start, local_start, local_end
    (both relative to cache_start, as passed to the attention op), and the new
    global_end / local_end values stored back into the cache (causal_model.py:1102-1103).
    """
    current_end = current_start + num_new
    roll = None
    if local_attn_size != -1 and current_end > global_end and num_new + local_end > cache_size:
        evicted = num_new + local_end - cache_size
        rolled = local_end - evicted - sink_tokens
        roll = (sink_tokens, sink_tokens + evicted, rolled)
        new_local_end = local_end + current_end - global_end - evicted
    else:
        new_local_end = local_end + current_end - global_end
    new_local_start = new_local_end - num_new
    cache_start = max(0, new_local_end - max_attention_size)
    return {
        "roll": roll,
        "cache_start": cache_start,
        "local_start": new_local_start - cache_start,
        "local_end": new_local_end - cache_start,
        "store_global_end": current_end,
        "store_local_end": new_local_end - cache_start,
    }

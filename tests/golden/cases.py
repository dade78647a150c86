"""Seeded input builders shared by ``make_golden.py`` (which runs the reference
on them) and the tests (which run the oracle and the CUDA kernels on them).

All randomness is ``numpy.random.default_rng(seed).standard_normal`` in fp32, a
stream that NumPy keeps stable across versions, so the fixtures only need to
store outputs.
"""
from __future__ import annotations

import numpy as np
import torch

SMALL_BLOCKINGS = [
    # name, f_tied, h_reduce, w_reduce, h, w
    ("framewise", 1, 1, 1, 6, 8),
    ("tied3frame", 3, 1, 1, 6, 8),
    ("reduce2xh", 1, 2, 1, 6, 8),
    ("reduce4xw2xh", 1, 2, 4, 6, 8),
    ("tied3_reduce", 3, 3, 2, 6, 8),
]
SMALL_ITERS = (1, 2, 5)
NOCACHE_ITERS = (1, 3)

REAL_BLOCKINGS = [("framewise", 1, 1, 1), ("tied3frame", 3, 1, 1),
                  ("reduce2xh", 1, 2, 1), ("reduce4xw2xh", 1, 2, 4)]

MAP_CASES = [(1, 1, 1, 30, 52, 4680), (3, 1, 1, 30, 52, 4680), (1, 2, 1, 30, 52, 4680),
             (1, 2, 4, 30, 52, 4680), (1, 6, 13, 30, 52, 4680), (1, 6, 4, 30, 52, 1560),
             (3, 3, 2, 6, 8, 288), (1, 5, 4, 30, 52, 3120), (3, 2, 4, 30, 52, 9360)]


def randn(rng, *shape):
    return torch.from_numpy(rng.standard_normal(shape, dtype=np.float32))


def rope_inputs():
    """x [2, 3*5*7+4, 2, 128] (4 trailing pass-through tokens), grid (3,5,7)."""
    rng = np.random.default_rng(101)
    return randn(rng, 2, 3 * 5 * 7 + 4, 2, 128), (3, 5, 7)


def rmsnorm_inputs():
    """x [2, 11, 3*128] (three heads wide) with a spread of row magnitudes, weight [384], eps."""
    rng = np.random.default_rng(303)
    x = randn(rng, 2, 11, 384) * torch.from_numpy(rng.uniform(0.2, 4.0, size=(2, 11, 1)).astype(np.float32))
    w = torch.from_numpy(rng.uniform(0.5, 1.5, size=384).astype(np.float32))
    return x, w, 1e-6


def cache_case(ci: int, iters: int):
    """Small cache-path case: B=2, H=2, D=32, chunk of 3 frames written at the
    end of a 3-chunk view of a 4-chunk buffer (so the batch stride exceeds the view)."""
    name, ft, hr, wr, h, w = SMALL_BLOCKINGS[ci]
    rng = np.random.default_rng(1000 + 10 * ci + iters)
    B, H, D = 2, 2, 32
    chunk = 3 * h * w
    n_buf, n_kv = 4 * chunk, 3 * chunk
    q = randn(rng, B, chunk, H, D)
    nk = randn(rng, B, chunk, H, D)
    nv = randn(rng, B, chunk, H, D)
    kbuf = randn(rng, B, n_buf, H, D)
    vbuf = randn(rng, B, n_buf, H, D)
    return dict(name=name, blocking=(ft, hr, wr, h, w), q=q, nk=nk, nv=nv, kbuf=kbuf, vbuf=vbuf,
                start=n_kv - chunk, end=n_kv, n_kv=n_kv, sm_scale=D ** -0.5, iters=iters)


def nocache_case(ci: int):
    name, ft, hr, wr, h, w = SMALL_BLOCKINGS[ci]
    rng = np.random.default_rng(2000 + ci)
    B, H, D = 1, 2, 32
    n = 6 * h * w
    q, k, v = randn(rng, B, n, H, D), randn(rng, B, n, H, D), randn(rng, B, n, H, D)
    return dict(name=name, blocking=(ft, hr, wr, h, w), q=q, k=k, v=v, sm_scale=D ** -0.5,
                block_causal=3 * h * w)


def real_case():
    """One head at the real block sizes: 30 x 52 grid, D=128, chunk appended to a 1-chunk cache."""
    rng = np.random.default_rng(3000)
    B, H, D, h, w = 1, 1, 128, 30, 52
    chunk = 3 * h * w
    q, nk, nv = randn(rng, B, chunk, H, D), randn(rng, B, chunk, H, D), randn(rng, B, chunk, H, D)
    kbuf, vbuf = randn(rng, B, 2 * chunk, H, D), randn(rng, B, 2 * chunk, H, D)
    return dict(q=q, nk=nk, nv=nv, kbuf=kbuf, vbuf=vbuf, start=chunk, end=2 * chunk, h=h, w=w,
                sm_scale=D ** -0.5)


def c1_case():
    """BASELINE config 1: B=1, 12 heads, D=128, one 3-frame chunk, empty cache."""
    rng = np.random.default_rng(0)
    B, H, D, h, w = 1, 12, 128, 30, 52
    chunk = 3 * h * w
    q, k, v = randn(rng, B, chunk, H, D), randn(rng, B, chunk, H, D), randn(rng, B, chunk, H, D)
    return dict(q=q, k=k, v=v, h=h, w=w, chunk=chunk, sm_scale=D ** -0.5)


# ---------------------------------------------------------------------------------------------
# second fixture file (pins_golden.npz): gradients, dense attention, cache bookkeeping
# ---------------------------------------------------------------------------------------------
PIN_CHANNEL_STRIDE = 2            # gradient fixtures keep every second head-dim channel (file size)


def _bf16_round(t):
    return t.to(torch.bfloat16).to(torch.float32)


def grad_case(ci: int):
    """Cache-path gradient case at head_dim 128 (the only size the kernels are built for): B=1, H=2, the
    last `frames_q` tied frame sets of a `groups` set cache written by the call.  Values are rounded to
    bf16 so that the reference (fp32 arithmetic) and the kernels (bf16 storage) see the same numbers."""
    name, ft, hr, wr, h, w = SMALL_BLOCKINGS[ci]
    rng = np.random.default_rng(8100 + ci)
    frames_q, sets = (2, 4) if ft == 1 else (1, 2)
    tied = ft * h * w
    n_q, n_kv = frames_q * tied, sets * tied
    B, H, D = 1, 2, 128
    mk = lambda n: _bf16_round(randn(rng, B, n, H, D))
    return dict(name=name, blocking=(ft, hr, wr, h, w), q=mk(n_q), nk=mk(n_q), nv=mk(n_q), kbuf=mk(n_kv + tied),
                vbuf=mk(n_kv + tied), g=mk(n_q), start=n_kv - n_q, end=n_kv, n_kv=n_kv, sm_scale=D ** -0.5)


CAUSAL_GRAD_CASES = [(0, 2), (3, 3)]      # (index into SMALL_BLOCKINGS, frames per causal block)


def causal_grad_case(i: int):
    ci, causal_frames = CAUSAL_GRAD_CASES[i]
    name, ft, hr, wr, h, w = SMALL_BLOCKINGS[ci]
    rng = np.random.default_rng(8600 + i)
    n = 6 * ft * h * w
    B, H, D = 1, 2, 128
    mk = lambda: _bf16_round(randn(rng, B, n, H, D))
    return dict(name=name, blocking=(ft, hr, wr, h, w), q=mk(), k=mk(), v=mk(), g=mk(),
                block_causal=causal_frames * ft * h * w, sm_scale=D ** -0.5)


DENSE_CASES = [(50, 170), (333, 1000)]


def dense_case(i: int):
    """Dense attention: B=1, H=2, D=128, K/V given as a view shorter than their buffer."""
    n_q, n_kv = DENSE_CASES[i]
    rng = np.random.default_rng(31 + n_q)
    mk = lambda n: _bf16_round(randn(rng, 1, n, 2, 128))
    return dict(q=mk(n_q), kbuf=mk(n_kv + 64), vbuf=mk(n_kv + 64), n_kv=n_kv)


# Rollouts replayed through the reference's CausalWanSelfAttention.forward cache branch.  Each scenario:
# cache size in frames, local_attn_size, sink_size (frames), and the list of (chunk index, repeats) layer
# calls: a chunk of 3 frames starts at token 3 * 1560 * chunk index and is called `repeats` times (the
# pipeline rewrites the chunk's slot with every denoising step and once more with the clean context).
BOOKKEEPING_SCENARIOS = {
    "global_7chunks": dict(cache_frames=21, local_attn_size=-1, sink_size=0,
                           calls=[(c, 5) for c in range(7)]),
    "window9_sink0": dict(cache_frames=9, local_attn_size=9, sink_size=0,
                          calls=[(c, 2) for c in range(6)]),
    "window12_sink3": dict(cache_frames=12, local_attn_size=12, sink_size=3,
                           calls=[(c, 3) for c in range(7)]),
    # a cache longer than the attention window: no eviction until it is full, but the view starts past 0
    "window6_cache21": dict(cache_frames=21, local_attn_size=6, sink_size=0,
                            calls=[(c, 2) for c in range(7)]),
    "window6_sink1_dense_init": dict(cache_frames=6, local_attn_size=6, sink_size=1,
                                     calls=[(c, 2) for c in range(5)], dense_init=True),
}
BOOKKEEPING_ID_STRIDE = 130       # the cache's token ids are stored every 130 tokens (12 per frame)

"""The allocation-free entry point (sfm_monarch_fwd_static) against the ordinary one.

Some callers may not allocate device memory at the point where they run attention (the
allocator is frozen, or all memory was handed out up front), so the library also offers the
Monarch forward on a 32 MiB scratch array compiled into it.  This test drives both entry points
through the C ABI on the same inputs, twice in a row (the array is shared and keeps the first
call's contents), and also checks that an oversized problem is refused without a launch.  The
file name sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes as C
import gc

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _run_both(lib, q, kc, vc, blocking, n_kv, num_iters=1):
    B, n_q, H, D = q.shape
    ft, hr, wr, h, w = blocking
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    cache_bs = kc.stride(0) if B > 1 else kc.shape[1] * H * D
    q_bs = n_q * H * D

    nbytes = lib.sfm_monarch_workspace_bytes(B, H, D, n_q, n_kv, ft, hr, wr, h, w, num_iters, 0)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    ref = torch.empty_like(q)
    rc = lib.sfm_monarch_fwd(_ptr(q), q_bs, _ptr(kc), _ptr(vc), cache_bs, _ptr(ref), _ptr(ws), nbytes, B, H, D, n_q,
                             n_kv, ft, hr, wr, h, w, D ** -0.5, num_iters, 0, stream)
    assert rc == 0, lib.sfm_error_string(rc)

    got = torch.full_like(q, float("nan"))
    gc.collect()                                            # garbage of earlier tests must not be freed in between
    before = torch.cuda.memory_allocated()
    rc = lib.sfm_monarch_fwd_static(_ptr(q), q_bs, _ptr(kc), _ptr(vc), cache_bs, _ptr(got), B, H, D, n_q, n_kv,
                                    ft, hr, wr, h, w, D ** -0.5, num_iters, stream)
    assert rc == 0, lib.sfm_error_string(rc)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before          # nothing went through torch's allocator
    return got, ref


def test_static_scratch_matches_workspace_entry_point():
    from self_forcing_b200 import _lib
    lib = _lib.load()
    assert lib.sfm_static_scratch_bytes() == 32 << 20
    rng = np.random.default_rng(2024)
    B, H, D, h, w = 2, 3, 128, 30, 52
    n, k = 3 * h * w, 2
    mk = lambda *s: torch.from_numpy(rng.standard_normal(s, dtype=np.float32)).to(torch.bfloat16).cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # three calls in a row on the shared array: two single-pass blockings, then the iterative variant
    for call, (blocking, iters) in enumerate([((1, 1, 1, h, w), 1), ((1, 2, 4, h, w), 1), ((1, 1, 1, h, w), 2)]):
        q = mk(B, n, H, D)
        kbuf, vbuf = mk(B, 3 * n, H, D), mk(B, 3 * n, H, D)                   # view shorter than the buffer
        got, ref = _run_both(lib, q, kbuf[:, :k * n], vbuf[:, :k * n], blocking, k * n, num_iters=iters)
        assert lib.sfm_static_scratch_status(stream) == 0                     # no kernel gave up on a wait
        assert torch.isfinite(got).all(), f"call {call}: non-finite output"
        # cutting the work into smaller chunks changes the launches, not one bit of the result
        assert torch.equal(got, ref), f"call {call}: max-abs {(got.float() - ref.float()).abs().max().item():.3e}"


def test_static_scratch_refuses_oversized_problems():
    from self_forcing_b200 import _lib
    lib = _lib.load()
    # a cache three times the 480p rollout: one (head, query group) slice of row-step results is
    # 52 columns x 1890 keys x 516 bytes = 50.7 MB > 32 MiB
    one = C.c_void_p(256)
    rc = lib.sfm_monarch_fwd_static(one, 0, one, one, 0, one, 1, 12, 128, 4680, 3 * 32760, 1, 1, 1, 30, 52, 0.088, 1,
                                    C.c_void_p(0))
    assert rc == -8
    assert b"built-in scratch" in lib.sfm_error_string(rc)

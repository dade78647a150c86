"""Two-rank CPU (gloo) tests of the multi-GPU host logic: the Ulysses token<->head all-to-alls and
the head-sharded attention wrapper, checked against the unsharded oracle.  The attention arithmetic
on each rank is the CPU oracle (injected), so no GPU is needed; the layout and collective code is
the product's."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from self_forcing_b200.ulysses import UlyssesSelfAttention, heads_to_tokens, tokens_to_heads
        from oracle import monarch_oracle as orc

        rng = np.random.default_rng(99)                      # same stream on every rank
        B, H, D, h, w = 2, 4, 16, 6, 8
        n = 3 * h * w
        mk = lambda *s: torch.from_numpy(rng.standard_normal(s, dtype=np.float32))
        q, k, v = mk(B, n, H, D), mk(B, n, H, D), mk(B, n, H, D)
        kbuf, vbuf = mk(B, 2 * n, H, D), mk(B, 2 * n, H, D)
        sp, hp = n // world, H // world
        tok = slice(rank * sp, (rank + 1) * sp)
        hd = slice(rank * hp, (rank + 1) * hp)

        # 1. layout round trip and content of the head shard
        qh, kh = tokens_to_heads([q[:, tok], k[:, tok]])
        assert torch.equal(qh, q[:, :, hd]) and torch.equal(kh, k[:, :, hd])
        assert torch.equal(heads_to_tokens(qh), q[:, tok])

        # 2. head-sharded attention == unsharded attention
        blocking = (1, 2, 4, h, w)

        def attn(qh, kh, vh, kc, vc, s, e, start_frame):
            rq = orc.rope_apply(qh, (3, h, w), start_frame)
            rk = orc.rope_apply(kh, (3, h, w), start_frame)
            return orc.monarch_attn_with_kv_cache(rq, kc[:, :e], vc[:, :e], rk, vh, s, e, *blocking)

        op = UlyssesSelfAttention(blocking, attn_fn=attn)
        kc_local, vc_local = kbuf[:, :, hd].clone(), vbuf[:, :, hd].clone()
        out = op(q[:, tok], k[:, tok], v[:, tok], kc_local, vc_local, n, 2 * n, start_frame=3)

        kc_full, vc_full = kbuf.clone(), vbuf.clone()
        ref = attn(q, k, v, kc_full, vc_full, n, 2 * n, 3)
        np.testing.assert_allclose(out.numpy(), ref[:, tok].numpy(), rtol=1e-5, atol=1e-6)
        assert torch.equal(kc_local, kc_full[:, :, hd])        # each rank's cache holds its heads only

        # 3. a rank with indivisible sizes gets a clear error instead of a hang
        with pytest.raises(ValueError):
            tokens_to_heads([mk(1, 4, 3, 8)])
        Path(result_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_ulysses_two_ranks(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_single_rank_is_identity():
    """With a one-rank group the layout functions are the identity (the single-GPU path)."""
    port = _free_port()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        from self_forcing_b200.ulysses import heads_to_tokens, tokens_to_heads
        x = torch.arange(2 * 6 * 4 * 8, dtype=torch.float32).reshape(2, 6, 4, 8)
        assert torch.equal(tokens_to_heads([x])[0], x) and torch.equal(heads_to_tokens(x), x)
    finally:
        dist.destroy_process_group()

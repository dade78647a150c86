"""Head sharding of the self-attention op across the GPUs of one box (Ulysses style).

Outside attention every rank holds a slice of the chunk's tokens ([B, S/P, H, D]); inside attention
every rank holds all tokens of a slice of the heads ([B, S, H/P, D]) together with the KV cache of
those heads only.  Two all-to-alls per layer move between the two layouts: q, k, v go in fused in
one message, the attention output comes back in a second one.  The collective is
``torch.distributed.all_to_all_single`` (NCCL over NVLink on GPUs, gloo in the CPU tests); the
attention itself is unchanged, since heads are independent in every kernel of this package.

The reference has no sequence/head parallel path for the causal model (its only precedent is the
xfuser-based wrapper for the bidirectional model, wan/distributed/xdit_context_parallel.py:131-184),
so this module has no reference counterpart to mirror; independent videos on different ranks
(plain data parallelism, inference.py:116-120 of the reference) need no code here at all.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


def _check(x: torch.Tensor, world: int, shard_dim: int) -> None:
    if x.dim() != 4:
        raise ValueError("expected [B, tokens, heads, dim]")
    if x.shape[shard_dim] % world:
        raise ValueError(f"dimension {shard_dim} ({x.shape[shard_dim]}) is not divisible by the group size {world}")


def tokens_to_heads(xs: Sequence[torch.Tensor], group: Optional[dist.ProcessGroup] = None) -> list:
    """[B, S/P, H, D] token shards -> [B, S, H/P, D] head shards, for several tensors in ONE
    all-to-all.  Rank r ends up with heads [r*H/P, (r+1)*H/P) of all S tokens (token order =
    rank order of the shards)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return [x.contiguous() for x in xs]
    n = len(xs)
    for x in xs:
        _check(x, world, 2)
    B, Sp, H, D = xs[0].shape
    Hp = H // world
    # send buffer [P(dest), n, B, S/P, H/P, D]: block p goes to rank p
    send = torch.stack([x.reshape(B, Sp, world, Hp, D).permute(2, 0, 1, 3, 4) for x in xs], dim=1).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv [P(src), n, B, S/P, H/P, D] -> per tensor [B, P*S/P, H/P, D]
    out = []
    for i in range(n):
        out.append(recv[:, i].permute(1, 0, 2, 3, 4).reshape(B, world * Sp, Hp, D).contiguous())
    return out


def heads_to_tokens(x: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """[B, S, H/P, D] head shard -> [B, S/P, H, D] token shard (inverse of tokens_to_heads)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return x.contiguous()
    _check(x, world, 1)
    B, S, Hp, D = x.shape
    Sp = S // world
    send = x.reshape(B, world, Sp, Hp, D).permute(1, 0, 2, 3, 4).contiguous()      # [P(dest), B, S/P, H/P, D]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv [P(src = head block), B, S/P, H/P, D] -> [B, S/P, P*H/P, D]
    return recv.permute(1, 2, 0, 3, 4).reshape(B, Sp, world * Hp, D).contiguous()


class UlyssesSelfAttention:
    """Self-attention of one layer with heads sharded over ``group``.

    ``attn_fn(q, k, v, k_cache, v_cache, start_idx, end_idx) -> out`` runs on the local heads; by
    default it is this package's fused RoPE + cache write + Monarch attention.  The caches passed to
    ``__call__`` hold the local heads only: [B, cache_tokens, H/P, D].
    """

    def __init__(self, blocking, group: Optional[dist.ProcessGroup] = None,
                 attn_fn: Optional[Callable] = None, num_iters: int = 1):
        self.blocking = tuple(blocking)          # (f_tied, h_reduce, w_reduce, h, w)
        self.group = group
        self.num_iters = num_iters
        self.attn_fn = attn_fn

    def _default_attn(self, q, k, v, k_cache, v_cache, start_idx, end_idx, start_frame):
        from . import ops
        n_kv = end_idx
        return ops.rope_monarch_attn_with_kv_cache(q, k, v, k_cache[:, :n_kv], v_cache[:, :n_kv], start_idx, end_idx,
                                                   start_frame, *self.blocking, num_iters=self.num_iters)

    def __call__(self, q, k, v, k_cache, v_cache, start_idx, end_idx, start_frame=0):
        """q, k, v: this rank's token shard [B, S/P, H, D] of the un-rotated projections (token order
        across ranks = rank order).  Returns this rank's token shard of the attention output."""
        qh, kh, vh = tokens_to_heads([q, k, v], self.group)
        if self.attn_fn is not None:
            out = self.attn_fn(qh, kh, vh, k_cache, v_cache, start_idx, end_idx, start_frame)
        else:
            out = self._default_attn(qh, kh, vh, k_cache, v_cache, start_idx, end_idx, start_frame)
        return heads_to_tokens(out, self.group)


class PeerShardedSelfAttention:
    """Head-sharded self-attention of one layer in which the kernels do the exchange themselves.

    Instead of two all-to-all collectives (and the packing copies around them), the fused RoPE +
    cache-write kernel READS every rank's token shard of q, k, v over NVLink and the attention
    kernel WRITES each result row straight into the token shard of the rank that owns the token.
    The shards live in symmetric memory (``torch.distributed._symmetric_memory``) so that every rank
    has the peers' addresses; two device-side barriers per call order the peer accesses:

        write q, k, v into ``self.q_in`` / ``k_in`` / ``v_in`` (e.g. as outputs of the projections)
        out = attn(k_cache, v_cache, start_idx, end_idx, start_frame)     # -> ``self.out`` (token shard)

    ``out`` is overwritten by the next call; the caches hold the local heads only.  GPUs only (the
    CPU tests cover the all-to-all path of UlyssesSelfAttention, which computes the same result).
    """

    def __init__(self, blocking, batch: int, chunk_tokens: int, heads_total: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.blocking = tuple(blocking)
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if chunk_tokens % self.world or heads_total % self.world:
            raise ValueError("tokens and heads must divide evenly over the ranks")
        self.shape = (batch, chunk_tokens // self.world, heads_total, 128)
        n = batch * (chunk_tokens // self.world) * heads_total * 128
        buf = symm_mem.empty(4 * n, dtype=torch.bfloat16, device=device)      # q, k, v in; out
        self._hdl = symm_mem.rendezvous(buf, self.group)
        self._buf = buf
        views = [buf[i * n:(i + 1) * n].view(self.shape) for i in range(4)]
        self.q_in, self.k_in, self.v_in, self.out = views
        base = [int(p) for p in self._hdl.buffer_ptrs]
        nbytes = n * 2
        self._ptrs = [[b + i * nbytes for b in base] for i in range(4)]

    def barrier(self):
        self._hdl.barrier()

    def __call__(self, k_cache, v_cache, start_idx, end_idx, start_frame=0, rotate=True):
        """``rotate=False`` when q_in / k_in already hold rotated values (ops.norm_rope_token_slice)."""
        from . import ops
        self._hdl.barrier()                       # every rank's q_in / k_in / v_in are complete
        ops.rope_monarch_attn_with_kv_cache_sharded(self._ptrs[0], self._ptrs[1], self._ptrs[2], self._ptrs[3],
                                                    self.rank, self.shape, k_cache, v_cache, start_idx, end_idx,
                                                    start_frame, *self.blocking, rotate=rotate)
        self._hdl.barrier()                       # every rank's rows have landed in self.out
        return self.out

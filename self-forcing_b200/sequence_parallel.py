"""Sequence-parallel KV-cache forward of the reference's causal Wan DiT over the GPUs of one box.

For Wan-14B the attention heads are sharded over P GPUs (``ulysses.py``).  Attention is under a tenth of
the model's arithmetic, so the rest of every block has to be sharded too or P GPUs run barely faster than
one: outside attention each rank therefore works on a contiguous slice of S/P tokens of the chunk, inside
attention on all tokens of H/P heads with the KV cache of those heads only, and the two layouts are
exchanged twice per layer (all-to-all, or the kernels' own peer-memory gather / scatter).

The reference's block cannot run on such a slice as written: it un-flattens the tokens into whole frames to
apply the per-frame modulation (``x.shape[1] // e.shape[1]``, wan/modules/causal_model.py:1176-1201; head
:1233-1235), and S/P tokens are not a whole number of frames.  ``SequenceParallelCausalWan`` re-states
``CausalWanModel._forward_inference`` (:1582-1720), ``CausalWanAttentionBlock.forward`` (:1152-1205) and
``CausalHead.forward`` (:1225-1236) around the model's OWN sub-modules and parameters with the modulation
looked up per token (``e[:, token // tokens_per_frame]``, applied frame piece by frame piece as broadcasts),
which is the same arithmetic element for element; nothing in the model object is modified.  The only precedent in the reference is the xfuser
wrapper for the bidirectional model (wan/distributed/xdit_context_parallel.py:66-146: chunk after the
embeddings, all-gather after the head).

Weights are replicated (28 GB in bf16 for Wan-14B).  The sliding-window cache is not supported here (the
global window is what the 21-frame rollout uses).
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

from .layer import KVCache, plan_cache_step
from .ulysses import UlyssesSelfAttention


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def shard_tokens(x: torch.Tensor, group=None) -> torch.Tensor:
    """[B, S, ...] -> this rank's contiguous token slice [B, S/P, ...]."""
    world, rank = _world(group), _rank(group)
    if x.shape[1] % world:
        raise ValueError(f"{x.shape[1]} tokens do not divide over {world} ranks")
    sp = x.shape[1] // world
    return x[:, rank * sp:(rank + 1) * sp].contiguous()


def gather_tokens(x: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of shard_tokens: [B, S/P, ...] on every rank -> [B, S, ...] on every rank."""
    world = _world(group)
    if world == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=1)


class SequenceParallelCausalWan:
    """``model`` is a ``CausalWanModel`` of the reference (or any module with its attributes).

    ``attn_fn(qh, kh, vh, k_cache, v_cache, start_idx, end_idx, start_frame) -> out`` runs attention on the
    local heads ([B, S, H/P, D], un-rotated q / k after their norms); by default it is this package's fused
    RoPE + cache write + Monarch attention.  ``blocking`` = (f_tied, h_reduce, w_reduce); the token grid comes
    from the input."""

    def __init__(self, model, blocking=(1, 1, 1), group=None, attn_fn: Optional[Callable] = None, num_iters: int = 1,
                 exchange: str = "all_to_all"):
        if exchange not in ("all_to_all", "peer"):
            raise ValueError("exchange must be 'all_to_all' (NCCL / gloo collectives) or 'peer' (the kernels gather "
                             "and scatter over peer memory; GPUs of one box, single-pass Monarch only)")
        self.model = model
        self.group = group
        self.blocking = tuple(blocking)
        self.attn_fn = attn_fn
        self.num_iters = num_iters
        self.exchange = exchange
        self._peer = None
        self.world, self.rank = _world(group), _rank(group)
        if model.num_heads % self.world:
            raise ValueError(f"{model.num_heads} heads do not divide over {self.world} ranks")
        self.local_heads = model.num_heads // self.world
        self._ulysses = None

    # ------------------------------------------------------------------------------ caches
    def allocate_kv_caches(self, batch: int, cache_tokens: int, device, dtype=torch.bfloat16) -> List[KVCache]:
        """One cache per block holding this rank's heads only: [B, cache_tokens, H/P, 128]."""
        hd = self.model.dim // self.model.num_heads
        mk = lambda: torch.zeros(batch, cache_tokens, self.local_heads, hd, dtype=dtype, device=device)
        return [KVCache(mk(), mk()) for _ in range(self.model.num_layers)]

    @staticmethod
    def allocate_crossattn_caches(model, batch: int, device, dtype=torch.bfloat16) -> List[dict]:
        hd = model.dim // model.num_heads
        return [{"k": torch.zeros(batch, 512, model.num_heads, hd, dtype=dtype, device=device),
                 "v": torch.zeros(batch, 512, model.num_heads, hd, dtype=dtype, device=device), "is_init": False}
                for _ in range(model.num_layers)]

    # ------------------------------------------------------------------------------ pieces
    def _self_attention(self, attn, h, cache: KVCache, current_start: int, grid):
        """The cache branch of CausalWanSelfAttention.forward on a token slice: projections and norms are
        per token; rotation, cache write and attention run on the local heads between the two exchanges."""
        frames, gh, gw = grid
        b, sp = h.shape[:2]
        n, d = attn.num_heads, attn.head_dim
        fused = (self.exchange == "peer" and self.world > 1 and h.dtype == torch.bfloat16 and
                 getattr(attn.norm_q, "weight", None) is not None and attn.norm_q.weight.dtype == torch.bfloat16)
        if fused:                                  # norms and rotation happen in one kernel further down
            q, k = attn.q(h).view(b, sp, n, d), attn.k(h).view(b, sp, n, d)
        else:
            q = attn.norm_q(attn.q(h)).view(b, sp, n, d)
            k = attn.norm_k(attn.k(h)).view(b, sp, n, d)
        v = attn.v(h).view(b, sp, n, d)
        n_new = sp * self.world
        step = plan_cache_step(current_start, n_new, cache.global_end, cache.local_end, cache.k.shape[1],
                               cache.k.shape[1])
        if step.roll is not None or step.cache_start != 0:
            raise NotImplementedError("sequence parallelism runs with the global attention window")
        start_frame = current_start // (gh * gw)
        if self.exchange == "peer" and self.world > 1:
            if self._peer is None or self._peer.shape != (b, sp, n, d):
                from .ulysses import PeerShardedSelfAttention
                self._peer = PeerShardedSelfAttention(self.blocking + (gh, gw), b, n_new, n, h.device, self.group)
            if fused:
                from . import ops
                # RMSNorm + RoPE of this rank's token slice, written straight into the buffers the peers read
                ops.norm_rope_token_slice(q, k, v, self._peer.q_in, self._peer.k_in, self._peer.v_in, self.rank * sp,
                                          start_frame, gh, gw, freqs=self.model.freqs, norm_q_weight=attn.norm_q.weight,
                                          norm_k_weight=attn.norm_k.weight, eps=attn.eps)
            else:
                self._peer.q_in.copy_(q)
                self._peer.k_in.copy_(k)
                self._peer.v_in.copy_(v)
            out = self._peer(cache.k, cache.v, step.local_start, step.local_end, start_frame, rotate=not fused)
        else:
            if self._ulysses is None:
                self._ulysses = UlyssesSelfAttention(self.blocking + (gh, gw), self.group, self.attn_fn, self.num_iters)
            out = self._ulysses(q, k, v, cache.k, cache.v, step.local_start, step.local_end, start_frame=start_frame)
        cache._store(step)
        return attn.o(out.flatten(2))

    @staticmethod
    def _modulate(x, scale, shift, segments):
        """x * (1 + scale[frame of token]) + shift[frame of token] without materialising per-token factors: a token
        slice covers a few whole or partial frames, each handled as one broadcast over its tokens.
        scale, shift: [B, F, C]; segments: [(first token, end token, frame)] of this rank's slice."""
        out = torch.empty_like(x)
        for t0, t1, f in segments:
            torch.addcmul(shift[:, f:f + 1], x[:, t0:t1], 1 + scale[:, f:f + 1], out=out[:, t0:t1])
        return out

    @staticmethod
    def _gated_add(x, y, gate, segments):
        """x + y * gate[frame of token], same segment-wise broadcast."""
        out = torch.empty_like(x)
        for t0, t1, f in segments:
            torch.addcmul(x[:, t0:t1], y[:, t0:t1], gate[:, f:f + 1], out=out[:, t0:t1])
        return out

    def _block(self, block, x, e0, segments, grid, context, context_lens, cache, crossattn_cache, current_start):
        """CausalWanAttentionBlock.forward on a token slice; e0 = per-frame time projection [B, F, 6, C]."""
        e = (block.modulation.unsqueeze(1) + e0).unbind(dim=2)         # six [B, F, C], as in the reference
        y = self._self_attention(block.self_attn, self._modulate(block.norm1(x), e[1], e[0], segments), cache,
                                 current_start, grid)
        x = self._gated_add(x, y, e[2], segments)
        x = x + block.cross_attn(block.norm3(x), context, context_lens, crossattn_cache=crossattn_cache)
        y = block.ffn(self._modulate(block.norm2(x), e[4], e[3], segments))
        return self._gated_add(x, y, e[5], segments)

    def _head(self, head, x, e, segments):
        """CausalHead.forward on a token slice; e = per-frame time embedding [B, F, 1, C]."""
        e = (head.modulation.unsqueeze(1) + e).unbind(dim=2)           # two [B, F, C]
        return head.head(self._modulate(head.norm(x), e[1], e[0], segments))

    # ------------------------------------------------------------------------------ forward
    def forward(self, x, t, context, kv_caches: List[KVCache], crossattn_caches: List[dict], current_start: int = 0):
        """x: list / batch of [C_in, F, H, W] latents (the chunk), t: [B, F] timesteps, context: list of [L, C]
        text embeddings.  Returns [B, C_out, F, H, W], identical on every rank."""
        from_model = _import_from_model_module(self.model)
        m = self.model
        device = m.patch_embedding.weight.device
        if m.freqs.device != device:
            m.freqs = m.freqs.to(device)
        x = [m.patch_embedding(u.unsqueeze(0)) for u in x]
        grid_sizes = torch.stack([torch.tensor(u.shape[2:], dtype=torch.long) for u in x])
        grid = tuple(int(g) for g in grid_sizes[0].tolist())
        if any(tuple(int(g) for g in row.tolist()) != grid for row in grid_sizes):
            raise NotImplementedError("all samples must share one token grid")
        x = torch.cat([u.flatten(2).transpose(1, 2) for u in x])                  # [B, S, C]
        frame_tokens = grid[1] * grid[2]

        e = m.time_embedding(from_model.sinusoidal_embedding_1d(m.freq_dim, t.flatten()).type_as(x))
        e0 = m.time_projection(e).unflatten(1, (6, m.dim)).unflatten(dim=0, sizes=t.shape)     # [B, F, 6, C]
        context = m.text_embedding(torch.stack([
            torch.cat([u, u.new_zeros(m.text_len - u.size(0), u.size(1))]) for u in context]))

        x = shard_tokens(x, self.group)
        sp = x.shape[1]
        # this rank's tokens [rank * sp, (rank + 1) * sp) cut at frame boundaries: (first, end, frame) per piece
        segments, g0 = [], self.rank * sp
        while g0 < (self.rank + 1) * sp:
            f = g0 // frame_tokens
            g1 = min((f + 1) * frame_tokens, (self.rank + 1) * sp)
            segments.append((g0 - self.rank * sp, g1 - self.rank * sp, f))
            g0 = g1
        for i, block in enumerate(m.blocks):
            x = self._block(block, x, e0, segments, grid, context, None, kv_caches[i], crossattn_caches[i], current_start)
        x = self._head(m.head, x, e.unflatten(dim=0, sizes=t.shape).unsqueeze(2), segments)
        x = gather_tokens(x, self.group)
        return torch.stack(m.unpatchify(x, grid_sizes))

    __call__ = forward


def _import_from_model_module(model):
    """The module that defines the model's class also exports sinusoidal_embedding_1d (imported there from
    wan/modules/model.py); take it from wherever the class lives so that no import path is assumed."""
    import sys
    mod = sys.modules[type(model).__module__]
    if not hasattr(mod, "sinusoidal_embedding_1d"):
        raise RuntimeError("the model's module does not provide sinusoidal_embedding_1d")
    return mod


class SequenceParallelModelAdapter(torch.nn.Module):
    """Stands where ``WanDiffusionWrapper.model`` stands, so that the reference's wrapper and pipeline run
    unchanged on top of the sequence-parallel forward: same call signature as ``CausalWanModel.forward`` with a
    KV cache (wan/modules/causal_model.py:1880-1894), attributes looked up on the wrapped model.  The per-layer
    cache dicts the pipeline hands in hold THIS rank's heads ([B, tokens, H/P, 128], see
    ``head_sharded_kv_cache``); they are adopted once per video (the pipeline resets a cache by putting new
    index tensors into the dict) and their device-side indices are kept up to date."""

    def __init__(self, net, sp: SequenceParallelCausalWan):
        super().__init__()
        self.net = net
        self._sp = sp
        self._adopted = {}

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("net"), name)

    def __setattr__(self, name, value):
        if name in ("num_frame_per_block", "independent_first_frame", "local_attn_size"):
            setattr(self.net, name, value)                     # the pipeline configures the model this way
        else:
            super().__setattr__(name, value)

    def forward(self, x, t=None, context=None, seq_len=None, kv_cache=None, crossattn_cache=None, current_start=0,
                cache_start=None, **unused):
        if kv_cache is None:
            raise NotImplementedError("the sequence-parallel forward is the KV-cache rollout path")
        caches = []
        for i, d in enumerate(kv_cache):
            c = self._adopted.get(i)
            if c is None or c.stale(d):
                c = KVCache.from_reference(d)
                self._adopted[i] = c
            caches.append(c)
        return self._sp.forward(x, t, context, caches, crossattn_cache, int(current_start))


def head_sharded_kv_cache(model, batch: int, cache_tokens: int, world: int, device, dtype=torch.bfloat16) -> List[dict]:
    """Per-layer cache dicts in the pipeline's layout (pipeline/causal_inference.py:300-306) but with this
    rank's H/P heads only."""
    hd = model.dim // model.num_heads
    hp = model.num_heads // world
    return [{"k": torch.zeros(batch, cache_tokens, hp, hd, dtype=dtype, device=device),
             "v": torch.zeros(batch, cache_tokens, hp, hd, dtype=dtype, device=device),
             "global_end_index": torch.tensor([0], dtype=torch.long, device=device),
             "local_end_index": torch.tensor([0], dtype=torch.long, device=device)} for _ in range(model.num_layers)]

"""Host side of one causal self-attention layer on the KV-cache rollout path.

Mirrors the cache branch of ``CausalWanSelfAttention.forward`` (wan/modules/causal_model.py:900-1103)
between the q/k/v projections and the output projection: cache bookkeeping (rolling eviction with
sink frames), RMSNorm + RoPE + cache write, dispatch to dense attention (dense-init chunk, or Monarch
disabled) or Monarch attention, and the update of the cache's end indices.

Differences from the reference, none of them visible in the results:
* the end indices live in Python ints beside the cache tensors, so a layer call never reads a device
  scalar back (the reference does two to four ``.item()`` round trips per layer, causal_model.py:900-940);
  the device tensors ``global_end_index`` / ``local_end_index`` of a reference cache dict are still
  updated when such a dict is adopted with ``KVCache.from_reference``;
* normalisation, rotation and the cache write are one kernel (`ops.norm_rope_cache_write`);
* the sliding window's eviction shift (causal_model.py:912-926) runs inside the cache-write kernel when the
  moved tokens end where the new ones start (a fresh chunk into a full window), else as in-place copies;
* the new keys / values are written before attention in both branches, as the Monarch branch of the
  reference does (monarch_attn.py:1230-1231); its dense branch writes them at the same place
  (causal_model.py:961-962).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import ops


@dataclass
class CacheStep:
    """Integer plan of one layer call (all token counts)."""
    roll: Optional[Tuple[int, int, int]]   # (dst_start, src_start, count) shifted left before the write, or None
    cache_start: int                       # first cache token attention may see
    local_start: int                       # slot of the new tokens, relative to cache_start
    local_end: int
    store_global_end: int                  # values of the end indices after the call
    store_local_end: int


def plan_cache_step(current_start: int, num_new: int, global_end: int, local_end: int, cache_size: int,
                    max_attention_size: int, local_attn_size: int = -1, sink_tokens: int = 0) -> CacheStep:
    """The index arithmetic of causal_model.py:907-938 and 1102-1103, exactly.

    When a sliding window is in use (``local_attn_size != -1``), the call moves past everything written
    so far (``current_end > global_end``) and the new tokens do not fit (``num_new + local_end >
    cache_size``), the oldest tokens after the sink are evicted by shifting the rest left."""
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
    return CacheStep(roll, cache_start, new_local_start - cache_start, new_local_end - cache_start, current_end,
                     new_local_end - cache_start)


class KVCache:
    """One layer's cache: ``k``, ``v`` [B, cache_tokens, H, 128] bf16 plus the two end indices as ints."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor, global_end: int = 0, local_end: int = 0, ref_dict=None):
        if k.shape != v.shape or k.dim() != 4:
            raise ValueError("k and v must be [B, tokens, H, D] tensors of one shape")
        self.k, self.v = k, v
        self.global_end, self.local_end = int(global_end), int(local_end)
        self._ref = ref_dict
        # the pipeline resets a cache by putting NEW index tensors into the dict
        # (pipeline/causal_inference.py:133-138): remember which one was read
        self._ref_index = ref_dict["global_end_index"] if ref_dict is not None else None

    def stale(self, kv_cache: dict) -> bool:
        """True when ``kv_cache`` no longer is the dict state this object was read from."""
        return self.k is not kv_cache["k"] or self._ref_index is not kv_cache["global_end_index"]

    @classmethod
    def allocate(cls, batch: int, cache_tokens: int, heads: int, device, dtype=torch.bfloat16) -> "KVCache":
        """Same shape as the pipeline's per-layer entry (pipeline/causal_inference.py:300-306)."""
        z = lambda: torch.zeros(batch, cache_tokens, heads, 128, dtype=dtype, device=device)
        return cls(z(), z())

    @classmethod
    def from_reference(cls, kv_cache: dict) -> "KVCache":
        """Adopts a reference cache dict {"k", "v", "global_end_index", "local_end_index"}: the tensors are
        shared, the indices are read ONCE here and kept on the host from then on."""
        return cls(kv_cache["k"], kv_cache["v"], int(kv_cache["global_end_index"].item()),
                   int(kv_cache["local_end_index"].item()), ref_dict=kv_cache)

    def reset(self) -> None:
        self.global_end = self.local_end = 0
        if self._ref is not None:
            self._ref["global_end_index"].fill_(0)
            self._ref["local_end_index"].fill_(0)

    def _store(self, step: CacheStep) -> None:
        self.global_end, self.local_end = step.store_global_end, step.store_local_end
        if self._ref is not None:                      # asynchronous fills, no read-back
            self._ref["global_end_index"].fill_(step.store_global_end)
            self._ref["local_end_index"].fill_(step.store_local_end)

    def _roll(self, roll) -> None:
        """Shift ``count`` tokens left from ``src`` to ``dst`` (the eviction of causal_model.py:917-926).  The
        ranges overlap, so the reference copies through a temporary; here the shift is done in place, in
        stream order, in pieces no longer than the shift distance (a piece's source is then disjoint from its
        destination, and a later piece only overwrites tokens an earlier piece has already read)."""
        dst, src, count = roll
        if count <= 0 or src == dst:
            return
        step = src - dst
        for t in (self.k, self.v):
            for off in range(0, count, step):
                n = min(step, count - off)
                t[:, dst + off:dst + off + n].copy_(t[:, src + off:src + off + n])


@dataclass
class LayerConfig:
    """Knobs of CausalWanSelfAttention that the cache branch reads (causal_model.py:735-775)."""
    use_framewise: bool = True            # f_tied = 1, else 3
    h_reduce: int = 1
    w_reduce: int = 1
    num_iters: int = 1
    disable_monarch: bool = False         # "regular" configuration: dense attention for every chunk
    use_dense_init: bool = False          # dense attention while the cache view is a single chunk
    local_attn_size: int = -1             # frames; -1 = no sliding window
    sink_size: int = 0                    # frames kept at the start of the cache
    max_attention_size: int = 32760       # tokens
    eps: float = 1e-6


def self_attention_kv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cache: KVCache, current_start: int,
                      grid: Tuple[int, int, int], cfg: LayerConfig, freqs: Optional[torch.Tensor] = None,
                      norm_q_weight: Optional[torch.Tensor] = None, norm_k_weight: Optional[torch.Tensor] = None,
                      sm_scale: Optional[float] = None) -> torch.Tensor:
    """q, k, v: the projections of the new chunk, [B, n, H, 128] bf16, before rotation (and before
    norm_q / norm_k when the two weights are given).  ``grid`` = (frames, height, width) of the chunk
    in tokens.  Updates ``cache`` in place and returns the attention output [B, n, H, 128], the
    tensor the reference flattens and feeds to ``self.o`` (causal_model.py:1105-1107)."""
    frames, gh, gw = (int(x) for x in grid)
    B, n, H, D = q.shape
    frame_tokens = gh * gw
    if n != frames * frame_tokens:
        raise ValueError("the chunk does not match its grid")
    start_frame = current_start // frame_tokens
    step = plan_cache_step(current_start, n, cache.global_end, cache.local_end, cache.k.shape[1],
                           cfg.max_attention_size, cfg.local_attn_size, cfg.sink_size * frame_tokens)
    roll = None
    if step.roll is not None:
        dst, src, count = step.roll
        if count > 0 and dst + count == step.cache_start + step.local_start and src - dst <= n:
            # the usual case (a fresh chunk evicts from a full window): the moved tokens end where the new
            # ones start, so the shift rides inside the cache-write kernel; positions relative to the view
            roll = (dst - step.cache_start, src - dst)
        else:
            cache._roll(step.roll)
    curr_k = cache.k[:, step.cache_start:step.cache_start + step.local_end]
    curr_v = cache.v[:, step.cache_start:step.cache_start + step.local_end]
    is_init = cfg.use_dense_init and curr_k.shape[1] == 3 * frame_tokens
    dense = cfg.disable_monarch or is_init
    f_tied = 1 if cfg.use_framewise else 3
    q_rot = ops.norm_rope_cache_write(q, k, v, curr_k, curr_v, step.local_start, start_frame, f_tied, cfg.h_reduce,
                                      cfg.w_reduce, gh, gw, freqs=freqs, norm_q_weight=norm_q_weight,
                                      norm_k_weight=norm_k_weight, eps=cfg.eps, monarch_order=not dense, roll=roll)
    if dense:
        out = ops.dense_attention_on_cache(q_rot, curr_k, curr_v, sm_scale)
    else:
        out = ops.monarch_attention_on_cache(q_rot, curr_k, curr_v, f_tied, cfg.h_reduce, cfg.w_reduce, gh, gw,
                                             sm_scale, cfg.num_iters)
    cache._store(step)
    return out

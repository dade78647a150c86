"""Drop-in installation into a checkout of the reference project.

``install_into_reference()`` registers this package's operators under the module names the
reference's model code imports them from, so ``wan/modules/causal_model.py`` and
``pipeline/causal_inference.py`` run unchanged:

* ``from .monarch_attn import monarch_attn, monarch_attn_with_kv_cache``  (causal_model.py:25)
* ``from wan.modules.attention import attention``                         (causal_model.py:1)

Call it before importing ``wan.modules.causal_model``.

``patch_self_attention_forward(cls)`` goes one step further (opt-in): it replaces the KV-cache branch of
``CausalWanSelfAttention.forward`` (causal_model.py:776-1108) by this package's layer path — q/k/v
projections, then ONE kernel for norm_q / norm_k + RoPE + cache write, then attention, then the output
projection — with the cache's end indices kept on the host, so that a layer call no longer reads device
scalars back.  Calls it cannot serve (no cache, top-k / SVG / radial variants) go to the original forward.
"""
from __future__ import annotations

import sys
import types


def install_into_reference(replace_dense: bool = True, replace_rope: bool = False) -> None:
    from . import ops

    pkg_names = ["wan", "wan.modules"]
    for name in pkg_names:
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__path__ = []          # namespace stub: the real package __init__ pulls heavy dependencies
            sys.modules[name] = mod

    m = types.ModuleType("wan.modules.monarch_attn")
    m.monarch_attn = ops.monarch_attn
    m.monarch_attn_with_kv_cache = ops.monarch_attn_with_kv_cache
    m.__all__ = ["monarch_attn", "monarch_attn_with_kv_cache"]
    sys.modules["wan.modules.monarch_attn"] = m
    setattr(sys.modules["wan.modules"], "monarch_attn", m)

    if replace_dense:
        a = types.ModuleType("wan.modules.attention")
        a.attention = ops.attention
        a.flash_attention = ops.flash_attention
        a.__all__ = ["flash_attention", "attention"]
        sys.modules["wan.modules.attention"] = a
        setattr(sys.modules["wan.modules"], "attention", a)

    if replace_rope and "wan.modules.causal_model" in sys.modules:
        sys.modules["wan.modules.causal_model"].causal_rope_apply = ops.causal_rope_apply


def patch_self_attention_forward(cls) -> None:
    """Replace ``cls.forward`` (cls = the reference's CausalWanSelfAttention, or any module with the same
    attributes: q, k, v, o, norm_q, norm_k, num_heads, head_dim, eps, use_framewise, h_reduce, w_reduce,
    num_iters, disable_monarch, use_dense_init, local_attn_size, sink_size, max_attention_size)."""
    import torch
    from . import layer

    original = cls.forward

    def forward(self, x, seq_lens, grid_sizes, freqs, block_mask, kv_cache=None, current_start=0, cache_start=None,
                timestep=None, **kw):
        special = getattr(self, "topk", None) is not None or getattr(self, "use_svg", False) or \
            getattr(self, "use_radial_attn", False)
        wq = getattr(self.norm_q, "weight", None)
        wk = getattr(self.norm_k, "weight", None)
        # The fused kernel multiplies by bf16 norm weights, as the bf16 module does; a module kept in another
        # precision (fp32 norm weights promote the reference's product to fp32) stays on the original forward.
        odd_norm = (wq is None) != (wk is None) or any(w is not None and w.dtype != torch.bfloat16 for w in (wq, wk))
        if kv_cache is None or special or odd_norm or x.dtype != torch.bfloat16:
            return original(self, x, seq_lens, grid_sizes, freqs, block_mask, kv_cache=kv_cache,
                            current_start=current_start, cache_start=cache_start, timestep=timestep, **kw)
        b, s, n, d = *x.shape[:2], self.num_heads, self.head_dim
        q = self.q(x).view(b, s, n, d)
        k = self.k(x).view(b, s, n, d)
        v = self.v(x).view(b, s, n, d)
        state = kv_cache.get("_sfm_state")
        if state is None or state.stale(kv_cache):
            state = layer.KVCache.from_reference(kv_cache)         # reads the two indices once
            kv_cache["_sfm_state"] = state
        if grid_sizes.device.type == "cpu":                        # the model builds it on the host: free to read
            grid = (int(s), tuple(int(t) for t in grid_sizes[0].tolist()))
        else:
            # a device tensor costs a read-back: do it once per tensor, not per call (same token count with
            # another (rows, columns) split arrives in another tensor)
            grid = getattr(self, "_sfm_grid", None)
            key = (int(s), grid_sizes.data_ptr(), grid_sizes._version)
            if grid is None or grid[2] != key:
                grid = (int(s), tuple(int(t) for t in grid_sizes[0].tolist()), key)
                self._sfm_grid = grid
        cfg = layer.LayerConfig(use_framewise=bool(self.use_framewise), h_reduce=int(self.h_reduce),
                                w_reduce=int(self.w_reduce), num_iters=int(self.num_iters),
                                disable_monarch=bool(self.disable_monarch), use_dense_init=bool(self.use_dense_init),
                                local_attn_size=int(self.local_attn_size), sink_size=int(self.sink_size),
                                max_attention_size=int(self.max_attention_size), eps=float(self.eps))
        out = layer.self_attention_kv(q, k, v, state, int(current_start), grid[1], cfg, freqs=freqs,
                                      norm_q_weight=wq, norm_k_weight=wk)
        return self.o(out.flatten(2))

    cls.forward = forward
    cls._sfm_original_forward = original

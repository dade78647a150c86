"""B200-native Monarch self-attention for the causal Wan DiT's KV-cache rollout.

Host-side mirror of the reference's attention interface
(wan/modules/monarch_attn.py, wan/modules/attention.py, causal_rope_apply in
wan/modules/causal_model.py) on top of libsfmonarch.so, hand-written CUDA for sm_100a.
"""
from .ops import (attention, causal_rope_apply, flash_attention, full_attention_with_kv_cache,
                  monarch_attn, monarch_attn_with_kv_cache, monarch_attn_with_kv_cache_backward,
                  rope_monarch_attn_with_kv_cache,
                  norm_rope_cache_write, build_maps, workspace_bytes)
from .install import install_into_reference
from .layer import KVCache, LayerConfig, plan_cache_step, self_attention_kv

__all__ = [
    "attention", "flash_attention", "causal_rope_apply", "full_attention_with_kv_cache",
    "monarch_attn", "monarch_attn_with_kv_cache", "monarch_attn_with_kv_cache_backward",
    "rope_monarch_attn_with_kv_cache",
    "norm_rope_cache_write", "build_maps", "workspace_bytes", "install_into_reference",
    "KVCache", "LayerConfig", "plan_cache_step", "self_attention_kv",
]

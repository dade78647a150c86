"""Drop-in installation into a checkout of the reference project.

``install_into_reference()`` registers this package's operators under the module names the
reference's model code imports them from, so ``wan/modules/causal_model.py`` and
``pipeline/causal_inference.py`` run unchanged:

* ``from .monarch_attn import monarch_attn, monarch_attn_with_kv_cache``  (causal_model.py:25)
* ``from wan.modules.attention import attention``                         (causal_model.py:1)

Call it before importing ``wan.modules.causal_model``.
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

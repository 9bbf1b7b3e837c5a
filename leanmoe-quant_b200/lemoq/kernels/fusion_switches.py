"""The seven decode-path switches: code defaults, ``LEMOQ_*`` environment overrides.

Mirrors src/lemoq/kernels/fusion_switches.py:40-76 of the reference: an env value of
``"1"`` turns a switch on, any other set value turns it off, unset means the default.
Every default is True (the canonical cell).
"""

from __future__ import annotations

import os
from typing import Any

ENV_VARS: dict[str, str] = {
    "fused_rope": "LEMOQ_FUSED_ROPE",
    "fused_route": "LEMOQ_FUSED_ROUTE",
    "skip_mask_fill": "LEMOQ_SKIP_MASK_FILL",
    "packed_qkv": "LEMOQ_PACKED_QKV",
    "kv_direct_write": "LEMOQ_KV_DIRECT_WRITE",
    "lm_head_w8": "LEMOQ_LMHEAD_W8",
    "kv_int8": "LEMOQ_KV_INT8",
}

FUSION_DEFAULTS: dict[str, bool] = {name: True for name in ENV_VARS}


def fusion_enabled(name: str, env: dict[str, str] | None = None) -> bool:
    """Effective state of one switch (env override first, then the code default)."""
    if name not in ENV_VARS:
        raise KeyError("未知融合开关 %r (unknown fusion switch); declared: %s" % (name, sorted(ENV_VARS)))
    raw = (os.environ if env is None else env).get(ENV_VARS[name])
    return FUSION_DEFAULTS[name] if raw is None else raw == "1"


def fusion_states(env: dict[str, str] | None = None) -> dict[str, bool]:
    return {name: fusion_enabled(name, env) for name in ENV_VARS}


def fusion_payload_fields(env: dict[str, str] | None = None) -> dict[str, Any]:
    """One key per switch for a result's ``config`` block."""
    return fusion_states(env)

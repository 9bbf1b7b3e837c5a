"""The seven switches of the decode path (interface of the reference's src/lemoq/kernels/fusion_switches.py:40-76).

One table: switch name, environment variable, default.  The environment wins over the default: the value ``"1"``
switches on, any other value that is set switches off.  Every default is on (the canonical cell).
"""

from __future__ import annotations

import os
from typing import Any, Mapping, NamedTuple


class _Switch(NamedTuple):
    name: str
    env: str
    default: bool


_TABLE = tuple(_Switch(name, "LEMOQ_" + suffix, True) for name, suffix in (
    ("fused_rope", "FUSED_ROPE"),
    ("fused_route", "FUSED_ROUTE"),
    ("skip_mask_fill", "SKIP_MASK_FILL"),
    ("packed_qkv", "PACKED_QKV"),
    ("kv_direct_write", "KV_DIRECT_WRITE"),
    ("lm_head_w8", "LMHEAD_W8"),
    ("kv_int8", "KV_INT8"),
))
_BY_NAME = {s.name: s for s in _TABLE}

ENV_VARS: dict[str, str] = {s.name: s.env for s in _TABLE}
FUSION_DEFAULTS: dict[str, bool] = {s.name: s.default for s in _TABLE}


def fusion_enabled(name: str, env: Mapping[str, str] | None = None) -> bool:
    """Is the switch on?  ``env`` replaces the process environment (tests)."""
    switch = _BY_NAME.get(name)
    if switch is None:
        raise KeyError("未知融合开关 %r (unknown fusion switch); declared: %s" % (name, sorted(_BY_NAME)))
    value = (os.environ if env is None else env).get(switch.env)
    return FUSION_DEFAULTS[name] if value is None else value == "1"


def fusion_states(env: Mapping[str, str] | None = None) -> dict[str, bool]:
    return {s.name: fusion_enabled(s.name, env) for s in _TABLE}


def fusion_payload_fields(env: Mapping[str, str] | None = None) -> dict[str, Any]:
    """The switch states as fields of a result's ``config`` block."""
    return dict(fusion_states(env))

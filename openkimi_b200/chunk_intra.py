"""Guarded-diagonal contract of the KDA backward.

The reference's backend selector imports ``fla.ops.kda.chunk_intra`` and refuses the fast
path unless that module carries the three attributes below with these exact values
(k3mini/backends.py:17-19, 68-109; produced for the reference's fork by
experiments/kda_sm90/patch_fla_guarded_intra.py:229-242).  This module is the object a
maintainer hands to ``_validated_kda_backend_name`` for the B200 kernels.

``_OPENKIMI_GUARD_MAX_LOG2_SPAN`` is read at every backward call, so validators can set it
to ``-1.0`` to force the exact pairwise evaluation of every diagonal tile without
recompiling (experiments/kda_sm90/validate_fla_guarded_integration.py:257-267).
"""

from __future__ import annotations

import math
import os

OPENKIMI_KDA_GUARDED_DIAGONAL_VERSION = 1
_OPENKIMI_GUARD_DOT_PRECISION = os.environ.get("K3MINI_KDA_GUARD_DOT_PRECISION", "tf32x3")
_OPENKIMI_GUARD_MAX_LOG2_SPAN = float(os.environ.get("K3MINI_KDA_GUARD_SPAN", "232.0"))

_ALLOWED_PRECISIONS = {"tf32", "tf32x3", "ieee"}
if _OPENKIMI_GUARD_DOT_PRECISION not in _ALLOWED_PRECISIONS:
    raise ValueError(f"K3MINI_KDA_GUARD_DOT_PRECISION must be one of {sorted(_ALLOWED_PRECISIONS)}")
if not math.isfinite(_OPENKIMI_GUARD_MAX_LOG2_SPAN):
    raise ValueError("K3MINI_KDA_GUARD_SPAN must be finite")


def current_guard_span() -> float:
    """The span the next backward call will use (negative = exact path everywhere)."""
    span = float(_OPENKIMI_GUARD_MAX_LOG2_SPAN)
    if not math.isfinite(span):
        raise RuntimeError("OpenKimi guarded KDA has an invalid runtime span")
    if span > 232.0:
        raise RuntimeError(f"K3MINI_KDA_GUARD_SPAN={span:g} exceeds the validated maximum 232")
    return span

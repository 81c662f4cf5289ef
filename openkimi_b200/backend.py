"""Backend report for the KDA path, mirroring the part of ``resolve_backend`` that concerns
it (k3mini/backends.py:155-243): the fast path is selected only on a capable GPU and only
if the guarded-diagonal contract validates (k3mini/backends.py:68-109)."""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib, chunk_intra

PATCH_VERSION = 1          # k3mini/backends.py:17
MAX_GUARD_SPAN = 232.0     # k3mini/backends.py:18
DOT_PRECISION = "tf32x3"   # k3mini/backends.py:19


@dataclass(frozen=True)
class KdaBackendStatus:
    selected: str
    kda: str
    short_conv: str

    def as_dict(self):
        return {"selected": self.selected, "kda": self.kda, "short_conv": self.short_conv}


def validated_kda_backend_name(module=chunk_intra) -> str:
    """Same checks, same messages and same return format as
    ``_validated_kda_backend_name`` (k3mini/backends.py:68-109), with this library's op name."""
    version = getattr(module, "OPENKIMI_KDA_GUARDED_DIAGONAL_VERSION", None)
    span = getattr(module, "_OPENKIMI_GUARD_MAX_LOG2_SPAN", None)
    precision = getattr(module, "_OPENKIMI_GUARD_DOT_PRECISION", None)
    if version != PATCH_VERSION:
        raise RuntimeError(f"kernel_backend=b200 requires the versioned OpenKimi guarded KDA patch v{PATCH_VERSION}")
    if not isinstance(span, float) or not math.isfinite(span):
        raise RuntimeError("OpenKimi guarded KDA has an invalid runtime span")
    if span > MAX_GUARD_SPAN:
        raise RuntimeError(f"K3MINI_KDA_GUARD_SPAN={span:g} exceeds the validated maximum {MAX_GUARD_SPAN:g}")
    if precision != DOT_PRECISION:
        raise RuntimeError(f"K3MINI_KDA_GUARD_DOT_PRECISION={precision!r} is not validated; use {DOT_PRECISION!r}")
    return f"openkimi_b200.chunk_kda(openkimi_guarded_diagonal_v{version},{precision},span<={span:g})"


def b200_capable() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 10


def resolve_kda_backend() -> KdaBackendStatus:
    """Fail closed: no capable GPU, a missing library or a broken contract is an error, never
    a silent fallback."""
    if not b200_capable():
        raise RuntimeError("kernel_backend=b200 requires an NVIDIA sm_100 GPU")
    lib = _lib.load()
    if lib.kda_guard_version() != PATCH_VERSION or abs(lib.kda_guard_max_span() - MAX_GUARD_SPAN) > 0 \
            or lib.kda_guard_dot_precision().decode() != DOT_PRECISION:
        raise RuntimeError("libkda_b200.so does not implement the guarded KDA contract v1")
    return KdaBackendStatus(selected="b200", kda=validated_kda_backend_name(),
                            short_conv="openkimi_b200.ShortConvolution")

"""B200-native Kimi Delta Attention: ``chunk_kda`` and its sublayer companions, as a drop-in
for the fast path the reference selects in k3mini/backends.py and calls at
k3mini/model.py:197-216."""

from . import chunk_intra
from .backend import KdaBackendStatus, resolve_kda_backend, validated_kda_backend_name
from .modules import FusedRMSNormGated, KimiDeltaAttention, ShortConvolution
from .ops import check_device_status, chunk_kda, fused_recurrent_kda, recurrent_kda_step
from .spans import gate_tile_spans, guarded_diagonal_backward

__all__ = ["chunk_kda", "check_device_status", "recurrent_kda_step", "fused_recurrent_kda", "chunk_intra", "ShortConvolution", "FusedRMSNormGated", "KimiDeltaAttention",
           "resolve_kda_backend", "validated_kda_backend_name", "KdaBackendStatus", "gate_tile_spans",
           "guarded_diagonal_backward"]

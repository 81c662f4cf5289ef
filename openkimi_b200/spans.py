"""Gate-span statistic and the guarded diagonal tile as callable utilities on the GPU.

``gate_tile_spans`` has the interface of scripts/profile_kda_gate_spans.py:21-56 of the reference
(log2 span of every [16 rows x 32 channels] tile of the within-chunk cumulative gate) and runs the
CUDA kernel ``kda_gate_tile_spans``.  ``guarded_diagonal_backward`` runs the CUDA tile kernel behind
the interface of experiments/kda_sm90/guarded_diagonal_oracle.py::guarded_diagonal_backward
(midpoint policy)."""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import torch

from . import _lib

_DT = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16}


def gate_tile_spans(raw_decay: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor) -> torch.Tensor:
    """raw_decay [B, T, H, d] (CUDA, FP32 or BF16), a_log [H], dt_bias [H, d] -> FP32 spans, one per
    tile, flattened in the order [B][T/64][4][H][d/32]."""
    if raw_decay.dim() != 4:
        raise ValueError("raw_decay must have shape [B, T, H, d]")
    batch, seqlen, heads, dim = raw_decay.shape
    if seqlen % 64:
        raise ValueError("sequence length must be divisible by the chunk size")
    if dim % 32:
        raise ValueError("head dimension must be a multiple of the 32-channel tile")
    if not raw_decay.is_cuda:
        raise RuntimeError("gate_tile_spans runs only on a CUDA device; there is no CPU fallback")
    if a_log.numel() != heads or dt_bias.numel() != heads * dim:
        raise ValueError("a_log must have H entries and dt_bias H*d entries")
    raw = raw_decay.contiguous() if raw_decay.dtype in _DT else raw_decay.float().contiguous()
    a = a_log.to(device=raw.device, dtype=torch.float32).contiguous()
    b = dt_bias.to(device=raw.device, dtype=torch.float32).contiguous()
    out = torch.empty(batch * (seqlen // 64) * 4 * heads * (dim // 32), dtype=torch.float32, device=raw.device)
    with torch.cuda.device(raw.device):
        rc = _lib.load().kda_gate_tile_spans(raw.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, seqlen,
                                             heads, dim, _DT[raw.dtype],
                                             C.c_void_p(torch.cuda.current_stream(raw.device).cuda_stream))
    _lib.check(rc, "kda_gate_tile_spans")
    return out


@dataclass(frozen=True)
class GuardedDiagonalResult:
    dq: torch.Tensor
    dk: torch.Tensor
    dkt: torch.Tensor
    guard_hits: torch.Tensor


def guarded_diagonal_backward(gate, q, k, beta, da_qk, da_kk, *, max_log2_span: float) -> GuardedDiagonalResult:
    """[blocks, 16, 32] tiles on the GPU; a negative ``max_log2_span`` forces the exact path."""
    if gate.ndim != 3 or gate.shape[1:] != (16, 32):
        raise ValueError("gate must have shape [blocks, 16, 32]")
    if q.shape != gate.shape or k.shape != gate.shape:
        raise ValueError("q and k must have the same shape as gate")
    if beta.shape != gate.shape[:2] or da_qk.shape != (gate.shape[0], 16, 16) or da_kk.shape != da_qk.shape:
        raise ValueError("beta must be [blocks,16] and the dA tensors [blocks,16,16]")
    if not gate.is_cuda:
        raise RuntimeError("guarded_diagonal_backward runs only on a CUDA device; there is no CPU fallback")
    if not (max_log2_span < 0 or (math.isfinite(max_log2_span) and max_log2_span < 252.0)):
        raise ValueError("max_log2_span must be negative (exact) or finite and below 252")
    ts = [t.float().contiguous() for t in (gate, q, k, beta, da_qk, da_kk)]
    n = gate.shape[0]
    dq, dk, dkt = (torch.empty_like(ts[0]) for _ in range(3))
    hits = torch.empty(n, dtype=torch.int32, device=gate.device)
    with torch.cuda.device(gate.device):
        rc = _lib.load().kda_guarded_diagonal_tiles(*(C.c_void_p(t.data_ptr()) for t in ts), C.c_void_p(dq.data_ptr()),
                                                    C.c_void_p(dk.data_ptr()), C.c_void_p(dkt.data_ptr()),
                                                    C.c_void_p(hits.data_ptr()), n, float(max_log2_span),
                                                    C.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, "kda_guarded_diagonal_tiles")
    return GuardedDiagonalResult(dq, dk, dkt, hits.bool())

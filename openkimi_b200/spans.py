"""Gate-span statistic and the guarded diagonal tile as callable utilities.

``gate_tile_spans`` mirrors scripts/profile_kda_gate_spans.py:21-56 of the reference (log2
span of every [16 rows x 32 channels] tile of the within-chunk cumulative gate); it is plain
tensor arithmetic and runs wherever its inputs live.  ``guarded_diagonal_backward`` runs the
CUDA tile kernel behind the interface of
experiments/kda_sm90/guarded_diagonal_oracle.py::guarded_diagonal_backward (midpoint policy)."""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib

CHUNK_SIZE, BLOCK_SIZE, CHANNEL_TILE = 64, 16, 32
RCP_LN2 = 1.0 / math.log(2.0)


def gate_tile_spans(raw_decay: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor) -> torch.Tensor:
    batch, seqlen, heads, dim = raw_decay.shape
    if seqlen % CHUNK_SIZE:
        raise ValueError("sequence length must be divisible by the chunk size")
    if dim % CHANNEL_TILE:
        raise ValueError("head dimension must be a multiple of the 32-channel tile")
    steps = (-a_log.float().exp().view(1, 1, heads, 1)
             * F.softplus(raw_decay.float() + dt_bias.float().view(1, 1, heads, dim)) * RCP_LN2)
    cum = steps.view(batch, seqlen // CHUNK_SIZE, CHUNK_SIZE, heads, dim).cumsum(dim=2)
    tiles = cum.view(batch, seqlen // CHUNK_SIZE, CHUNK_SIZE // BLOCK_SIZE, BLOCK_SIZE, heads, dim // CHANNEL_TILE,
                     CHANNEL_TILE)
    return (tiles[:, :, :, :1] - tiles).amax(dim=(3, 6)).flatten()


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

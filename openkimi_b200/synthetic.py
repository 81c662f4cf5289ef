"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations: q, k, v ~ N(0,1); gate input x ~ N(x_mean, 1); A_log ~ U(ln a_lo, ln a_hi)
per head; beta logits ~ N(beta_mean, 1); upstream gradient do ~ N(0,1); dt_bias = 0.
Generated on the CPU in FP32 from one generator and then cast, so a CPU check and the GPU
see the same bits.  (Stands in for real activations: the reference's kernel benchmarks are
synthetic too, scripts/benchmark_kda_backends.py:30-59.)"""

from __future__ import annotations

import math

import torch


def make_inputs(batch, time, heads, dim, *, seed=0, dtype=torch.float32, x_mean=0.0, a_lo=1.0, a_hi=16.0,
                beta_mean=0.0):
    gen = torch.Generator().manual_seed(seed)
    shape = (batch, time, heads, dim)
    q = torch.randn(shape, generator=gen)
    k = torch.randn(shape, generator=gen)
    v = torch.randn(shape, generator=gen)
    x = torch.randn(shape, generator=gen) + x_mean
    bl = torch.randn(shape[:-1], generator=gen) + beta_mean
    a_log = torch.empty(heads).uniform_(math.log(a_lo), math.log(a_hi), generator=gen)
    do = torch.randn(shape, generator=gen)
    return dict(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype), g=x.to(dtype), beta=bl.to(dtype), a_log=a_log,
                dt_bias=torch.zeros(heads * dim), do=do.to(dtype))


def random_cu_seqlens(total, n_docs, seed=0):
    """n_docs document lengths from sorted distinct random cut points, summing to total."""
    gen = torch.Generator().manual_seed(seed)
    cuts = torch.randperm(total - 1, generator=gen)[: n_docs - 1] + 1
    return torch.cat([torch.zeros(1, dtype=torch.long), cuts.sort().values, torch.tensor([total])]).to(torch.long)

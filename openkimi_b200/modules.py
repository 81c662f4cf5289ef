"""Companion modules of the KDA op inside the reference's ``KimiDeltaAttention`` sublayer
(k3mini/model.py:132-227): the causal depthwise short convolution, the gated headwise
RMSNorm, and the sublayer itself wired to the B200 kernels.  Parameter names and shapes
match the reference's modules so ``state_dict`` keys are interchangeable."""

from __future__ import annotations

import ctypes as C
import math

import torch
import torch.nn as nn

from . import _lib
from .ops import chunk_kda, _DTYPES, _require_cuda


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


class _ShortConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cu_seqlens):
        _require_cuda(x)
        lib = _lib.load()
        x = x.contiguous()
        w = weight.float().contiguous()
        B, T, Cc = x.shape
        y = torch.empty_like(x)
        n = 0 if cu_seqlens is None else cu_seqlens.numel() - 1
        with torch.cuda.device(x.device):
            _lib.check(lib.kda_short_conv_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), B, T, Cc, w.shape[-1],
                                              _DTYPES[x.dtype], None if cu_seqlens is None else cu_seqlens.data_ptr(),
                                              n, _stream(x)), "kda_short_conv_fwd")
        ctx.save_for_backward(x, w, cu_seqlens)
        ctx.wdtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.load()
        x, w, cu_seqlens = ctx.saved_tensors
        dy = dy.contiguous()
        B, T, Cc = x.shape
        ks = w.shape[-1]
        n_partial = 128
        dx = torch.empty_like(x)
        dw = torch.empty(Cc, 1, ks, dtype=torch.float32, device=x.device)
        part = torch.empty(n_partial, Cc, ks, dtype=torch.float32, device=x.device)
        n = 0 if cu_seqlens is None else cu_seqlens.numel() - 1
        with torch.cuda.device(x.device):
            _lib.check(lib.kda_short_conv_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                              part.data_ptr(), n_partial, B, T, Cc, ks, _DTYPES[x.dtype],
                                              None if cu_seqlens is None else cu_seqlens.data_ptr(), n, _stream(x)),
                       "kda_short_conv_bwd")
        return dx, dw.to(ctx.wdtype), None


def short_convolution(x, weight, cu_seqlens=None):
    """Causal depthwise convolution + SiLU over x [B, T, C] with filter [C, 1, ksize]."""
    return _ShortConvFn.apply(x, weight, cu_seqlens)


class ShortConvolution(nn.Module):
    """Causal depthwise conv1d (kernel <= 4) + SiLU over [B, T, hidden]; the interface the
    reference uses from ``fla.modules.ShortConvolution`` (k3mini/model.py:147-155, 181-185):
    ``forward(x, cu_seqlens=None) -> (y, None)``; ``weight`` is ``[hidden, 1, kernel]`` as in
    the reference's ``CausalDepthwiseConv1d`` (k3mini/model.py:76-88)."""

    def __init__(self, hidden_size, kernel_size, bias=False, activation="silu"):
        super().__init__()
        if bias or activation != "silu" or not 1 <= kernel_size <= 4:
            raise ValueError("ShortConvolution supports bias=False, activation='silu', kernel_size <= 4")
        self.hidden_size, self.kernel_size = hidden_size, kernel_size
        self.weight = nn.Parameter(torch.empty(hidden_size, 1, kernel_size))
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x, cu_seqlens=None, **unused):
        if x.shape[-1] != self.hidden_size:
            raise ValueError(f"expected last dimension {self.hidden_size}, got {x.shape[-1]}")
        if cu_seqlens is not None:
            cu_seqlens = cu_seqlens.to(device=x.device, dtype=torch.int64).contiguous()
        return _ShortConvFn.apply(x, self.weight, cu_seqlens), None


class _NormGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, weight, eps):
        _require_cuda(x)
        lib = _lib.load()
        x, gate = x.contiguous(), gate.to(x.dtype).contiguous()
        w = weight.float().contiguous()
        dim = x.shape[-1]
        rows = x.numel() // dim
        y = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _lib.check(lib.kda_norm_gate_fwd(x.data_ptr(), gate.data_ptr(), w.data_ptr(), y.data_ptr(), None, rows, dim,
                                             eps, _DTYPES[x.dtype], _stream(x)), "kda_norm_gate_fwd")
        ctx.save_for_backward(x, gate, w)
        ctx.eps, ctx.wdtype = eps, weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.load()
        x, gate, w = ctx.saved_tensors
        dy = dy.contiguous()
        dim = x.shape[-1]
        rows = x.numel() // dim
        n_partial = 592
        dx, dgate = torch.empty_like(x), torch.empty_like(gate)
        dw = torch.empty(dim, dtype=torch.float32, device=x.device)
        part = torch.empty(n_partial, dim, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(lib.kda_norm_gate_bwd(x.data_ptr(), gate.data_ptr(), w.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                             dgate.data_ptr(), dw.data_ptr(), part.data_ptr(), n_partial, rows, dim,
                                             ctx.eps, _DTYPES[x.dtype], _stream(x)), "kda_norm_gate_bwd")
        return dx, dgate, dw.to(ctx.wdtype), None


class FusedRMSNormGated(nn.Module):
    """``rms_norm(x) * weight * sigmoid(gate)`` over the last axis (64 or 128 wide); the
    interface the reference uses from ``fla.modules.FusedRMSNormGated``
    (k3mini/model.py:171-175, 226) and the math of its ``HeadwiseRMSNormGate``
    (k3mini/model.py:91-98)."""

    def __init__(self, hidden_size, activation="sigmoid", eps=1e-6):
        super().__init__()
        if activation != "sigmoid":
            raise ValueError("FusedRMSNormGated supports activation='sigmoid'")
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x, g):
        return _NormGateFn.apply(x, g, self.weight, self.eps)


class _InputProjections(torch.autograd.Function):
    """The sublayer's four projections of x (q, k, v and the merged narrow one) as one autograd node.
    Forward: four library GEMMs, as ``F.linear`` would run them.  Backward: the input gradient is
    accumulated inside the GEMMs (``addmm_`` with beta = 1, FP32 accumulators) instead of four separate
    products and three read-modify-write additions over the [tokens, d_model] tensor, and the gradient
    of the narrow output is assembled from its three slices with one concatenation."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx, x, wq, wk, wv, wn, hd, nh):
        x2 = x.reshape(-1, x.shape[-1])
        q, k, v, n = (x2 @ w.t() for w in (wq, wk, wv, wn))
        ctx.save_for_backward(x2, wq, wk, wv, wn)
        ctx.split = (hd, nh, wn.shape[0])
        ctx.x_shape = tuple(x.shape)
        lead = x.shape[:-1]
        # the three slices of the narrow output leave as separate outputs (views of one buffer)
        return (q.view(*lead, -1), k.view(*lead, -1), v.view(*lead, -1), n[:, :hd].view(*lead, hd),
                n[:, hd:2 * hd].view(*lead, hd), n[:, 2 * hd:2 * hd + nh].contiguous().view(*lead, nh))

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, dq, dk, dv, dd, dg, db):
        x2, wq, wk, wv, wn = ctx.saved_tensors
        hd, nh, wide = ctx.split
        flat = lambda t: t.reshape(-1, t.shape[-1])
        dq, dk, dv = flat(dq), flat(dk), flat(dv)
        parts = [flat(dd), flat(dg), flat(db)]
        if wide > 2 * hd + nh:
            parts.append(dq.new_zeros(dq.shape[0], wide - 2 * hd - nh))
        dn = torch.cat(parts, dim=1)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = dq @ wq
            dx.addmm_(dk, wk)
            dx.addmm_(dv, wv)
            dx.addmm_(dn, wn)
            dx = dx.view(*ctx.x_shape)
        grads = [g.t() @ x2 if need else None for g, need in zip((dq, dk, dv, dn), ctx.needs_input_grad[1:5])]
        return (dx, *grads, None, None)


class KimiDeltaAttention(nn.Module):
    """The KDA sublayer of k3mini/model.py:132-227 on the B200 kernels: q/k/v projections,
    short conv + SiLU, decay and beta projections, ``chunk_kda`` with the fused L2 norm /
    gate / sigmoid prologue, gated RMSNorm and the output projection.  Constructor arguments
    replace the reference's ``ModelConfig`` fields (k3mini/config.py:56-59)."""

    def __init__(self, d_model, n_heads, head_dim=128, conv_kernel=4, rms_norm_eps=1e-6, disable_recompute=False,
                 fuse_short_conv=True):
        super().__init__()
        self.d_model, self.n_heads, self.head_dim = d_model, n_heads, head_dim
        self.disable_recompute = disable_recompute
        # True: the three short convolutions run inside the KDA forward's load stage (same bits)
        self.fuse_short_conv = fuse_short_conv
        proj = n_heads * head_dim
        self.q_proj = nn.Linear(d_model, proj, bias=False)
        self.k_proj = nn.Linear(d_model, proj, bias=False)
        self.v_proj = nn.Linear(d_model, proj, bias=False)
        self.q_conv = ShortConvolution(proj, conv_kernel)
        self.k_conv = ShortConvolution(proj, conv_kernel)
        self.v_conv = ShortConvolution(proj, conv_kernel)
        self.A_log = nn.Parameter(torch.log(torch.empty(n_heads).uniform_(1.0, 16.0)))
        self.f_a_proj = nn.Linear(d_model, head_dim, bias=False)
        self.f_b_proj = nn.Linear(head_dim, proj, bias=False)
        self.dt_bias = nn.Parameter(torch.zeros(n_heads, head_dim, dtype=torch.float32))
        self.beta_proj = nn.Linear(d_model, n_heads, bias=False)
        self.out_gate_a = nn.Linear(d_model, head_dim, bias=False)
        self.out_gate_b = nn.Linear(head_dim, proj, bias=False)
        self.out_norm_gate = FusedRMSNormGated(head_dim, activation="sigmoid", eps=rms_norm_eps)
        self.out_proj = nn.Linear(proj, d_model, bias=False)
        self.scale = head_dim ** -0.5

    def _heads(self, x):
        return x.view(*x.shape[:2], self.n_heads, self.head_dim)

    def forward(self, x, cu_seqlens=None):
        # The three narrow projections of x (decay rank, output-gate rank, beta) share one GEMM: x is
        # read once instead of three times.  Same parameters, same arithmetic per output column.  All four
        # projections of x form one autograd node (see _InputProjections).
        hd, nh = self.head_dim, self.n_heads
        pad = (-(2 * hd + nh)) % 8
        w_narrow = torch.cat([self.f_a_proj.weight, self.out_gate_a.weight, self.beta_proj.weight]
                             + ([self.beta_proj.weight.new_zeros(pad, self.d_model)] if pad else []), dim=0)
        q, k, v, decay_rank, gate_rank, beta_logits = _InputProjections.apply(
            x, self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, w_narrow, hd, nh)
        conv_w = None
        if self.fuse_short_conv:
            q, k, v = self._heads(q), self._heads(k), self._heads(v)
            conv_w = (self.q_conv.weight, self.k_conv.weight, self.v_conv.weight)
        else:
            q = self._heads(self.q_conv(q, cu_seqlens=cu_seqlens)[0])
            k = self._heads(self.k_conv(k, cu_seqlens=cu_seqlens)[0])
            v = self._heads(self.v_conv(v, cu_seqlens=cu_seqlens)[0])
        raw_decay = self._heads(self.f_b_proj(decay_rank))
        out, _ = chunk_kda(q=q, k=k, v=v, g=raw_decay, beta=beta_logits, A_log=self.A_log,
                           dt_bias=self.dt_bias.reshape(-1), scale=self.scale, use_qk_l2norm_in_kernel=True,
                           use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True, safe_gate=False,
                           output_final_state=False, state_v_first=True, cu_seqlens=cu_seqlens,
                           disable_recompute=self.disable_recompute, short_conv_weights=conv_w)
        gate = self._heads(self.out_gate_b(gate_rank))
        out = self.out_norm_gate(out, gate).flatten(2)
        return self.out_proj(out)

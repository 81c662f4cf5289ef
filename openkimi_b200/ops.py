"""``chunk_kda``: the KDA chunkwise gated delta rule, forward and backward, on B200.

Drop-in for the call the reference makes at k3mini/model.py:197-216
(``fla.ops.kda.chunk_kda``): same arguments, same gate / beta / initial-state /
final-state / ``cu_seqlens`` meaning, same return value ``(o, final_state_or_None)``.
The arithmetic runs in ``libkda_b200.so`` (hand-written CUDA for sm_100a) through the C ABI
of include/kda_b200.h; PyTorch only owns the memory and the stream.
"""

from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache

import torch

from . import _lib, chunk_intra

_DTYPES = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16}


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


@lru_cache(maxsize=64)
def _chunk_tables_cached(cu: tuple, device_index: int):
    lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
    if any(l < 0 for l in lens):
        raise ValueError("cu_seqlens must be non-decreasing")
    counts = [(l + _lib.CHUNK - 1) // _lib.CHUNK for l in lens]
    off = [0]
    for c in counts:
        off.append(off[-1] + c)
    seq = [n for n, c in enumerate(counts) for _ in range(c)]
    # per chunk: sequence, chunk inside the sequence, first flattened token, valid rows
    tab = [(n, j, cu[n] + j * _lib.CHUNK, min(_lib.CHUNK, lens[n] - j * _lib.CHUNK))
           for n, c in enumerate(counts) for j in range(c)]
    dev = torch.device("cuda", device_index)
    return (torch.tensor(seq if seq else [0], dtype=torch.int32, device=dev),
            torch.tensor(off, dtype=torch.int32, device=dev), off[-1],
            torch.tensor(tab if tab else [(0, 0, 0, 0)], dtype=torch.int32, device=dev))


def _chunk_tables(cu_seqlens, cu_seqlens_cpu, device):
    """Per-chunk sequence index and per-sequence first chunk.  Chunks never straddle a
    document boundary, so the table depends on the lengths; it is built on the host
    (``cu_seqlens_cpu`` avoids the device-to-host copy) and cached per length tuple."""
    host = cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens.cpu()
    return _chunk_tables_cached(tuple(int(x) for x in host.tolist()), device.index or 0)


class _DeviceStatus:
    """One int32 status word per device, mirrored in pinned host memory.  A kernel whose bounded wait
    gives up ORs a code into the device word (``KdaParams.status``) and stores the word into the pinned
    mirror (``KdaParams.status_host``, device-mapped) itself, so the next
    call on that device (or ``check_device_status``) notices it by reading host memory: no copy engine,
    no synchronisation on the hot path."""

    _per_device: dict = {}

    def __init__(self, device):
        self.dev = torch.zeros(1, dtype=torch.int32, device=device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()  # device-mapped under unified addressing

    @classmethod
    def get(cls, device):
        key = device.index if device.index is not None else torch.cuda.current_device()
        st = cls._per_device.get(key)
        if st is None:
            st = cls._per_device[key] = cls(torch.device("cuda", key))
        return st

    def poll(self, sync=False):
        if sync:
            self.host.copy_(self.dev)
        code = int(self.host[0])
        if code:
            self.dev.zero_()
            self.host.zero_()
            msg = _lib.load().kda_status_string(_lib.ERR_DEVICE_WAIT).decode()
            raise RuntimeError(f"chunk_kda: {msg} (stage bits 0x{code:x}); the results of the affected call are invalid")


def check_device_status(device=None, sync=True):
    """Raise if a KDA kernel on ``device`` reported a bounded wait that gave up.  ``sync=True``
    reads the status word now (blocking); ``sync=False`` only looks at copies already finished."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _DeviceStatus.get(dev).poll(sync=sync)


class _Call:
    """Builds the KdaParams block for one forward (+ backward) call."""

    def __init__(self, q, k, v, g, beta, A_log, dt_bias, scale, h0, cu_seqlens, cu_seqlens_cpu, flags, conv=None):
        B, T, H, dk = q.shape
        self.shape = (B, T, H, dk, v.shape[-1])
        self.dev = q.device
        self.cu = None
        if cu_seqlens is not None:
            self.cu = cu_seqlens.to(device=q.device, dtype=torch.int64).contiguous()
            self.chunk_seq, self.seq_off, self.NT, self.chunk_tab = _chunk_tables(cu_seqlens, cu_seqlens_cpu, q.device)
            self.N = self.cu.numel() - 1
        else:
            self.chunk_seq = self.seq_off = None
            self.N = B
            self.NT = B * ((T + _lib.CHUNK - 1) // _lib.CHUNK)
        p = _lib.KdaParams()
        p.B, p.T, p.H, p.dk, p.dv = self.shape
        p.N, p.NT = self.N, max(self.NT, 1)
        p.dtype = _DTYPES[q.dtype]
        p.flags = flags
        p.scale = float(scale)
        p.guard_span = chunk_intra.current_guard_span()
        p.q, p.k, p.v, p.g, p.beta = (t.data_ptr() for t in (q, k, v, g, beta))
        p.A_log = A_log.data_ptr() if A_log is not None else None
        p.dt_bias = dt_bias.data_ptr() if dt_bias is not None else None
        p.h0 = h0.data_ptr() if h0 is not None else None
        if self.cu is not None:
            p.cu_seqlens = self.cu.data_ptr()
            p.chunk_seq = self.chunk_seq.data_ptr()
            p.seq_chunk_off = self.seq_off.data_ptr()
            p.chunk_tab = self.chunk_tab.data_ptr()
        if conv is not None:
            p.conv_q, p.conv_k, p.conv_v = (w.data_ptr() for w in conv)
            p.conv_ksize = conv[0].shape[-1]
        self.status = _DeviceStatus.get(q.device)
        self.status.poll()  # a wait that gave up in an earlier call surfaces here
        p.status = self.status.dev.data_ptr()
        p.status_host = self.status.host.data_ptr()
        self.p = p
        fb, bb = C.c_size_t(0), C.c_size_t(0)
        _lib.check(_lib.load().kda_workspace_bytes(C.byref(p), C.byref(fb), C.byref(bb)), "kda_workspace_bytes")
        self.fwd_bytes, self.bwd_bytes = fb.value, bb.value

    def stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)


_warned = set()


def _warn_once(msg):
    if msg not in _warned:
        _warned.add(msg)
        import warnings
        warnings.warn(msg, RuntimeWarning, stacklevel=3)


def _require_cuda(t):
    if not t.is_cuda:
        raise RuntimeError("chunk_kda runs only on a CUDA device (sm_100a); there is no CPU fallback")


class ChunkKDAFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, A_log, dt_bias, h0, conv_q, conv_k, conv_v, scale, flags, output_final_state,
                cu_seqlens, cu_seqlens_cpu, disable_recompute):
        lib = _lib.load()
        in_dtypes = (g.dtype, beta.dtype)
        dt = q.dtype
        q, k, v, g, beta = (t.to(dt).contiguous() for t in (q, k, v, g, beta))
        A_log = A_log.float().contiguous() if A_log is not None else None
        dt_bias = dt_bias.float().contiguous() if dt_bias is not None else None
        h0 = h0.contiguous() if h0 is not None else None
        # fused short convolution: q, k, v are the projections, conv_* the [H*K, 1, ksize] filters
        conv = None
        if conv_q is not None:
            conv = tuple(w.float().reshape(w.shape[0], w.shape[-1]).contiguous() for w in (conv_q, conv_k, conv_v))
            ctx.conv_dtypes = tuple(w.dtype for w in (conv_q, conv_k, conv_v))
        # Nothing is kept when nobody will differentiate this call (no_grad, e.g. the forward an
        # activation-checkpointed block runs first, k3mini/model.py:825-831) or when the backward rebuilds
        # the records anyway (recompute policy): the forward-only kernels skip every record that only the
        # backward reads and the workspace is the small one.
        keep = disable_recompute and any(ctx.needs_input_grad)
        fwd_flags = flags if keep else flags | _lib.FLAG_NO_SAVE
        with torch.cuda.device(q.device):
            call = _Call(q, k, v, g, beta, A_log, dt_bias, scale, h0, cu_seqlens, cu_seqlens_cpu, fwd_flags, conv)
            B, T, H, dk, dv = call.shape
            o = torch.empty(B, T, H, dv, dtype=dt, device=q.device)
            state_shape = (call.N, H, dv, dk) if flags & _lib.FLAG_STATE_V_FIRST else (call.N, H, dk, dv)
            ht = torch.empty(state_shape, dtype=torch.float32, device=q.device) if output_final_state else None
            ws = torch.empty(call.fwd_bytes, dtype=torch.uint8, device=q.device)
            p = call.p
            p.o, p.ht = o.data_ptr(), (ht.data_ptr() if ht is not None else None)
            p.workspace, p.workspace_bytes = ws.data_ptr(), call.fwd_bytes
            if call.NT > 0:
                _lib.check(lib.kda_fwd(C.byref(p), call.stream()), "kda_fwd")
            elif ht is not None:
                ht.copy_(h0 if h0 is not None else torch.zeros_like(ht))
        ctx.save_for_backward(q, k, v, g, beta, A_log, dt_bias, h0, cu_seqlens, cu_seqlens_cpu,
                              ws if keep else None, *(conv or ()))
        ctx.meta = (scale, flags, in_dtypes, state_shape)
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        lib = _lib.load()
        q, k, v, g, beta, A_log, dt_bias, h0, cu_seqlens, cu_seqlens_cpu, ws, *conv = ctx.saved_tensors
        conv = tuple(conv) or None
        scale, flags, in_dtypes, state_shape = ctx.meta
        dt = q.dtype
        with torch.cuda.device(q.device):
            call = _Call(q, k, v, g, beta, A_log, dt_bias, scale, h0, cu_seqlens, cu_seqlens_cpu, flags, conv)
            p = call.p
            B, T, H, dk, dv = call.shape
            if ws is None:  # recompute policy: rebuild the per-chunk records instead of keeping them
                ws = torch.empty(call.fwd_bytes, dtype=torch.uint8, device=q.device)
                o_tmp = torch.empty(B, T, H, dv, dtype=dt, device=q.device)
                p.o, p.ht = o_tmp.data_ptr(), None
                p.workspace, p.workspace_bytes = ws.data_ptr(), call.fwd_bytes
                if call.NT > 0:
                    _lib.check(lib.kda_fwd(C.byref(p), call.stream()), "kda_fwd (recompute)")
            do = (do if do is not None else torch.zeros(B, T, H, dv, dtype=dt, device=q.device)).to(dt).contiguous()
            dht = dht.float().contiguous() if dht is not None else None
            dq, dk_, dg = torch.empty_like(q), torch.empty_like(k), torch.empty_like(g)
            dv_, dbeta = torch.empty_like(v), torch.empty_like(beta)
            gate = bool(flags & _lib.FLAG_GATE)
            # written in full by the fixed-order reduction kernel (no zero fill needed)
            dA = torch.empty(H, dtype=torch.float32, device=q.device) if gate else None
            dbias = torch.empty(H * dk, dtype=torch.float32, device=q.device) if gate and dt_bias is not None else None
            dh0 = torch.empty(state_shape, dtype=torch.float32, device=q.device) if h0 is not None else None
            scratch = torch.empty(call.bwd_bytes, dtype=torch.uint8, device=q.device)
            p.o = dq.data_ptr()  # unused by the backward; must be non-NULL
            p.workspace, p.workspace_bytes = ws.data_ptr(), call.fwd_bytes
            p.grad_o = do.data_ptr()
            p.grad_ht = dht.data_ptr() if dht is not None else None
            p.grad_q, p.grad_k, p.grad_v = dq.data_ptr(), dk_.data_ptr(), dv_.data_ptr()
            p.grad_g, p.grad_beta = dg.data_ptr(), dbeta.data_ptr()
            p.grad_A_log = dA.data_ptr() if dA is not None else None
            p.grad_dt_bias = dbias.data_ptr() if dbias is not None else None
            p.grad_h0 = dh0.data_ptr() if dh0 is not None else None
            p.bwd_scratch, p.bwd_scratch_bytes = scratch.data_ptr(), call.bwd_bytes
            dconv_f32 = None
            if conv is not None:
                # the backward of the three short convolutions runs inside the KDA backward kernels: dq, dk_, dv_
                # come back as gradients of the projections, the filter gradients in FP32 [H*K, ksize]
                # (written in full by the fixed-order reduction kernel; zero only when there is no chunk at all)
                mk = torch.empty if call.NT > 0 else torch.zeros
                dconv_f32 = [mk(H * dk, w.shape[-1], dtype=torch.float32, device=q.device) for w in conv]
                p.grad_conv_q, p.grad_conv_k, p.grad_conv_v = (t.data_ptr() for t in dconv_f32)
            if call.NT > 0:
                _lib.check(lib.kda_bwd(C.byref(p), call.stream()), "kda_bwd")
            else:
                for t in (dq, dk_, dv_, dg, dbeta, dA, dbias):
                    if t is not None:
                        t.zero_()
                if dh0 is not None:
                    dh0.copy_(dht if dht is not None else torch.zeros_like(dh0))
            dconv = (None, None, None)
            if conv is not None:
                dconv = tuple(dw.view(H * dk, 1, -1).to(wd) for dw, wd in zip(dconv_f32, ctx.conv_dtypes))
        return (dq, dk_, dv_, dg.to(in_dtypes[0]), dbeta.to(in_dtypes[1]), dA, dbias, dh0, *dconv,
                None, None, None, None, None, None)


@torch.compiler.disable
def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
              use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
              cu_seqlens=None, cu_seqlens_cpu=None, safe_gate=False, lower_bound=None, disable_recompute=False,
              state_v_first=False, A_log=None, dt_bias=None, chunk_size=64, fp32_math=False,
              short_conv_weights=None, **kwargs):
    """Kimi Delta Attention, chunkwise (k3mini/model.py:200-216).

    q, k, g: [B, T, H, K]; v: [B, T, H, V]; beta: [B, T, H].  With
    ``use_gate_in_kernel`` g is the raw gate input and the op applies
    ``-exp(A_log) * softplus(g + dt_bias)`` (k3mini/model.py:220-222), otherwise g is the
    natural-log decay per token.  ``use_qk_l2norm_in_kernel`` normalises q and k as
    k3mini/model.py:218-219 does; ``use_beta_sigmoid_in_kernel`` treats beta as logits.
    ``initial_state`` / the returned final state are FP32 ``[N, H, K, V]`` (``[N, H, V, K]``
    with ``state_v_first``).  ``cu_seqlens`` ([N+1], batch 1) packs N documents; chunks and
    the state restart at every document.  ``disable_recompute=True`` keeps the per-chunk
    records between forward and backward, ``False`` rebuilds them in the backward.
    ``fp32_math=True`` forces FP32 CUDA-core arithmetic in every stage (validation mode;
    FP32 inputs always run that way).  Returns ``(o, final_state or None)``.

    ``short_conv_weights=(wq, wk, wv)`` (each ``[H*K, 1, ksize]``, ksize <= 4; an extension, the
    reference has no such argument) says that q, k, v are the projections BEFORE the three
    causal depthwise convolutions + SiLU of k3mini/model.py:181-185.  For BF16 with K = 128 the
    forward kernel applies the filter while it loads the chunk (three halo rows included, the
    window restarting at every sequence start) and the backward kernels run the convolution
    backward on the gradient rows while they are still on chip; otherwise the stand-alone
    convolution kernels run first.  Both routes give the same bits as ``ShortConvolution`` followed
    by ``chunk_kda`` (the filter gradients agree to FP32 summation accuracy).
    """
    state_v_first = bool(kwargs.pop("transpose_state_layout", state_v_first))
    for name in ("return_intermediate_states", "cp_context"):
        if kwargs.pop(name, None):
            raise NotImplementedError(f"chunk_kda: {name} is not supported by the B200 kernels")
    if kwargs:
        raise TypeError(f"chunk_kda: unexpected arguments {sorted(kwargs)}")
    for t in (q, k, v, g, beta):
        _require_cuda(t)
    if safe_gate or lower_bound is not None:
        raise NotImplementedError("chunk_kda: safe_gate/lower_bound are not part of the reference path "
                                  "(k3mini/model.py:212 always passes safe_gate=False)")
    if chunk_size != 64:
        raise ValueError(f"`chunk_size` must be 64 for the B200 KDA kernels, got {chunk_size}.")
    if q.dim() != 4 or q.shape != k.shape:
        raise ValueError(f"q and k must have the same shape [B,T,H,K], got q={tuple(q.shape)} vs k={tuple(k.shape)}")
    B, T, H, K = q.shape
    if v.shape[:3] != q.shape[:3]:
        raise ValueError("grouped value heads (HV != H) are not supported: v must be [B,T,H,V]")
    if g.shape != (B, T, H, K):
        raise ValueError(f"g must have shape {[B, T, H, K]}, got {list(g.shape)}")
    if beta.shape != (B, T, H):
        raise ValueError(f"beta must have shape {[B, T, H]}, got {list(beta.shape)}")
    if K != v.shape[-1] or K not in (64, 128):
        raise ValueError(f"the B200 KDA kernels need K == V in (64, 128), got K={K}, V={v.shape[-1]}")
    if q.dtype not in _DTYPES:
        raise TypeError(f"q/k/v must be float32 or bfloat16, got {q.dtype}")
    if cu_seqlens is not None:
        if B != 1:
            raise ValueError(f"The batch size is expected to be 1 rather than {B} when using `cu_seqlens`."
                             "Please flatten variable-length inputs before processing.")
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError("The number of initial states is expected to be equal to the number of input "
                             f"sequences, i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}.")
    n_seq = B if cu_seqlens is None else len(cu_seqlens) - 1
    if initial_state is not None:
        if initial_state.dtype != torch.float32:
            raise TypeError("initial_state must be in float32.")
        want = (n_seq, H, v.shape[-1], K) if state_v_first else (n_seq, H, K, v.shape[-1])
        if tuple(initial_state.shape) != want:
            raise ValueError(f"initial_state must have shape {want}, got {tuple(initial_state.shape)}")
    if use_gate_in_kernel:
        if A_log is None:
            raise ValueError("A_log must be provided when use_gate_in_kernel=True.")
        if A_log.numel() != H or (dt_bias is not None and dt_bias.numel() != H * K):
            raise ValueError("A_log must have H entries and dt_bias H*K entries")
    else:
        A_log = dt_bias = None
    if scale is None:
        scale = K ** -0.5
    flags = ((_lib.FLAG_QK_L2NORM if use_qk_l2norm_in_kernel else 0) | (_lib.FLAG_GATE if use_gate_in_kernel else 0)
             | (_lib.FLAG_BETA_SIGMOID if use_beta_sigmoid_in_kernel else 0)
             | (_lib.FLAG_STATE_V_FIRST if state_v_first else 0))
    if fp32_math or os.environ.get("OPENKIMI_B200_FP32_MATH") == "1":
        flags |= _lib.FLAG_FORCE_SIMT
    # debugging / A-B measurement: bit s of this mask runs stage s (0 fwd_intra, 1 fwd_state,
    # 2 bwd_state, 3 bwd_chunk as one fused kernel, 4 bwd_wy) with FP32 CUDA-core arithmetic
    # instead of tensor cores
    stage_mask = int(os.environ.get("OPENKIMI_B200_FP32_STAGES", "0")) & 31
    if stage_mask:
        _warn_once(f"OPENKIMI_B200_FP32_STAGES={stage_mask}: the selected KDA stages run the FP32 CUDA-core "
                   "validation kernels instead of the tensor-core kernels (debugging switch, much slower)")
    flags |= stage_mask << 5
    if os.environ.get("OPENKIMI_B200_ROW_COPIES") == "1":  # A-B switch: row copies instead of bulk-tensor tile copies
        flags |= _lib.FLAG_ROW_COPIES
    conv = (None, None, None)
    if short_conv_weights is not None:
        wq, wk, wv = short_conv_weights
        for w in (wq, wk, wv):
            if w.dim() != 3 or w.shape[0] != H * K or w.shape[1] != 1 or not 1 <= w.shape[2] <= 4 or w.shape != wq.shape:
                raise ValueError(f"short_conv_weights must be three [H*K, 1, ksize<=4] filters, got {tuple(w.shape)}")
        if q.dtype == torch.bfloat16 and K == 128 and not flags & ~15:
            conv = (wq, wk, wv)
        else:  # FP32 validation mode and d = 64: same arithmetic, separate kernels
            from .modules import short_convolution
            cu = None if cu_seqlens is None else cu_seqlens.to(device=q.device, dtype=torch.int64).contiguous()
            q, k, v = (short_convolution(x.reshape(B, T, H * K), w, cu).view(B, T, H, K)
                       for x, w in zip((q, k, v), (wq, wk, wv)))
    return ChunkKDAFunction.apply(q, k, v, g, beta, A_log, dt_bias, initial_state, *conv, float(scale), flags,
                                  bool(output_final_state), cu_seqlens, cu_seqlens_cpu, bool(disable_recompute))


def recurrent_kda_step(q, k, v, g, beta, state, *, scale=None, A_log=None, dt_bias=None,
                       use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
                       state_v_first=False, inplace=False):
    """One decoding step of KDA: the recurrence of k3mini/model.py:121-128 for a single token.

    q, k, g: [N, H, K]; v: [N, H, V]; beta: [N, H]; ``state``: FP32 ``[N, H, K, V]`` (``[N, H, V, K]``
    with ``state_v_first``), e.g. the final state ``chunk_kda`` returned for the prompt.  The prologue
    switches mean what they mean in ``chunk_kda``.  Returns ``(o [N, H, V], new_state)``; with
    ``inplace=True`` the state tensor itself is updated and returned.  Inference only (no autograd).
    """
    for t in (q, k, v, g, beta, state):
        _require_cuda(t)
    if q.dim() != 3 or q.shape != k.shape or g.shape != q.shape:
        raise ValueError(f"q, k, g must share one shape [N,H,K], got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(g.shape)}")
    N, H, K = q.shape
    if v.shape != (N, H, K) or K not in (64, 128):
        raise ValueError(f"the B200 KDA kernels need K == V in (64, 128), got K={K}, v={tuple(v.shape)}")
    if beta.shape != (N, H):
        raise ValueError(f"beta must have shape {[N, H]}, got {list(beta.shape)}")
    if q.dtype not in _DTYPES:
        raise TypeError(f"q/k/v must be float32 or bfloat16, got {q.dtype}")
    if state.dtype != torch.float32 or tuple(state.shape) != (N, H, K, K):
        raise ValueError(f"state must be float32 [N,H,{K},{K}], got {state.dtype} {tuple(state.shape)}")
    if use_gate_in_kernel and (A_log is None or A_log.numel() != H or (dt_bias is not None and dt_bias.numel() != H * K)):
        raise ValueError("use_gate_in_kernel=True needs A_log with H entries (and dt_bias with H*K entries)")
    dt = q.dtype
    q, k, v, g, beta = (t.detach().to(dt).contiguous() for t in (q, k, v, g, beta))
    a = A_log.detach().float().contiguous() if use_gate_in_kernel else None
    b = dt_bias.detach().float().contiguous() if (use_gate_in_kernel and dt_bias is not None) else None
    s_in = state.detach().contiguous()
    s_out = s_in if inplace and s_in.data_ptr() == state.data_ptr() else torch.empty_like(s_in)
    o = torch.empty_like(v)
    flags = ((_lib.FLAG_QK_L2NORM if use_qk_l2norm_in_kernel else 0) | (_lib.FLAG_GATE if use_gate_in_kernel else 0)
             | (_lib.FLAG_BETA_SIGMOID if use_beta_sigmoid_in_kernel else 0)
             | (_lib.FLAG_STATE_V_FIRST if state_v_first else 0))
    with torch.cuda.device(q.device):
        st = _DeviceStatus.get(q.device)
        st.poll()
        rc = _lib.load().kda_recurrent_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                            _ptr(a), _ptr(b), s_in.data_ptr(), s_out.data_ptr(), o.data_ptr(), N, H, K, K,
                                            _DTYPES[dt], flags, float(K ** -0.5 if scale is None else scale),
                                            st.dev.data_ptr(), C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
        _lib.check(rc, "kda_recurrent_step")
    return o, s_out


def fused_recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, **kw):
    """Token-by-token KDA over ``[B, T, H, K]`` inputs through ``recurrent_kda_step`` (the decoding
    counterpart of ``chunk_kda``, same prologue keywords; meant for the few tokens of a decode loop).
    Returns ``(o [B, T, H, V], final_state or None)``."""
    B, T, H, K = q.shape
    vfirst = bool(kw.get("state_v_first", False))
    state = (initial_state.detach().clone() if initial_state is not None
             else torch.zeros(B, H, K, K, dtype=torch.float32, device=q.device))
    outs = []
    for t in range(T):
        o, state = recurrent_kda_step(q[:, t], k[:, t], v[:, t], g[:, t], beta[:, t], state, scale=scale, inplace=True, **kw)
        outs.append(o)
    o = torch.stack(outs, dim=1) if outs else v.new_zeros(B, 0, H, K)
    return o, (state if output_final_state else None)

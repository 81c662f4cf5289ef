"""CPU oracle for Kimi Delta Attention (KDA).  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the reference algorithm that the
CUDA kernels of ``openkimi_b200`` must reproduce.  Only the test-suite, the smoke entry
and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it; the
product package never does.

Parity pin: ``tests/golden/make_golden.py`` runs the reference's own
``k3mini.model.kda_recurrent_reference`` (k3mini/model.py:101-129) and its prologue
(k3mini/model.py:217-223) on seeded inputs and commits the results under
``tests/golden/``; ``tests/test_oracle_golden.py`` checks this restatement against them.
Initial state, final state, ``cu_seqlens`` and the state gradients have no counterpart in
the reference's oracle (it always starts from a zero state and returns only ``o``): for
those arguments parity is unpinned by the reference and is anchored on the recurrence
itself (same update, state seeded from ``h0``, documents run one after another).

Every function cites the reference lines it follows.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

LOG2E = 1.0 / math.log(2.0)


def l2_normalize(x: torch.Tensor, eps: float = 1e-6, dtype=torch.float32) -> torch.Tensor:
    """x / max(||x||_2, eps) over the last axis in FP32 (k3mini/model.py:218-219)."""
    xf = x.to(dtype)
    return xf / xf.norm(dim=-1, keepdim=True).clamp_min(eps)


def kda_gate(raw: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor | None, dtype=torch.float32) -> torch.Tensor:
    """log-decay  -exp(A_log)[h] * softplus(raw + dt_bias[h, :])  (k3mini/model.py:220-222)."""
    heads, dim = raw.shape[-2], raw.shape[-1]
    x = raw.to(dtype)
    if dt_bias is not None:
        x = x + dt_bias.to(dtype).view(heads, dim)
    return -a_log.to(dtype).exp().view(heads, 1) * F.softplus(x)


def kda_prologue(q, k, g, beta, *, a_log=None, dt_bias=None, use_qk_l2norm=True,
                 use_gate=True, use_beta_sigmoid=True, round_to=None, dtype=torch.float32):
    """Reference-branch prologue of KimiDeltaAttention.forward (k3mini/model.py:217-223).

    ``round_to`` reproduces the ``.to(x.dtype)`` round trip the reference applies to the
    normalised q and k (model.py:218-219) when the activations are BF16.  ``dtype`` is the
    arithmetic type: float32 as in the reference, float64 for a check free of the oracle's
    own rounding.
    """
    if use_qk_l2norm:
        q, k = l2_normalize(q, dtype=dtype), l2_normalize(k, dtype=dtype)
        if round_to is not None:
            q, k = q.to(round_to), k.to(round_to)
    log_alpha = kda_gate(g, a_log, dt_bias, dtype) if use_gate else g.to(dtype)
    beta = beta.to(dtype).sigmoid() if use_beta_sigmoid else beta.to(dtype)
    return q, k, log_alpha, beta


def kda_recurrent_oracle(q, k, v, log_alpha, beta, *, scale=None, initial_state=None,
                         output_final_state=False, cu_seqlens=None, dtype=torch.float32):
    """Token-by-token delta rule with per-channel decay (k3mini/model.py:115-129).

    Per token, exactly in the reference's order: decay the state rows by
    alpha_t = exp(log_alpha_t) (model.py:122), read the prediction k_t^T S (:123), form the
    error v_t - prediction (:124), add the rank-one correction k_t (beta_t error)^T (:125-127)
    and emit o_t = scale * S^T q_t from the *updated* state (:128).

    Extensions with no counterpart in the reference's oracle: ``initial_state`` /
    final state of shape [N, H, dk, dv], and ``cu_seqlens`` (batch 1, documents processed
    independently, each starting from its own initial state).  ``dtype`` is the state and
    arithmetic type (float32 as in the reference; float64 for a tighter check).
    """
    if not (q.shape == k.shape == log_alpha.shape) or q.shape[:-1] != v.shape[:-1]:
        raise ValueError("q, k, v, and log_alpha must have identical shapes")
    if beta.shape != q.shape[:-1]:
        raise ValueError("beta must have shape [B,T,H]")
    batch, time, heads, dk = q.shape
    dv = v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    alpha, bf = log_alpha.to(dtype).exp(), beta.to(dtype)

    if cu_seqlens is None:
        spans = [(b, 0, time) for b in range(batch)]
    else:
        if batch != 1:
            raise ValueError("cu_seqlens requires batch size 1")
        cs = [int(x) for x in cu_seqlens]
        spans = [(0, cs[i], cs[i + 1]) for i in range(len(cs) - 1)]
    n_seq = len(spans)
    if initial_state is not None and initial_state.shape[0] != n_seq:
        raise ValueError("initial_state must hold one state per sequence")

    outs, finals = [], []
    for n, (b, t0, t1) in enumerate(spans):
        state = (torch.zeros(heads, dk, dv, dtype=dtype) if initial_state is None
                 else initial_state[n].to(dtype))
        rows = []
        for t in range(t0, t1):
            state = state * alpha[b, t].unsqueeze(-1)
            pred = torch.einsum("hd,hdv->hv", kf[b, t], state)
            err = vf[b, t] - pred
            state = state + kf[b, t].unsqueeze(-1) * (bf[b, t].unsqueeze(-1) * err).unsqueeze(-2)
            rows.append(torch.einsum("hdv,hd->hv", state, qf[b, t]) * scale)
        outs.append(torch.stack(rows) if rows else torch.zeros(0, heads, dv, dtype=dtype))
        finals.append(state)
    # assembled by stack/cat (no in-place writes) so autograd flows through
    if cu_seqlens is None:
        out = torch.stack(outs, dim=0)
    else:
        out = torch.cat(outs, dim=0).unsqueeze(0)
        if out.shape[1] != time:
            raise ValueError("cu_seqlens must cover every token")
    final = torch.stack(finals, dim=0) if output_final_state else None
    return out, final


def kda_oracle(q, k, v, g, beta, *, a_log=None, dt_bias=None, scale=None, initial_state=None,
               output_final_state=False, use_qk_l2norm=True, use_gate=True,
               use_beta_sigmoid=True, cu_seqlens=None, dtype=torch.float32, round_qk_to=None):
    """Prologue + recurrence, i.e. the reference branch of KimiDeltaAttention.forward
    (k3mini/model.py:217-223) with the state extensions described above."""
    qn, kn, log_alpha, b = kda_prologue(q, k, g, beta, a_log=a_log, dt_bias=dt_bias,
                                        use_qk_l2norm=use_qk_l2norm, use_gate=use_gate,
                                        use_beta_sigmoid=use_beta_sigmoid, round_to=round_qk_to, dtype=dtype)
    return kda_recurrent_oracle(qn, kn, v, log_alpha, b, scale=scale, initial_state=initial_state,
                                output_final_state=output_final_state, cu_seqlens=cu_seqlens,
                                dtype=dtype)


def short_conv_oracle(x: torch.Tensor, weight: torch.Tensor, cu_seqlens=None) -> torch.Tensor:
    """Causal depthwise conv1d + SiLU (k3mini/model.py:84-88): left-pad k-1 zeros, one filter
    per channel (weight [C,1,k]), SiLU.  With ``cu_seqlens`` every document is padded
    separately so no tap reads across a document boundary."""
    ksz = weight.shape[-1]

    def one(seq):  # [1, T, C]
        xt = F.pad(seq.transpose(1, 2), (ksz - 1, 0))
        return F.silu(F.conv1d(xt, weight.to(seq.dtype), groups=weight.shape[0]).transpose(1, 2))

    if cu_seqlens is None:
        return one(x)
    cs = [int(c) for c in cu_seqlens]
    return torch.cat([one(x[:, cs[i]:cs[i + 1]]) for i in range(len(cs) - 1)], dim=1)


def rms_norm_gate_oracle(x, gate_logits, weight, eps: float = 1e-6) -> torch.Tensor:
    """Headwise RMSNorm(x) * sigmoid(gate) (k3mini/model.py:69-73, 97-98)."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    return (xf * weight.float()).to(x.dtype) * gate_logits.sigmoid()


def kda_sublayer_oracle(x, params, *, n_heads, head_dim, cu_seqlens=None, eps=1e-6, dtype=torch.float32):
    """The reference branch of KimiDeltaAttention.forward (k3mini/model.py:190-227):
    projections -> causal conv + SiLU -> head split -> prologue -> recurrent oracle -> gated
    headwise RMSNorm -> output projection.  ``params`` uses the reference module's parameter
    names (q_proj.weight, q_conv.weight, A_log, dt_bias, out_norm_gate.weight, ...)."""
    w = lambda n: params[n].to(dtype)
    xx = x.to(dtype)
    heads = lambda t: t.view(*t.shape[:2], n_heads, head_dim)
    q, k, v = (heads(short_conv_oracle(F.linear(xx, w(f"{n}_proj.weight")), w(f"{n}_conv.weight"), cu_seqlens))
               for n in ("q", "k", "v"))
    raw = heads(F.linear(F.linear(xx, w("f_a_proj.weight")), w("f_b_proj.weight")))
    beta_logits = F.linear(xx, w("beta_proj.weight"))
    o, _ = kda_oracle(q, k, v, raw, beta_logits, a_log=params["A_log"], dt_bias=params["dt_bias"].reshape(-1),
                      scale=head_dim ** -0.5, cu_seqlens=cu_seqlens, dtype=dtype)
    gate = heads(F.linear(F.linear(xx, w("out_gate_a.weight")), w("out_gate_b.weight")))
    y = rms_norm_gate_oracle(o, gate, w("out_norm_gate.weight"), eps).flatten(2)
    return F.linear(y.to(dtype), w("out_proj.weight"))


def gate_tile_spans_oracle(raw, a_log, dt_bias, chunk=64, block=16, ch_tile=32) -> torch.Tensor:
    """log2 span of every [16 rows x 32 channels] tile of the within-chunk cumulative gate
    (scripts/profile_kda_gate_spans.py:21-56): first row of the tile minus the minimum."""
    b, t, h, d = raw.shape
    if t % chunk or d % ch_tile:
        raise ValueError("sequence length / head dim incompatible with the tile")
    steps = kda_gate(raw, a_log, dt_bias.reshape(-1)) * LOG2E
    cum = steps.view(b, t // chunk, chunk, h, d).cumsum(dim=2)
    tiles = cum.view(b, t // chunk, chunk // block, block, h, d // ch_tile, ch_tile)
    return (tiles[:, :, :, :1] - tiles).amax(dim=(3, 6)).flatten()


# --------------------------------------------------------------------------------------
# Guarded diagonal backward (experiments/kda_sm90/guarded_diagonal_oracle.py:57-180)
# --------------------------------------------------------------------------------------

def diagonal_exact_oracle(gate, q, k, beta, da_qk, da_kk):
    """Exact pairwise 2^(g_i-g_j) evaluation of one 16-row diagonal tile
    (guarded_diagonal_oracle.py:57-107).  Returns dq, dk, dkt.

    dq[i]  = sum_{j<=i} dAqk[i,j] k[j] 2^(g_i-g_j)
    dk[i]  = sum_{j<=i} dAkk[i,j] k[j] 2^(g_i-g_j)
    dkt[i] = sum_{j>=i} (dAqk[i,j] q[j] + dAkk[i,j] beta[j] k[j]) 2^(g_j-g_i)
    (the dA arguments of the third line are indexed exactly as the reference indexes them:
    row index first, so the caller passes the transposed matrices for the column term).
    """
    n = gate.shape[1]
    idx = torch.arange(n)
    low = idx[:, None] >= idx[None, :]
    upp = idx[:, None] <= idx[None, :]
    diff = gate[:, :, None, :] - gate[:, None, :, :]
    dec_l = torch.exp2(torch.where(low[None, :, :, None], diff, torch.zeros((), dtype=gate.dtype)))
    dec_u = torch.exp2(torch.where(upp[None, :, :, None], -diff, torch.zeros((), dtype=gate.dtype)))
    qk_l, kk_l = da_qk * low, da_kk * low
    qk_u, kk_u = da_qk * upp, da_kk * upp
    dq = torch.einsum("bij,bjc,bijc->bic", qk_l, k, dec_l)
    dk = torch.einsum("bij,bjc,bijc->bic", kk_l, k, dec_l)
    dkt = torch.einsum("bij,bjc,bijc->bic", qk_u, q, dec_u)
    dkt = dkt + torch.einsum("bij,bjc,bijc->bic", kk_u, k * beta[..., None], dec_u)
    return dq, dk, dkt


def diagonal_guard_oracle(gate, max_log2_span):
    """Tile acceptance rule (guarded_diagonal_oracle.py:131-141): per-channel monotone
    non-increasing, finite, and max over channels of (max - min) <= span."""
    gmax = gate.amax(dim=1, keepdim=True)
    gmin = gate.amin(dim=1, keepdim=True)
    spans = (gmax - gmin).amax(dim=(1, 2))
    mono = torch.all(gate[:, 1:, :] <= gate[:, :-1, :], dim=(1, 2))
    return mono & torch.isfinite(spans) & (spans <= max_log2_span), (gmax + gmin) * 0.5


def diagonal_guarded_oracle(gate, q, k, beta, da_qk, da_kk, *, max_log2_span):
    """Midpoint-factorised fast path on accepted tiles, exact fallback elsewhere
    (guarded_diagonal_oracle.py:110-180, reference_policy="midpoint")."""
    if not (0.0 < max_log2_span < 252.0) or not math.isfinite(max_log2_span):
        raise ValueError("max_log2_span must be finite and between 0 and 252")
    dq, dk, dkt = (t.clone() for t in diagonal_exact_oracle(gate, q, k, beta, da_qk, da_kk))
    hits, ref = diagonal_guard_oracle(gate, max_log2_span)
    n = gate.shape[1]
    idx = torch.arange(n)
    low = idx[:, None] >= idx[None, :]
    upp = idx[:, None] <= idx[None, :]
    if bool(hits.any()):
        g, r = gate[hits], ref[hits]
        pos, neg = torch.exp2(g - r), torch.exp2(r - g)
        dq[hits] = torch.bmm((da_qk * low)[hits], k[hits] * neg) * pos
        dk[hits] = torch.bmm((da_kk * low)[hits], k[hits] * neg) * pos
        dkt[hits] = (torch.bmm((da_qk * upp)[hits], q[hits] * pos)
                     + torch.bmm((da_kk * upp)[hits], k[hits] * beta[hits][..., None] * pos)) * neg
    return dq, dk, dkt, hits


# --------------------------------------------------------------------------------------
# Seeded input recipes of the benchmark configurations
# --------------------------------------------------------------------------------------

def make_inputs(batch, time, heads, dim, *, seed=0, dtype=torch.float32, x_mean=0.0,
                a_lo=1.0, a_hi=16.0, beta_mean=0.0, fused=True):
    """Seeded synthetic inputs with the distributions the benchmark configurations name:
    q,k,v ~ N(0,1); gate input x ~ N(x_mean,1); A_log ~ U(ln a_lo, ln a_hi) per head;
    beta logits ~ N(beta_mean,1); upstream gradient do ~ N(0,1).  Generated on the CPU in
    FP32 with one generator and then cast, so the oracle and the GPU see the same bits.

    ``fused=True`` returns raw tensors for the in-kernel prologue (L2 norm, gate, sigmoid);
    ``fused=False`` returns already normalised q/k, the natural-log decay g and beta.
    """
    gen = torch.Generator().manual_seed(seed)
    shape = (batch, time, heads, dim)
    q = torch.randn(shape, generator=gen)
    k = torch.randn(shape, generator=gen)
    v = torch.randn(shape, generator=gen)
    x = torch.randn(shape, generator=gen) + x_mean
    bl = torch.randn(shape[:-1], generator=gen) + beta_mean
    a_log = torch.empty(heads).uniform_(math.log(a_lo), math.log(a_hi), generator=gen)
    do = torch.randn(shape, generator=gen)
    dt_bias = torch.zeros(heads * dim)
    d = dict(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype), g=x.to(dtype), beta=bl.to(dtype),
             a_log=a_log, dt_bias=dt_bias, do=do.to(dtype))
    if not fused:
        d["q"] = l2_normalize(d["q"]).to(dtype)
        d["k"] = l2_normalize(d["k"]).to(dtype)
        d["g"] = kda_gate(d["g"], a_log, dt_bias).to(dtype)
        d["beta"] = d["beta"].float().sigmoid().to(dtype)
    return d


def random_cu_seqlens(total, n_docs, seed=0):
    """n_docs document lengths drawn uniformly (sorted distinct cut points) summing to total."""
    gen = torch.Generator().manual_seed(seed)
    cuts = torch.randperm(total - 1, generator=gen)[: n_docs - 1] + 1
    cs = torch.cat([torch.zeros(1, dtype=torch.long), cuts.sort().values, torch.tensor([total])])
    return cs.to(torch.long)


def kda_oracle_fwd_bwd(q, k, v, g, beta, do, *, a_log=None, dt_bias=None, scale=None,
                       initial_state=None, dht=None, cu_seqlens=None, use_qk_l2norm=True,
                       use_gate=True, use_beta_sigmoid=True, dtype=torch.float32, round_qk_to=None):
    """Forward through ``kda_oracle`` and gradients by autograd, the way the reference's
    parity test obtains them (tests/test_h100_parity.py:84-113 with ``output.backward(do)``
    as in scripts/benchmark_kda_backends.py:139-147).  Returns a dict with o, ht and the
    gradients of every differentiable input."""
    leaves = {}

    def leaf(name, t):
        if t is None:
            return None
        x = t.detach().clone().to(dtype if t.is_floating_point() else t.dtype).requires_grad_(True)
        leaves[name] = x
        return x

    ql, kl, vl, gl, bl = leaf("q", q), leaf("k", k), leaf("v", v), leaf("g", g), leaf("beta", beta)
    al = leaf("A_log", a_log) if use_gate else None
    dl = leaf("dt_bias", dt_bias) if use_gate else None
    hl = leaf("h0", initial_state)
    o, ht = kda_oracle(ql, kl, vl, gl, bl, a_log=al, dt_bias=dl, scale=scale, initial_state=hl,
                       output_final_state=True, use_qk_l2norm=use_qk_l2norm, use_gate=use_gate,
                       use_beta_sigmoid=use_beta_sigmoid, cu_seqlens=cu_seqlens, dtype=dtype,
                       round_qk_to=round_qk_to)
    loss = (o * do.to(dtype)).sum()
    if dht is not None:
        loss = loss + (ht * dht.to(dtype)).sum()
    loss.backward()
    res = {"o": o.detach(), "ht": ht.detach()}
    for name, x in leaves.items():
        res["d" + name] = x.grad if x.grad is not None else torch.zeros_like(x)
    return res

"""Chunkwise KDA forward and hand-derived backward on the CPU.  TEST INFRASTRUCTURE ONLY.

The CUDA kernels do not run the token-by-token recurrence of k3mini/model.py:115-129; they
run its chunkwise (C = 64) reformulation with a WY / UT-transform solve inside each chunk
and an explicitly derived backward pass.  This file states that reformulation once, in
FP64 PyTorch without autograd, in the same stages the kernels use, so that

* the algebra is checked against autograd through the recurrent oracle
  (``tests/test_blueprint.py``), and
* every intermediate a kernel writes (W, U, Aqk, V', chunk states, dV', dS ...) has a
  CPU value to be compared with when a kernel is debugged.

It follows the recurrence of k3mini/model.py:122-128: with G the within-chunk inclusive
cumulative log-decay and S0 the state entering the chunk,

    Aqk[i,j] = scale * sum_d q[i,d] k[j,d] e^(G[i,d]-G[j,d])     (i >= j)
    L[i,j]   =         sum_d k[i,d] k[j,d] e^(G[i,d]-G[j,d])     (i >  j)
    T = (I + diag(beta) L)^-1,  W = T diag(beta) (k * e^G),  U = T diag(beta) V
    V' = U - W S0,   O = (scale q * e^G) S0 + Aqk V',
    S1 = diag(e^G_last) S0 + (k * e^(G_last - G))^T V'.
"""

from __future__ import annotations

import torch

CHUNK = 64


def _chunks(t0, t1, chunk):
    return [(s, min(s + chunk, t1)) for s in range(t0, t1, chunk)]


def chunk_forward_one(q, k, v, g, beta, s0, scale, chunk=CHUNK):
    """One (sequence, head): q,k,g [T,dk], v [T,dv], beta [T], s0 [dk,dv] -> o, s_final, saved."""
    T = q.shape[0]
    S = s0.clone()
    o = torch.zeros(T, v.shape[1], dtype=q.dtype)
    saved = []
    for (a, b) in _chunks(0, T, chunk):
        qc, kc, vc, bc = q[a:b], k[a:b], v[a:b], beta[a:b]
        G = g[a:b].cumsum(0)
        n = b - a
        gam = G.exp()
        D = (G[:, None, :] - G[None, :, :])
        low = torch.tril(torch.ones(n, n, dtype=torch.bool))
        D = torch.where(low[:, :, None], D, torch.zeros((), dtype=q.dtype)).exp() * low[:, :, None]
        Aqk = scale * torch.einsum("id,jd,ijd->ij", qc, kc, D)
        L = torch.einsum("id,jd,ijd->ij", kc, kc, D) * torch.tril(torch.ones(n, n, dtype=q.dtype), -1)
        M = torch.eye(n, dtype=q.dtype) + bc[:, None] * L
        Tm = torch.linalg.solve_triangular(M, torch.eye(n, dtype=q.dtype), upper=False)
        Kt = kc * gam
        Kh = kc * (G[-1:] - G).exp()
        Qt = scale * qc * gam
        W = Tm @ (bc[:, None] * Kt)
        U = Tm @ (bc[:, None] * vc)
        Vn = U - W @ S
        o[a:b] = Qt @ S + Aqk @ Vn
        saved.append(dict(a=a, b=b, G=G, D=D, Aqk=Aqk, L=L, T=Tm, Kt=Kt, Kh=Kh, Qt=Qt, W=W, U=U,
                          Vn=Vn, S0=S.clone()))
        S = gam[-1][:, None] * S + Kh.t() @ Vn
    return o, S, saved


def chunk_backward_one(q, k, v, g, beta, scale, saved, do, dS_final):
    """Adjoint of ``chunk_forward_one``: returns dq, dk, dv, dg, dbeta, dS0."""
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    dg, dbeta = torch.zeros_like(g), torch.zeros_like(beta)
    dS = dS_final.clone()
    for st in reversed(saved):
        a, b = st["a"], st["b"]
        n = b - a
        qc, kc, vc, bc = q[a:b], k[a:b], v[a:b], beta[a:b]
        G, D, Aqk, L, Tm = st["G"], st["D"], st["Aqk"], st["L"], st["T"]
        Kt, Kh, Qt, W, Vn, S0 = st["Kt"], st["Kh"], st["Qt"], st["W"], st["Vn"], st["S0"]
        gam = G.exp()
        dOc = do[a:b]
        # ---- state stage (reverse sequential): needs dS entering from the right
        dVn = Aqk.t() @ dOc + Kh @ dS
        dS0 = gam[-1][:, None] * dS + Qt.t() @ dOc - W.t() @ dVn
        # ---- chunk-local stage (parallel over chunks once S0, dS, dVn are known)
        dAqk = torch.tril(dOc @ Vn.t())
        dQt = dOc @ S0.t()
        dKh = Vn @ dS.t()
        dW = -dVn @ S0.t()
        dgamC = (dS * S0).sum(1)
        Kb, Vb = bc[:, None] * Kt, bc[:, None] * vc
        dT = torch.tril(dW @ Kb.t() + dVn @ Vb.t())
        dKb, dVb = Tm.t() @ dW, Tm.t() @ dVn
        dM = -Tm.t() @ dT @ Tm.t()
        dL = torch.tril(bc[:, None] * dM, -1)
        dbeta[a:b] = (dM * L).sum(1) + (dKb * Kt).sum(1) + (dVb * vc).sum(1)
        dv[a:b] = bc[:, None] * dVb
        dKt = bc[:, None] * dKb
        # ---- intra step: pairwise decays D[i,j,d] = e^(G_i-G_j), i >= j
        dq_in = scale * torch.einsum("ij,jd,ijd->id", dAqk, kc, D)
        dk_row = torch.einsum("ij,jd,ijd->id", dL, kc, D)
        dk_col = scale * torch.einsum("ij,id,ijd->jd", dAqk, qc, D) + torch.einsum("ij,id,ijd->jd", dL, kc, D)
        dG = qc * dq_in + kc * dk_row - kc * dk_col
        # ---- decay-scaled operands
        dqc = dq_in + scale * dQt * gam
        dkc = dk_row + dk_col + dKt * gam + dKh * (G[-1:] - G).exp()
        dG = dG + dQt * Qt + dKt * Kt - dKh * Kh
        dG[-1] = dG[-1] + (dKh * Kh).sum(0) + dgamC * gam[-1]
        dq[a:b], dk[a:b] = dqc, dkc
        dg[a:b] = dG.flip(0).cumsum(0).flip(0)
        dS = dS0
    return dq, dk, dv, dg, dbeta, dS


def prologue_forward(q_raw, k_raw, x, beta_raw, a_log_h, dt_bias_h, flags, eps=1e-6):
    """Per head: optional L2 norm, gate, sigmoid.  Returns the activated tensors and what the
    chain rule needs."""
    use_l2, use_gate, use_sig = flags
    if use_l2:
        qn_ = q_raw.norm(dim=-1, keepdim=True).clamp_min(eps)
        kn_ = k_raw.norm(dim=-1, keepdim=True).clamp_min(eps)
        q, k = q_raw / qn_, k_raw / kn_
    else:
        qn_ = kn_ = None
        q, k = q_raw, k_raw
    if use_gate:
        z = x + dt_bias_h
        g = -a_log_h.exp() * torch.nn.functional.softplus(z)
    else:
        z, g = None, x
    beta = beta_raw.sigmoid() if use_sig else beta_raw
    return q, k, g, beta, (qn_, kn_, z)


def prologue_backward(q, k, g, beta, aux, dq, dk, dg, dbeta, a_log_h, flags):
    use_l2, use_gate, use_sig = flags
    qn_, kn_, z = aux
    if use_l2:
        dq = (dq - q * (q * dq).sum(-1, keepdim=True)) / qn_
        dk = (dk - k * (k * dk).sum(-1, keepdim=True)) / kn_
    dA = torch.zeros((), dtype=q.dtype)
    dbias = torch.zeros(q.shape[-1], dtype=q.dtype)
    if use_gate:
        dA = (dg * g).sum()
        dx = dg * (-a_log_h.exp()) * z.sigmoid()
        dbias = dx.sum(0)
    else:
        dx = dg
    if use_sig:
        dbeta = dbeta * beta * (1 - beta)
    return dq, dk, dx, dbeta, dA, dbias


def kda_chunk_blueprint(q, k, v, g, beta, do, *, a_log=None, dt_bias=None, scale=None, h0=None,
                        dht=None, cu_seqlens=None, use_qk_l2norm=True, use_gate=True,
                        use_beta_sigmoid=True, chunk=CHUNK, dtype=torch.float64):
    """Full op on [B,T,H,d] tensors: returns dict(o, ht, dq, dk, dv, dg, dbeta, dA_log, ddt_bias, dh0)."""
    B, T, H, dk_ = q.shape
    dv_ = v.shape[-1]
    scale = dk_ ** -0.5 if scale is None else scale
    flags = (use_qk_l2norm, use_gate, use_beta_sigmoid)
    if cu_seqlens is None:
        spans = [(b, 0, T) for b in range(B)]
    else:
        cs = [int(c) for c in cu_seqlens]
        spans = [(0, cs[i], cs[i + 1]) for i in range(len(cs) - 1)]
    N = len(spans)
    cast = lambda t: None if t is None else t.to(dtype)
    q, k, v, g, beta, do, h0, dht = map(cast, (q, k, v, g, beta, do, h0, dht))
    a_log = cast(a_log) if a_log is not None else torch.zeros(H, dtype=dtype)
    dt_bias = cast(dt_bias).view(H, dk_) if dt_bias is not None else torch.zeros(H, dk_, dtype=dtype)
    out = {n: torch.zeros_like(t) for n, t in (("o", v), ("dq", q), ("dk", k), ("dv", v), ("dg", g), ("dbeta", beta))}
    out["ht"] = torch.zeros(N, H, dk_, dv_, dtype=dtype)
    out["dh0"] = torch.zeros(N, H, dk_, dv_, dtype=dtype)
    out["dA_log"] = torch.zeros(H, dtype=dtype)
    out["ddt_bias"] = torch.zeros(H, dk_, dtype=dtype)
    for n, (b, t0, t1) in enumerate(spans):
        for h in range(H):
            sl = (b, slice(t0, t1), h)
            qa, ka, ga, ba, aux = prologue_forward(q[sl], k[sl], g[sl], beta[sl], a_log[h], dt_bias[h], flags)
            s0 = h0[n, h] if h0 is not None else torch.zeros(dk_, dv_, dtype=dtype)
            o, sT, saved = chunk_forward_one(qa, ka, v[sl], ga, ba, s0, scale, chunk)
            dsT = dht[n, h] if dht is not None else torch.zeros(dk_, dv_, dtype=dtype)
            dq, dk, dv, dg, dbeta, dS0 = chunk_backward_one(qa, ka, v[sl], ga, ba, scale, saved, do[sl], dsT)
            dq, dk, dx, dbeta, dA, dbias = prologue_backward(qa, ka, ga, ba, aux, dq, dk, dg, dbeta, a_log[h], flags)
            out["o"][sl], out["dq"][sl], out["dk"][sl], out["dv"][sl] = o, dq, dk, dv
            out["dg"][sl], out["dbeta"][sl] = dx, dbeta
            out["ht"][n, h], out["dh0"][n, h] = sT, dS0
            out["dA_log"][h] += dA
            out["ddt_bias"][h] += dbias
    out["ddt_bias"] = out["ddt_bias"].reshape(-1)
    return out

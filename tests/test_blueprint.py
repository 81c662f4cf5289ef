"""The chunkwise reformulation (what the kernels compute) against autograd through the
recurrent oracle, in FP64."""
import pytest
import torch

from oracle import kda_oracle as O
from oracle.kda_chunk_blueprint import kda_chunk_blueprint


@pytest.mark.parametrize("B,T,H,d,cu,fused", [
    (2, 150, 2, 16, None, True),
    (1, 200, 2, 8, [0, 3, 70, 134, 200], False),
    (1, 64, 1, 32, None, True),
])
def test_blueprint_matches_autograd(B, T, H, d, cu, fused):
    inp = O.make_inputs(B, T, H, d, seed=1, dtype=torch.float64, fused=fused)
    cu_t = None if cu is None else torch.tensor(cu)
    N = B if cu is None else len(cu) - 1
    gen = torch.Generator().manual_seed(2)
    h0 = torch.randn(N, H, d, d, dtype=torch.float64, generator=gen) * 0.1
    dht = torch.randn(N, H, d, d, dtype=torch.float64, generator=gen) * 0.1
    inp["dt_bias"] = torch.randn(H * d, dtype=torch.float64, generator=gen) * 0.3
    kw = dict(a_log=inp["a_log"].double(), dt_bias=inp["dt_bias"], use_qk_l2norm=fused, use_gate=fused,
              use_beta_sigmoid=fused, cu_seqlens=cu_t)
    ref = O.kda_oracle_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["do"], initial_state=h0,
                               dht=dht, dtype=torch.float64, **kw)
    bp = kda_chunk_blueprint(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["do"], h0=h0, dht=dht, **kw)
    for name in ("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dA_log", "ddt_bias", "dh0"):
        if name in ref:
            # the oracle's prologue runs in FP32 like the reference's (model.py:218-222)
            torch.testing.assert_close(bp[name], ref[name].double(), atol=2e-6, rtol=1e-5)

"""Weighted combine (the consumer of inverse_perm / combine_weights): bit-exact
against the CPU oracle, and the dispatch -> combine round trip."""
import numpy as np
import pytest
import torch

import moe_rd
from oracle import cpu_oracle
from moe_rd import workloads
import _util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,T,H,shared", [("c2", 3000, 1024, True), ("c3", 5000, 512, False),
                                             ("c1", 512, 1024, True), ("c3", 32768, 2048, True)])
def test_combine_bit_exact(name, T, H, shared):
    t, kw = workloads.make(name, T=T, H=H)
    kw = dict(kw, gate_impl="simt")
    res = _util.run_gpu(t, kw)
    R = res.permuted.shape[0]
    g = torch.Generator().manual_seed(T)
    y = torch.randn(R, H, generator=g).to(torch.bfloat16)
    sh = torch.randn(T, H, generator=g).to(torch.bfloat16) if shared else None
    out = moe_rd.combine(y.cuda(), res.inverse_perm, res.combine_weights, None if sh is None else sh.cuda())
    torch.cuda.synchronize()
    ref = cpu_oracle.combine(_util.bf16_bits(y), res.inverse_perm.cpu().numpy(), res.combine_weights.cpu().numpy(),
                             None if sh is None else _util.bf16_bits(sh))
    np.testing.assert_array_equal(_util.bf16_bits(out.cpu()), ref)


def test_combine_many_slots():
    g = torch.Generator().manual_seed(5)
    T, K, H, R = 300, 20, 264, 900
    y = torch.randn(R, H, generator=g).to(torch.bfloat16)
    inv = torch.randint(-1, R, (T, K), generator=g, dtype=torch.int32)
    w = torch.rand(T, K, generator=g)
    out = moe_rd.combine(y.cuda(), inv.cuda(), w.cuda())
    ref = cpu_oracle.combine(_util.bf16_bits(y), inv.numpy(), w.numpy())
    np.testing.assert_array_equal(_util.bf16_bits(out.cpu()), ref)


def test_dispatch_then_combine_returns_the_tokens():
    """With renormalised weights (sum 1) and identity experts, combine(dispatch(x)) = x up to bf16 rounding."""
    t, kw = workloads.make("c2", T=4096)
    res = _util.run_gpu(t, kw)
    out = moe_rd.combine(res.permuted, res.inverse_perm, res.combine_weights)
    x = t["x"].cuda().float()
    assert torch.allclose(out.float(), x, rtol=2 ** -7, atol=1e-6)

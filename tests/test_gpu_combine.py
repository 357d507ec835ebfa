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


def _rows_case(T, H, R, seed):
    g = torch.Generator().manual_seed(seed)
    y = torch.randn(R, H, generator=g).to(torch.bfloat16)
    out0 = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w = torch.rand(R, generator=g) * 2 - 0.5
    return g, y, out0, w


@pytest.mark.parametrize("T,H,R,live", [(4096, 1024, 3000, 2500), (700, 264, 700, 700), (512, 7168, 64, 0)])
def test_residual_combine_one_row_per_token_is_bit_exact(T, H, R, live):
    """Every token receives at most one row, so the order of the bf16 adds cannot matter: exact.
    Rows past the device-side count, and rows without a token, must leave ``out`` untouched."""
    g, y, out0, w = _rows_case(T, H, R, 11 + T)
    tok = torch.randperm(T, generator=g)[:R].to(torch.int32)
    tok[::17] = -1
    n = torch.tensor([live], dtype=torch.int32)
    out = out0.clone().cuda()
    got = moe_rd.combine_add_rows(y.cuda(), tok.cuda(), w.cuda(), n.cuda(), out)
    torch.cuda.synchronize()
    assert got.data_ptr() == out.data_ptr()
    ref = cpu_oracle.combine_add_rows(_util.bf16_bits(y), tok.numpy(), w.numpy(), live, _util.bf16_bits(out0))
    np.testing.assert_array_equal(_util.bf16_bits(out.cpu()), ref)
    untouched = np.ones(T, bool)
    untouched[tok[:live][tok[:live] >= 0].numpy()] = False
    np.testing.assert_array_equal(_util.bf16_bits(out.cpu())[untouched], _util.bf16_bits(out0)[untouched])


def test_residual_combine_after_dispatch_within_rounding():
    """All K rows of every token folded in through the forward permutation of a real dispatch.  The
    adds of one token arrive in no fixed order and each rounds to bf16, so the comparison is with the
    fp64 sum, within K + 1 roundings of the running magnitude (2^-8 relative each)."""
    t, kw = workloads.make("c3", T=6000, H=512)
    res = _util.run_gpu(t, dict(kw, gate_impl="simt"), return_row_meta=True)
    R = res.permuted.shape[0]
    T, K = res.inverse_perm.shape
    g = torch.Generator().manual_seed(3)
    y = torch.randn(R, 512, generator=g).to(torch.bfloat16)
    out0 = torch.randn(T, 512, generator=g).to(torch.bfloat16)
    out = out0.clone().cuda()
    moe_rd.combine_add_rows(y.cuda(), res.row_token, res.row_weight, res.offsets[-1:], out)
    torch.cuda.synchronize()
    live = int(res.offsets[-1])
    tok = res.row_token.cpu().numpy()[:live]
    w = res.row_weight.cpu().numpy()[:live].astype(np.float64)
    terms = w[:, None] * y[:live].double().numpy()
    exact = out0.double().numpy().copy()
    mag = np.abs(exact)
    np.add.at(exact, tok, terms)
    np.add.at(mag, tok, np.abs(terms))
    err = np.abs(out.cpu().double().numpy() - exact)
    assert (err <= (K + 1) * 2.0 ** -8 * mag + 1e-30).all(), float((err / (mag + 1e-30)).max())
    # one fixed order (ascending rows) lies inside the same bound
    ref = cpu_oracle.combine_add_rows(_util.bf16_bits(y), res.row_token.cpu().numpy(), res.row_weight.cpu().numpy(),
                                      live, _util.bf16_bits(out0))
    ref_f = torch.from_numpy(ref.view(np.int16).copy()).view(torch.bfloat16).double().numpy()
    assert (np.abs(ref_f - exact) <= (K + 1) * 2.0 ** -8 * mag + 1e-30).all()

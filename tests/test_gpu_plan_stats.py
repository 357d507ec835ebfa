"""Forward permutation, identity-expert shortcut, grouped-GEMM plan and
per-expert statistics against the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

import moe_rd
from oracle import cpu_oracle
from moe_rd import workloads
import _util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,T", [("c1", None), ("c3", 2048), ("c4", 700)])
def test_row_meta_and_expert_stats_match_oracle(name, T):
    t, kw = workloads.make(name, T=T) if T else workloads.make(name)
    dev = torch.device("cuda:0")
    res = moe_rd.route_dispatch(t["x"].to(dev), t["w"].to(dev), None if t["bias"] is None else t["bias"].to(dev),
                                return_row_meta=True, **kw)
    inv = res.inverse_perm.cpu().numpy()
    wts = res.combine_weights.cpu().numpy()
    offs = res.offsets.cpu().numpy()
    kept = int(offs[-1])
    tok_ref, w_ref = cpu_oracle.row_meta(inv, wts, res.row_token.numel())
    np.testing.assert_array_equal(res.row_token.cpu().numpy()[:kept], tok_ref[:kept])
    np.testing.assert_array_equal(res.row_weight.cpu().numpy()[:kept].view(np.uint32), w_ref[:kept].view(np.uint32))
    # rows of an expert are in token order (stable)
    rt = res.row_token.cpu().numpy()
    for e in range(offs.size - 1):
        seg = rt[offs[e]:offs[e + 1]]
        assert np.all(np.diff(seg) > 0)

    st = moe_rd.expert_stats(res.offsets, res.row_weight)
    ws, mw, ld = cpu_oracle.expert_stats(offs, w_ref)
    np.testing.assert_array_equal(st.weight_sum.cpu().numpy().view(np.uint32), ws.view(np.uint32))
    np.testing.assert_array_equal(st.mean_weight.cpu().numpy().view(np.uint32), mw.view(np.uint32))
    np.testing.assert_array_equal(st.load.cpu().numpy().view(np.uint32), ld.view(np.uint32))
    st2 = moe_rd.expert_stats(res.offsets, res.row_weight)
    assert torch.equal(st.weight_sum, st2.weight_sum)


def _bias_dominated(T=600, H=256, E=16, K=4, seed=5):
    """Two experts get a large selection bias, so every token picks both."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(H, E, generator=g) * 0.02).to(torch.bfloat16)
    bias = torch.zeros(E)
    bias[3] = 5.0
    bias[11] = 4.0
    return x, w, bias, dict(top_k=K, score_fn="softmax", bias_mode="select")


def test_identity_experts_are_skipped_and_planned_onto_x():
    x, w, bias, kw = _bias_dominated()
    dev = torch.device("cuda:0")
    xd, wd, bd = x.to(dev), w.to(dev), bias.to(dev)
    full = moe_rd.route_dispatch(xd, wd, bd, **kw)
    T, H = x.shape
    E = w.shape[1]
    # sentinel-filled output: rows of identity experts must stay untouched
    sk = moe_rd.route_dispatch(xd, wd, bd, skip_identity_rows=True, **kw)
    offs = full.offsets.cpu().numpy()
    assert torch.equal(full.offsets, sk.offsets) and torch.equal(full.inverse_perm, sk.inverse_perm)
    cnt = np.diff(offs)
    dense = [e for e in range(E) if cnt[e] == T]
    assert dense == [3, 11]
    fp = full.permuted.cpu().view(torch.int16).numpy()
    sp = sk.permuted.cpu().view(torch.int16).numpy()
    xb = x.view(torch.int16).numpy()
    for e in range(E):
        lo, hi = offs[e], offs[e + 1]
        if e in dense:
            np.testing.assert_array_equal(fp[lo:hi], xb)  # the full copy IS x, in token order
        else:
            np.testing.assert_array_equal(sp[lo:hi], fp[lo:hi])

    # the plan aims identity experts at x
    N = 64
    ew = torch.zeros(E, N, H, dtype=torch.bfloat16, device=dev)
    out = torch.empty(T * kw["top_k"], N, dtype=torch.bfloat16, device=dev)
    plan = moe_rd.decode_gemm_plan(moe_rd.gemm_plan(sk.offsets, sk.permuted, ew, out, identity_source=xd))
    ref = cpu_oracle.gemm_plan(offs, sk.permuted.data_ptr(), H * 2, ew.data_ptr(), N * H * 2, out.data_ptr(), N * 2,
                               N, H, ident_base=xd.data_ptr(), ident_m=T)
    for g, r in zip(plan, ref):
        assert (g.m, g.n, g.k, g.identity) == (r["m"], r["n"], r["k"], r["identity"])
        assert (g.a or 0, g.b or 0, g.d or 0) == (r["a"], r["b"], r["d"])
        assert (g.lda, g.ldb, g.ldd) == (H * 2, N * H * 2, N * 2)
    assert [g.identity for g in plan] == [1 if e in dense else 0 for e in range(E)]

    # a ragged GEMM driven by the plan gives the same result from either buffer
    def run(planned, a_full):
        ys = []
        for e, g in enumerate(planned):
            a = xd if g.identity else a_full[offs[e]:offs[e + 1]]
            ys.append(a.float().sum(dim=1))
        return torch.cat(ys)
    assert torch.equal(run(plan, sk.permuted), run(plan, full.permuted))


def test_gemm_plan_without_identity_and_flag_validation():
    t, kw = workloads.make("c1")
    dev = torch.device("cuda:0")
    res = moe_rd.route_dispatch(t["x"].to(dev), t["w"].to(dev), None, **kw)
    E = res.offsets.numel() - 1
    H = t["x"].shape[1]
    ew = torch.zeros(E, 32, H, dtype=torch.bfloat16, device=dev)
    out = torch.empty(res.permuted.shape[0], 32, dtype=torch.bfloat16, device=dev)
    plan = moe_rd.decode_gemm_plan(moe_rd.gemm_plan(res.offsets, res.permuted, ew, out))
    offs = res.offsets.cpu().numpy()
    assert [g.m for g in plan] == list(np.diff(offs))
    assert all(g.identity == 0 for g in plan)
    assert [(g.a or 0) for g in plan] == [res.permuted.data_ptr() + int(o) * H * 2 for o in offs[:-1]]
    with pytest.raises(moe_rd.MoeRdError):  # the shortcut is defined for bf16 rows only
        t4, kw4 = workloads.make("c4", T=256)
        moe_rd.route_dispatch(t4["x"].to(dev), t4["w"].to(dev), t4["bias"].to(dev), skip_identity_rows=True, **kw4)

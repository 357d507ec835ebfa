"""Parity of the CUDA path (through the C ABI) with the CPU oracle.

Bit-exact: expert ids, counts, offsets, inverse permutation, drop mask, bf16
row copies, fp8 bytes and fp8 scales.  Combine weights: tolerance 1e-6 relative
(fp32); where the gate product runs in the fixed order they are also compared
bit for bit.
"""
import numpy as np
import pytest
import torch

from moe_rd import workloads
import _util

pytestmark = pytest.mark.gpu

WEIGHT_RTOL = 1e-6


def check(tensors, kw, *, exact_weights=True, **extra):
    res = _util.run_gpu(tensors, kw, **extra)
    got = _util.to_np(res)
    ref = _util.run_oracle(tensors, kw)
    _util.assert_parity(got, ref, weight_rtol=WEIGHT_RTOL, exact_weights=exact_weights)
    return got, ref


# ----------------------------------------------------- the five workloads --
def test_c1_full_size():
    t, kw = workloads.make("c1")
    got, ref = check(t, kw, gate_impl="simt", return_logits=True)
    np.testing.assert_array_equal(got["router_logits"].view(np.uint32), ref["logits"].view(np.uint32))
    assert got["permuted"].shape == (1024, 1024) and got["offsets"].shape == (9,)
    assert got["inverse_perm"].shape == (512, 2) and got["combine_weights"].shape == (512, 2)


def test_c2_full_size():
    t, kw = workloads.make("c2")
    check(t, kw, gate_impl="simt")


@pytest.mark.parametrize("name,T,H", [("c1", None, None), ("c2", None, None), ("c2", 1000, 1096), ("c1", 33, 264)])
def test_fused_gemv_gate_matches_oracle_bit_for_bit(name, T, H):
    """E <= 32: the default path is the warp GEMV fused with routing; its logits
    follow the same fixed order, so even the logits are bit-exact."""
    t, kw = workloads.make(name, T=T, H=H)
    got, ref = check(t, kw, gate_impl="gemv", return_logits=True)
    np.testing.assert_array_equal(got["router_logits"].view(np.uint32), ref["logits"].view(np.uint32))
    check(t, kw)  # auto picks the same kernel


@pytest.mark.parametrize("E,wdt,layout", [(5, torch.float32, "HE"), (13, torch.bfloat16, "EH"), (16, torch.bfloat16, "HE"),
                                          (24, torch.float32, "EH"), (32, torch.bfloat16, "HE")])
def test_fused_gemv_expert_counts_and_layouts(E, wdt, layout):
    g = torch.Generator().manual_seed(E)
    T, H = 500, 520
    w = (torch.randn(H, E, generator=g) * 0.1).to(wdt)
    t = dict(x=torch.randn(T, H, generator=g).to(torch.bfloat16), w=w, bias=torch.randn(E, generator=g) * 0.1)
    kw = dict(top_k=min(4, E), bias_mode="logit", score_fn="softmax")
    ref = _util.run_oracle(t, kw)
    if layout == "EH":
        t = dict(t, w=w.t().contiguous())
        kw = dict(kw, w_layout="EH")
    for impl in ("gemv", "simt"):
        got = _util.to_np(_util.run_gpu(t, kw, gate_impl=impl, return_logits=True))
        _util.assert_parity(got, ref)
        np.testing.assert_array_equal(got["router_logits"].view(np.uint32), ref["logits"].view(np.uint32))


def test_c3_full_size_with_capacity_drops():
    t, kw = workloads.make("c3")
    got, ref = check(t, kw, gate_impl="simt")
    assert ref["drop_mask"].sum() > 0 and kw["capacity"] == 2560
    assert got["offsets"][-1] == ref["offsets"][-1] < 32768 * 8


def test_c4_full_size_group_limited_fp8():
    t, kw = workloads.make("c4")
    check(t, kw, gate_impl="simt")


@pytest.mark.parametrize("name,T,H", [("c2", 640, 1024), ("c3", 1500, 512), ("c4", 333, 1024),
                                      ("c1", 1, 1024), ("c3", 129, 256), ("c4", 127, 128)])
def test_ragged_sizes(name, T, H):
    t, kw = workloads.make(name, T=T, H=H)
    check(t, kw, gate_impl="simt")


def test_empty_input():
    t, kw = workloads.make("c1", T=0)
    res = _util.run_gpu(t, kw)
    assert res.offsets.cpu().tolist() == [0] * 9
    assert res.inverse_perm.shape == (0, 2) and res.permuted.shape[0] == 0


# ------------------------------------------------------------ option grid --
def test_weight_layout_and_dtype_variants_agree():
    t, kw = workloads.make("c1", T=300)
    base, _ = check(t, kw, gate_impl="simt", return_logits=True)
    for wdt in (torch.float32, torch.bfloat16):
        tt = dict(t)
        tt["w"] = t["w"].to(wdt)
        a, _ = check(tt, kw, gate_impl="simt", return_logits=True)
        tt_eh = dict(tt)
        tt_eh["w"] = tt["w"].t().contiguous()
        kw_eh = dict(kw, w_layout="EH")
        res = _util.to_np(_util.run_gpu(tt_eh, kw_eh, gate_impl="simt", return_logits=True))
        np.testing.assert_array_equal(res["router_logits"].view(np.uint32), a["router_logits"].view(np.uint32))
        np.testing.assert_array_equal(res["inverse_perm"], a["inverse_perm"])


def test_odd_expert_count_scalar_weight_path():
    g = torch.Generator().manual_seed(2)
    T, H, E = 200, 264, 13
    t = dict(x=torch.randn(T, H, generator=g).to(torch.bfloat16), w=torch.randn(H, E, generator=g) * 0.1,
             bias=torch.randn(E, generator=g) * 0.1)
    for mode in ("logit", "select", "select_and_weight"):
        check(t, dict(top_k=3, bias_mode=mode), gate_impl="simt")
    check(t, dict(top_k=13, renorm=False, score_fn="sigmoid"), gate_impl="simt")


@pytest.mark.parametrize("case", [
    dict(E=64, K=6, score_fn="sigmoid", n_groups=8, topk_groups=3, group_topk=2, routed_scale=2.5),
    dict(E=96, K=4, score_fn="sigmoid", n_groups=4, topk_groups=2, group_topk=3),
    dict(E=128, K=8, score_fn="softmax", n_groups=2, topk_groups=1, group_topk=1),
    dict(E=256, K=32, score_fn="softmax"),
    dict(E=32, K=1, score_fn="softmax", renorm=False),
    dict(E=160, K=12, score_fn="softmax", n_groups=5, topk_groups=2, group_topk=4),
    dict(E=72, K=3, score_fn="sigmoid", n_groups=8, topk_groups=5, group_topk=1),
])
def test_routing_modes_on_given_logits_with_ties(case):
    """Logits are supplied, so only scoring/selection/dispatch run; rows of
    equal logits exercise the lowest-index tie-break and the group limit."""
    E, K = case["E"], case["K"]
    g = torch.Generator().manual_seed(E + K)
    T, H = 700, 128
    z = torch.randn(T, E, generator=g)
    z[3] = 0.25
    z[4, : E // 2] = 1.5
    z[5:200] = torch.round(z[5:200] * 2) / 2
    z[200:260] = 0.0
    z[200:260, 7] = 9.0  # everything to one expert first
    bias = torch.rand(E, generator=g) * 0.2 - 0.1
    kw = {k: v for k, v in case.items() if k not in ("E", "K")}
    kw.update(top_k=K, bias_mode="select")
    t = dict(x=torch.randn(T, H, generator=g).to(torch.bfloat16), w=None, bias=bias)
    res = _util.to_np(_util.run_gpu(t, kw, given_logits=z))
    ref = _util.run_oracle(t, kw, given_logits=z.numpy())
    _util.assert_parity(res, ref)


def test_all_tokens_to_one_expert_and_empty_experts_with_capacity():
    T, H, E = 1000, 256, 16
    g = torch.Generator().manual_seed(9)
    z = torch.full((T, E), -5.0)
    z[:, 3] = 5.0
    z[:, 11] = 4.0
    t = dict(x=torch.randn(T, H, generator=g).to(torch.bfloat16), w=None, bias=None)
    for cap, fmt in ((0, "bf16"), (100, "bf16"), (1, "fp8"), (2000, "fp8")):
        kw = dict(top_k=2, capacity=cap, rows_format=fmt)
        res = _util.to_np(_util.run_gpu(t, kw, given_logits=z))
        ref = _util.run_oracle(t, kw, given_logits=z.numpy())
        _util.assert_parity(res, ref)
        kept = T if cap == 0 else min(T, cap)
        assert res["offsets"].tolist() == [0] * 4 + [kept] * 8 + [2 * kept] * 5


def test_fp8_extreme_values():
    T, H = 64, 256
    g = torch.Generator().manual_seed(4)
    x = torch.randn(T, H, generator=g)
    x[0] = 0.0
    x[1, :128] = 0.0
    x[2] *= 1e-20
    x[3] *= 3e4
    x[4, 5] = 448.0
    x[5] = torch.round(x[5] * 8) / 8
    t = dict(x=x.to(torch.bfloat16), w=torch.randn(H, 8, generator=g) * 0.1, bias=None)
    check(t, dict(top_k=2, rows_format="fp8"), gate_impl="simt")


def test_run_twice_is_bit_identical():
    t, kw = workloads.make("c3", T=5000)
    a = _util.to_np(_util.run_gpu(t, kw, gate_impl="simt"))
    b = _util.to_np(_util.run_gpu(t, kw, gate_impl="simt"))
    for k in ("expert_ids", "offsets", "inverse_perm", "combine_weights", "drop_mask", "counts"):
        np.testing.assert_array_equal(a[k], b[k])
    R = int(a["offsets"][-1])
    np.testing.assert_array_equal(a["permuted"][:R], b["permuted"][:R])


def test_device_status_stays_clean_and_launches_are_counted():
    import ctypes
    from moe_rd import _cabi
    before = _cabi.launch_count()
    t, kw = workloads.make("c1")
    _util.run_gpu(t, kw)
    assert _cabi.launch_count() - before >= 3  # fused gate+route (scans in its last block), positions, scatter


def test_round_trip_property_at_full_size():
    """Size-independent property on the full c2 problem: every kept pair's row
    equals its token's row, and offsets partition [0, R)."""
    t, kw = workloads.make("c2")
    res = _util.run_gpu(t, kw)
    x = t["x"].cuda()
    inv = res.inverse_perm.long()
    for k in range(inv.shape[1]):
        assert torch.equal(res.permuted[inv[:, k]], x)
    ids = res.expert_ids.long()
    offs = res.offsets.long()
    assert bool(((inv >= offs[ids]) & (inv < offs[ids + 1])).all())
    assert int(offs[-1]) == inv.numel()
    assert torch.equal(torch.sort(inv.reshape(-1)).values, torch.arange(inv.numel(), device="cuda"))


@pytest.mark.parametrize("name,T,H", [("c2", None, None), ("c3", None, None), ("c4", None, None), ("c1", 37, 1024),
                                      ("c3", 1500, 512), ("c4", 333, 1024), ("c2", 1, 4096)])
def test_bulk_copy_scatter_matches_oracle(name, T, H):
    """The shared-memory / bulk-copy scatter must produce the same bytes as the
    plain one (and as the oracle), including capacity drops and fp8 scales."""
    t, kw = workloads.make(name, T=T, H=H)
    check(t, kw, gate_impl="simt", scatter_impl="bulk")

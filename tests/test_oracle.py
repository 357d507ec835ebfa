"""CPU tests of the oracle itself: the C restatement against independent
numpy/Python restatements of the same definitions, against torch's e4m3 cast,
against the committed golden fixtures, and the structural invariants of the
dispatch (bijection, monotone offsets, stable order, tail drops)."""
import hashlib
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import cpu_oracle
from moe_rd import workloads
import _util

GOLDEN = Path(__file__).resolve().parent / "golden"


def f32(a):
    return np.asarray(a, dtype=np.float32)


def bf16_to_f32_np(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------- numerics --
def test_expf_close_to_libm():
    L = cpu_oracle.lib()
    xs = np.concatenate([np.linspace(-87, 10, 20001), np.linspace(-1, 1, 2001)]).astype(np.float32)
    worst = 0.0
    for v in xs:
        got = L.moe_oracle_expf(float(v))
        ref = math.exp(float(v))
        worst = max(worst, abs(got - ref) / ref)
    assert worst < 2.5 * 2 ** -24
    assert L.moe_oracle_expf(-100.0) == 0.0
    assert L.moe_oracle_expf(0.0) == 1.0
    assert math.isinf(L.moe_oracle_expf(89.0))


def test_e4m3_matches_torch_cast_on_finite_range():
    L = cpu_oracle.lib()
    # every bf16 value with |v| <= 448 plus a dense fp32 sweep
    allb = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    vals = bf16_to_f32_np(allb)
    vals = vals[np.isfinite(vals) & (np.abs(vals) <= 448.0)]
    rng = np.random.default_rng(0)
    vals = np.concatenate([vals, rng.uniform(-448, 448, 20000).astype(np.float32),
                           (rng.standard_normal(20000) * 0.01).astype(np.float32)])
    ref = torch.from_numpy(vals).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([L.moe_oracle_f32_to_e4m3(float(v)) for v in vals], dtype=np.uint8)
    # -0.0 and +0.0 keep their sign in both
    np.testing.assert_array_equal(got, ref)
    # saturation instead of NaN above the finite range
    assert L.moe_oracle_f32_to_e4m3(1e9) == 0x7E and L.moe_oracle_f32_to_e4m3(-470.0) == 0xFE
    for b in range(256):
        v = L.moe_oracle_e4m3_to_f32(b)
        if not math.isnan(v):
            assert L.moe_oracle_f32_to_e4m3(v) == b or (v == 0.0)


def _logits_py(x_u16, w_f32, logit_bias=None):
    """Independent restatement of the fixed summation order (32 lanes x 2
    chains, then a tree) with float64 emulation of the fused multiply-add
    (products of a bf16 and an fp32 value are exact in float64; the sum is
    rounded once to fp32)."""
    T, H = x_u16.shape
    E = w_f32.shape[1]
    xf = bf16_to_f32_np(x_u16).astype(np.float64)
    wd = w_f32.astype(np.float64)
    z = np.zeros((T, E), np.float32)
    for t in range(T):
        acc = np.zeros((32, 2, E), np.float32)  # chain (lane, parity of h)
        for c in range((H + 255) // 256):
            for j in range(8):
                hs = c * 256 + np.arange(32) * 8 + j
                ok = hs < H
                prod = xf[t, hs[ok]][:, None] * wd[hs[ok], :]
                acc[ok, j & 1] = (prod + acc[ok, j & 1].astype(np.float64)).astype(np.float32)
        lane = acc[:, 0] + acc[:, 1]
        off = 16
        while off:
            lane[:off] = lane[:off] + lane[off:2 * off]
            off //= 2
        z[t] = lane[0] + logit_bias if logit_bias is not None else lane[0]
    return z


@pytest.mark.parametrize("H,E,wdt", [(1024, 8, "f32"), (384, 5, "bf16"), (72, 16, "f32")])
def test_logits_fixed_order_matches_python_restatement(H, E, wdt):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(9, H, generator=g).to(torch.bfloat16)
    w = torch.randn(H, E, generator=g) * 0.05
    lb = torch.randn(E, generator=g).numpy()
    if wdt == "bf16":
        wb = w.to(torch.bfloat16)
        w_or, w_f = _util.bf16_bits(wb), wb.float().numpy()
    else:
        w_or, w_f = w.numpy(), w.numpy()
    xb = _util.bf16_bits(x)
    ref = _logits_py(xb, w_f, lb)
    got = cpu_oracle.logits(xb, w_or, logit_bias=lb)
    np.testing.assert_array_equal(got.view(np.uint32), ref.view(np.uint32))
    # [E,H] layout holds the same numbers
    w_eh = np.ascontiguousarray(w_or.T)
    got2 = cpu_oracle.logits(xb, w_eh, w_layout="EH", logit_bias=lb)
    np.testing.assert_array_equal(got2.view(np.uint32), ref.view(np.uint32))
    # and is close to the double-precision product
    z64 = cpu_oracle.logits(xb, w_or, logit_bias=lb, f64=True)
    assert np.max(np.abs(got - z64)) < 1e-4


def _route_py(z, K, score_fn, sb, G, topk_groups, group_topk, weight_from_key, renorm, scale, norm_min):
    """Independent (slow) restatement with numpy float32 scalars."""
    L = cpu_oracle.lib()
    T, E = z.shape
    ids = np.zeros((T, K), np.int32)
    wts = np.zeros((T, K), np.float32)
    one = np.float32(1)
    for t in range(T):
        zr = z[t]
        if score_fn == "softmax":
            m = zr.max()
            p = np.array([L.moe_oracle_expf(float(np.float32(v - m))) for v in zr], np.float32)
            part = np.zeros(32, np.float32)
            for e in range(E):
                part[e % 32] = part[e % 32] + p[e]
            off = 16
            while off:
                part[:off] = part[:off] + part[off:2 * off]
                off //= 2
            sc = p * (one / part[0])
        else:
            sc = np.array([one / (one + np.float32(L.moe_oracle_expf(float(-v)))) for v in zr], np.float32)
        key = sc + sb if sb is not None else sc.copy()
        elig = np.ones(E, bool)
        if G > 1:
            gs = E // G
            gscore = []
            for g in range(G):
                top = np.sort(key[g * gs:(g + 1) * gs])[::-1][:group_topk]
                s = top[0]
                for v in top[1:]:
                    s = np.float32(s + v)
                gscore.append(s)
            order = sorted(range(G), key=lambda g: (-gscore[g], g))
            for g in order[topk_groups:]:
                elig[g * gs:(g + 1) * gs] = False
        cand = sorted([e for e in range(E) if elig[e]], key=lambda e: (-key[e], e))[:K]
        u = np.array([key[e] if weight_from_key else sc[e] for e in cand], np.float32)
        tot = np.float32(0)
        for v in u:
            tot = np.float32(tot + v)
        w = u / max(tot, np.float32(norm_min)) if renorm else u
        ids[t] = cand
        wts[t] = w.astype(np.float32) * np.float32(scale)
    return ids, wts


@pytest.mark.parametrize("case", [
    dict(E=8, K=2, score_fn="softmax"),
    dict(E=128, K=8, score_fn="softmax", bias=True, weight_from_key=True),
    dict(E=64, K=6, score_fn="sigmoid", bias=True, G=8, topk_groups=3, group_topk=2, scale=2.5),
    dict(E=256, K=8, score_fn="sigmoid", bias=True, G=8, topk_groups=4, group_topk=2, scale=2.5),
    dict(E=20, K=20, score_fn="softmax", renorm=False),
    dict(E=96, K=4, score_fn="sigmoid", G=4, topk_groups=2, group_topk=3),
])
def test_route_matches_python_restatement(case):
    E, K = case["E"], case["K"]
    g = torch.Generator().manual_seed(E * 131 + K)
    z = torch.randn(24, E, generator=g).numpy()
    z[3] = 0.25          # all keys tie: lowest indices must win
    z[4, : E // 2] = 1.5  # a block of ties
    z[5] = np.round(z[5] * 2) / 2  # many pairwise ties
    sb = (torch.rand(E, generator=g) * 0.2 - 0.1).numpy() if case.get("bias") else None
    kw = dict(top_k=K, score_fn=case["score_fn"], select_bias=sb, n_groups=case.get("G", 1),
              topk_groups=case.get("topk_groups", 1), group_topk=case.get("group_topk", 1),
              weight_from_key=case.get("weight_from_key", False), renorm=case.get("renorm", True),
              routed_scale=case.get("scale", 1.0), norm_min=1e-20)
    ids, wts = cpu_oracle.route(z, **kw)
    rid, rw = _route_py(z, K, case["score_fn"], sb, kw["n_groups"], kw["topk_groups"], kw["group_topk"],
                        kw["weight_from_key"], kw["renorm"], kw["routed_scale"], 1e-20)
    np.testing.assert_array_equal(ids, rid)
    np.testing.assert_array_equal(wts.view(np.uint32), rw.view(np.uint32))
    if not case.get("bias") and case.get("G", 1) == 1:
        assert list(ids[3]) == list(range(K))


def test_route_rejects_bad_groups():
    z = np.zeros((2, 12), np.float32)
    with pytest.raises(ValueError):
        cpu_oracle.route(z, top_k=2, n_groups=5)
    with pytest.raises(ValueError):
        cpu_oracle.route(z, top_k=7, n_groups=4, topk_groups=2, group_topk=1)


# ---------------------------------------------------------------- dispatch --
@pytest.mark.parametrize("T,K,E,cap", [(0, 2, 8, 0), (1, 1, 1, 0), (300, 4, 16, 0), (300, 4, 16, 50),
                                        (257, 8, 128, 3), (64, 2, 8, 1)])
def test_dispatch_invariants(T, K, E, cap):
    rng = np.random.default_rng(T + K + E)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32) if T else np.zeros((0, K), np.int32)
    if T > 10:
        ids[:, 0] = 0  # a hot expert
    counts, offsets, inv, drop = cpu_oracle.dispatch(ids, E, cap)
    assert offsets[0] == 0 and np.all(np.diff(offsets) >= 0)
    np.testing.assert_array_equal(counts, np.bincount(ids.ravel(), minlength=E))
    kept = np.minimum(counts, cap) if cap else counts
    np.testing.assert_array_equal(np.diff(offsets), kept)
    flat, fi = inv.ravel(), ids.ravel()
    keep = flat >= 0
    np.testing.assert_array_equal(drop.ravel(), (~keep).astype(np.uint8))
    # bijection onto [0, offsets[E])
    assert sorted(flat[keep]) == list(range(offsets[E]))
    # every kept pair lies in its expert's segment, in stable (token, slot) order
    for e in range(E):
        sel = np.nonzero(fi == e)[0]
        pos = flat[sel]
        k = int(kept[e])
        np.testing.assert_array_equal(pos[:k], offsets[e] + np.arange(k))
        assert np.all(pos[k:] == -1)  # drops are exactly the tail in token order


def test_permute_bf16_and_fp8():
    g = torch.Generator().manual_seed(11)
    T, H, K, E = 37, 256, 3, 8
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    x[5, :128] = 0  # an all-zero scale block
    x[6, 3] = 300.0
    xb = _util.bf16_bits(x)
    rng = np.random.default_rng(1)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    _, offsets, inv, _ = cpu_oracle.dispatch(ids, E, 10)
    rows, _ = cpu_oracle.permute(xb, inv)
    for t in range(T):
        for k in range(K):
            if inv[t, k] >= 0:
                np.testing.assert_array_equal(rows[inv[t, k]], xb[t])
    q, sc = cpu_oracle.permute(xb, inv, quant="fp8")
    xf = x.float().numpy()
    for t in range(T):
        am = np.abs(xf[t].reshape(-1, 128)).max(axis=1)
        s_ref = np.maximum(am, np.float32(1e-30)) * (np.float32(1.0) / np.float32(448.0))
        qt = (torch.from_numpy(xf[t].reshape(-1, 128) * (np.float32(1) / s_ref)[:, None])
              .clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy().reshape(-1))
        for k in range(K):
            if inv[t, k] >= 0:
                np.testing.assert_array_equal(sc[inv[t, k]].view(np.uint32), s_ref.astype(np.float32).view(np.uint32))
                np.testing.assert_array_equal(q[inv[t, k]], qt)


def test_ep_exchange_equals_global_routing():
    """Routing W ranks separately and exchanging equals, per owner and expert,
    the concatenation in (rank, token) order of what each rank dispatched."""
    W, E = 4, 16
    per_rank = []
    for r in range(W):
        t, kw = workloads.make("c1", T=50 + r, H=128, rank=r)
        g = torch.Generator().manual_seed(5)
        t["w"] = (torch.randn(128, E, generator=g) * 0.1)
        per_rank.append(_util.run_oracle(t, kw))
    out = cpu_oracle.ep_exchange(per_rank, E, W)
    epr = E // W
    for d in range(W):
        tot = 0
        for le in range(epr):
            e = d * epr + le
            for s in range(W):
                o = per_rank[s]["offsets"]
                n = o[e + 1] - o[e]
                np.testing.assert_array_equal(out[d]["rows"][tot:tot + n], per_rank[s]["permuted"][o[e]:o[e + 1]])
                tot += n
            assert out[d]["offsets"][le + 1] == tot
        assert out[d]["rows"].shape[0] == tot


# ------------------------------------------------------------------ golden --
def _digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("name", ["c1", "c2_small", "c3_small", "c4_small"])
def test_golden_fixture(name):
    """Fixtures written by tests/golden/make_golden.py.  The reference project
    has no vectors for this path; these pin the oracle against regressions and
    against drift of the seeded input generator."""
    meta = json.loads((GOLDEN / f"{name}.json").read_text())
    data = np.load(GOLDEN / f"{name}.npz")
    t, kw = workloads.make(meta["workload"], T=meta["T"], H=meta["H"])
    assert _digest(_util.bf16_bits(t["x"])) == meta["x_sha256"], "seeded input generator drifted"
    r = _util.run_oracle(t, kw)
    np.testing.assert_array_equal(r["expert_ids"], data["expert_ids"])
    np.testing.assert_array_equal(r["offsets"], data["offsets"])
    np.testing.assert_array_equal(r["inverse_perm"], data["inverse_perm"])
    np.testing.assert_array_equal(r["combine_weights"].view(np.uint32), data["combine_weights"].view(np.uint32))
    assert _digest(r["permuted"]) == meta["permuted_sha256"]
    if r["scales"] is not None:
        assert _digest(r["scales"]) == meta["scales_sha256"]


def test_combine_matches_numpy_restatement():
    g = torch.Generator().manual_seed(21)
    T, K, H, R = 40, 3, 64, 100
    y = torch.randn(R, H, generator=g).to(torch.bfloat16)
    sh = torch.randn(T, H, generator=g).to(torch.bfloat16)
    rng = np.random.default_rng(3)
    inv = rng.integers(-1, R, size=(T, K)).astype(np.int32)
    w = rng.random((T, K)).astype(np.float32)
    yb, sb = _util.bf16_bits(y), _util.bf16_bits(sh)
    for shared in (None, sb):
        got = cpu_oracle.combine(yb, inv, w, shared)
        yf = y.float().numpy().astype(np.float64)
        acc = (sh.float().numpy() if shared is not None else np.zeros((T, H), np.float32)).astype(np.float32)
        for k in range(K):
            sel = inv[:, k] >= 0
            prod = w[sel, k].astype(np.float64)[:, None] * yf[inv[sel, k]]
            acc[sel] = (prod + acc[sel].astype(np.float64)).astype(np.float32)  # one fused multiply-add
        ref = torch.from_numpy(acc).to(torch.bfloat16)
        np.testing.assert_array_equal(got, _util.bf16_bits(ref))


def _bf16_nearest_even(s):
    """float64 -> bf16 bits, one rounding, by comparing with the two neighbouring bf16 values."""
    f = s.astype(np.float32)
    lo_bits = f.view(np.uint32) & np.uint32(0xffff0000)          # toward zero
    hi_bits = lo_bits + np.uint32(0x10000)                        # away from zero
    lo = lo_bits.view(np.float32).astype(np.float64)
    hi = hi_bits.view(np.float32).astype(np.float64)
    dl, dh = np.abs(s - lo), np.abs(hi - s)
    up = (dh < dl) | ((dh == dl) & (((lo_bits >> 16) & 1) == 1))
    return np.where(up, hi_bits >> 16, lo_bits >> 16).astype(np.uint16)


def test_residual_combine_matches_numpy_restatement():
    g = torch.Generator().manual_seed(22)
    T, H, R, live = 50, 72, 120, 97
    y = torch.randn(R, H, generator=g).to(torch.bfloat16)
    out0 = (torch.randn(T, H, generator=g) * 3).to(torch.bfloat16)
    rng = np.random.default_rng(4)
    tok = rng.integers(-1, T, size=R).astype(np.int32)              # several rows per token, some without one
    w = (rng.random(R) * 2 - 0.5).astype(np.float32)
    got = cpu_oracle.combine_add_rows(_util.bf16_bits(y), tok, w, live, _util.bf16_bits(out0))
    ref = out0.float().numpy().astype(np.float64)
    yf = y.float().numpy()
    for p in range(live):                                           # ascending rows, one bf16 add each
        if tok[p] < 0:
            continue
        term = torch.from_numpy(w[p] * yf[p]).to(torch.bfloat16).float().numpy().astype(np.float64)
        bits = _bf16_nearest_even(ref[tok[p]] + term)
        ref[tok[p]] = (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    np.testing.assert_array_equal(got, _bf16_nearest_even(ref))
    # rows past the live count and tokens nobody points at are untouched
    hit = np.zeros(T, bool)
    hit[tok[:live][tok[:live] >= 0]] = True
    np.testing.assert_array_equal(got[~hit], _util.bf16_bits(out0)[~hit])


def test_send_once_marks_on_a_hand_checked_case():
    """2 ranks, 8 experts (0-3 on rank 0, 4-7 on rank 1), 2 tokens per rank, top-3: worked out by hand."""
    def routed(ids):
        ids = np.array(ids, np.int32)
        T, K = ids.shape
        flat = ids.flatten()
        order = np.argsort(flat, kind="stable")
        offs = np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=8))]).astype(np.int32)
        inv = np.empty(T * K, np.int32)
        inv[order] = np.arange(T * K)
        return dict(expert_ids=ids, inverse_perm=inv.reshape(T, K), offsets=offs)
    per = [routed([[0, 4, 5], [6, 7, 1]]), routed([[0, 1, 2], [4, 3, 0]])]
    m0, m1 = cpu_oracle.ep_send_once_marks(per, 8, 2, 8)
    # rank 0's buffer: expert 0 rows [s0 t0 | s1 t0, s1 t1], expert 1 [s0 t1 | s1 t0], expert 2 [s1 t0], expert 3 [s1 t1]
    # source 1, token 0 has experts 0,1,2 here: rows 1 (sent), 4 and 5 (marks -> 1); token 1 has 3 then 0: row 6 sent, row 2 marked
    np.testing.assert_array_equal(m0, [-1, -1, 6, -1, 1, 1, -1, -1])
    # rank 1's buffer: expert 4 [s0 t0 | s1 t1], 5 [s0 t0], 6 [s0 t1], 7 [s0 t1]; source 0: token 0 rows 0 (sent), 2; token 1 rows 3 (sent), 4
    np.testing.assert_array_equal(m1, [-1, -1, 0, -1, 3, -1, -1, -1])


def test_row_meta_expert_stats_and_plan_restatements():
    inv = np.array([[2, 0], [-1, 1], [3, 4]], dtype=np.int32)
    w = np.array([[0.5, 0.25], [0.125, 1.0], [2.0, 4.0]], dtype=np.float32)
    tok, wt = cpu_oracle.row_meta(inv, w, 6)
    assert list(tok) == [0, 1, 0, 2, 2, -1]
    assert list(wt) == [0.25, 1.0, 0.5, 2.0, 4.0, 0.0]
    offs = np.array([0, 2, 2, 5], dtype=np.int32)
    ws, mw, ld = cpu_oracle.expert_stats(offs, wt)
    assert list(ws) == [1.25, 0.0, 6.5] and list(mw) == [0.625, 0.0, np.float32(6.5) / np.float32(3)]
    assert np.allclose(ld, [0.4, 0.0, 0.6])
    # order: 600 equal tiny weights next to a large one do not depend on numpy's pairwise sum
    big = np.concatenate([[1e8], np.full(599, 1.0)]).astype(np.float32)
    s, _, _ = cpu_oracle.expert_stats(np.array([0, 600]), big)
    part = np.zeros(256, dtype=np.float32)
    for i, v in enumerate(big):
        part[i % 256] = np.float32(part[i % 256] + v)
    off = 128
    while off:
        part[:off] = part[:off] + part[off:2 * off]
        off >>= 1
    assert s[0] == part[0]
    plan = cpu_oracle.gemm_plan(offs, 1000, 16, 5000, 64, 9000, 8, n=4, k=8, ident_base=77, ident_m=3)
    assert [g["m"] for g in plan] == [2, 0, 3]
    assert plan[0]["a"] == 1000 and plan[2]["a"] == 77 and plan[2]["identity"] == 1
    assert plan[2]["b"] == 5000 + 2 * 64 and plan[2]["d"] == 9000 + 2 * 8

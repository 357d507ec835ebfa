"""An independent statement of the path in plain PyTorch (CPU), compared with
the C oracle on the five workloads and the reference kernel's own shape.

The reference ships no runnable implementation, vectors or fixtures for this
path, so the C oracle cannot be pinned against the reference itself.  This is
the nearest substitute: every step is restated with library operations that
share no code with the oracle - ``torch.matmul`` for the gate product,
``torch.softmax`` / ``torch.sigmoid`` (libm-grade exp) for the scores, a stable
descending ``argsort`` for the selection (on equal keys the lower index comes
first, the reference's tie-break, kernel.cu:1886), ``torch.topk`` only for the
group scores, a stable ``argsort`` of the expert ids for the slot order, and
torch's own float8_e4m3fn cast for the quantiser - and the two must agree:

* logits: within 2e-6 absolute of the fp32 ``matmul`` (different summation order);
* expert ids: equal for every token whose decisive keys are further apart than
  the score tolerance (1e-6 relative); the near-tie tokens are counted and printed;
* combine weights: 1e-6 relative where the ids agree;
* offsets, inverse permutation, drop mask, row copies, fp8 bytes and scales:
  exact, given the oracle's ids (integer and byte work has no tolerance).
"""
import numpy as np
import pytest
import torch

from oracle import cpu_oracle
from moe_rd import workloads
import _util

SCORE_TOL = 1e-6   # relative: scores from libm-grade exp versus the oracle's polynomial exp (a few ulp)
WEIGHT_RTOL = 1e-6


def torch_logits(t, kw):
    x = t["x"].to(torch.float32)
    w = t["w"].to(torch.float32)
    z = x @ (w if kw.get("w_layout", "HE") == "HE" else w.t())
    if kw.get("bias_mode") == "logit" and t["bias"] is not None:
        z = z + t["bias"]
    return z


def torch_route(z, bias, kw):
    """ids [T,K], weights [T,K], and the smallest relative gap between neighbours among the
    first K+1 keys (and between the last kept and the first dropped group)."""
    K = kw["top_k"]
    mode = kw.get("bias_mode", "select")
    scores = torch.softmax(z, dim=-1) if kw.get("score_fn", "softmax") == "softmax" else torch.sigmoid(z)
    keys = scores.clone()
    if bias is not None and mode in ("select", "select_and_weight"):
        keys = keys + bias
    T, E = keys.shape
    G = kw.get("n_groups", 1)
    gap_groups = torch.full((T,), float("inf"))
    if G > 1:
        gs = E // G
        gscore = keys.view(T, G, gs).topk(kw["group_topk"], dim=-1).values.sum(-1)
        gorder = torch.argsort(gscore, dim=-1, descending=True, stable=True)
        kept = gorder[:, : kw["topk_groups"]]
        sorted_g = torch.gather(gscore, 1, gorder)
        gap_groups = ((sorted_g[:, kw["topk_groups"] - 1] - sorted_g[:, kw["topk_groups"]]) /
                      sorted_g[:, kw["topk_groups"] - 1].abs().clamp_min(1e-30))
        mask = torch.zeros(T, G, dtype=torch.bool)
        mask.scatter_(1, kept, True)
        keys = torch.where(mask.repeat_interleave(gs, dim=1), keys, torch.full_like(keys, -float("inf")))
    order = torch.argsort(keys, dim=-1, descending=True, stable=True)
    ids = order[:, :K]
    sk = torch.gather(keys, 1, order[:, : K + 1])
    # smallest gap between neighbours of the first K+1 keys: below the tolerance the order may flip
    gap = ((sk[:, :-1] - sk[:, 1:]) / sk[:, :-1].abs().clamp_min(1e-30)).min(dim=-1).values
    gap = torch.minimum(gap, gap_groups)
    u = torch.gather(keys if mode == "select_and_weight" else scores, 1, ids)
    w = u
    if kw.get("renorm", True):
        w = u / u.sum(-1, keepdim=True).clamp_min(kw.get("norm_min", 1e-20))
    w = w * kw.get("routed_scale", 1.0)
    return ids.to(torch.int32), w, gap


def torch_dispatch(ids, E, capacity):
    """Slot order = stable order of the flat pairs by expert; pairs past the capacity are dropped."""
    T, K = ids.shape
    flat = ids.flatten().to(torch.int64)
    counts = torch.bincount(flat, minlength=E)
    order = torch.argsort(flat, stable=True)                     # pairs grouped by expert, token order inside
    starts_all = torch.cumsum(counts, 0) - counts
    rank = torch.empty_like(flat)
    rank[order] = torch.arange(flat.numel()) - starts_all[flat[order]]
    dropped = (rank >= capacity) if capacity > 0 else torch.zeros_like(rank, dtype=torch.bool)
    kept = counts.clamp_max(capacity) if capacity > 0 else counts
    offsets = torch.zeros(E + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(kept, 0)
    inv = torch.where(dropped, torch.full_like(rank, -1), offsets[flat] + rank)
    return counts, offsets, inv.view(T, K), dropped.view(T, K)


def torch_rows(x, inv, fp8):
    T, K = inv.shape
    R = int((inv >= 0).sum())
    src = torch.arange(T).repeat_interleave(K)[inv.flatten() >= 0]
    dst = inv.flatten()[inv.flatten() >= 0]
    if not fp8:
        rows = torch.zeros((R, x.shape[1]), dtype=torch.bfloat16)
        rows[dst] = x[src]
        return rows.view(torch.int16).numpy().view(np.uint16), None
    xf = x.to(torch.float32).view(T, -1, 128)
    amax = xf.abs().amax(dim=-1)
    scale = amax.clamp_min(1e-30) * torch.tensor(1.0 / 448.0, dtype=torch.float32)
    q = (xf * (1.0 / scale).unsqueeze(-1)).to(torch.float8_e4m3fn).view(torch.uint8).view(T, -1)
    rows = torch.zeros((R, x.shape[1]), dtype=torch.uint8)
    scales = torch.zeros((R, scale.shape[1]), dtype=torch.float32)
    rows[dst] = q[src]
    scales[dst] = scale[src]
    return rows.numpy(), scales.numpy()


@pytest.mark.parametrize("name,T,H", [("c1", 512, 1024), ("c2", 2048, 4096), ("c3", 4096, 2048),
                                      ("c4", 2048, 7168), ("ref", 1024, 8192), ("c3", 777, 256)])
def test_oracle_agrees_with_a_plain_pytorch_statement(name, T, H):
    t, kw = workloads.make(name, T=T, H=H)
    if name == "c3" and T != 4096:
        kw = dict(kw, capacity=int(np.ceil(1.25 * T * kw["top_k"] / 128)))
    ref = _util.run_oracle(t, kw)
    E = ref["offsets"].shape[0] - 1

    # gate product
    z = torch_logits(t, kw)
    err = float((z - torch.from_numpy(ref["logits"])).abs().max())
    assert err < 2e-6 * max(1.0, float(z.abs().max())), f"logits differ by {err}"

    # scoring and selection, from the oracle's logits so that only these steps are compared
    ids, w, gap = torch_route(torch.from_numpy(ref["logits"]), t["bias"], kw)
    same = (ids.numpy() == ref["expert_ids"]).all(axis=1)
    near_tie = (gap < SCORE_TOL).numpy()
    print(f"{name}: {int((~same).sum())} of {T} tokens select differently, {int(near_tie.sum())} tokens have "
          f"decisive keys closer than {SCORE_TOL}")
    assert not (~same & ~near_tie).any(), "selection differs outside the near-tie set"
    assert near_tie.mean() < 0.02
    np.testing.assert_allclose(w.numpy()[same], ref["combine_weights"][same], rtol=WEIGHT_RTOL, atol=0)

    # dispatch and row movement: exact, given the same ids
    cap = int(kw.get("capacity", 0) or 0)
    counts, offsets, inv, dropped = torch_dispatch(torch.from_numpy(ref["expert_ids"]), E, cap)
    np.testing.assert_array_equal(counts.numpy(), ref["counts"])
    np.testing.assert_array_equal(offsets.numpy(), ref["offsets"])
    np.testing.assert_array_equal(inv.numpy(), ref["inverse_perm"])
    np.testing.assert_array_equal(dropped.numpy().astype(np.uint8), ref["drop_mask"])
    fp8 = kw.get("rows_format", "bf16") == "fp8"
    rows, scales = torch_rows(t["x"], inv, fp8)
    R = int(offsets[-1])
    np.testing.assert_array_equal(rows, ref["permuted"][:R])
    if fp8:
        np.testing.assert_array_equal(scales.view(np.uint32), ref["scales"][:R].view(np.uint32))

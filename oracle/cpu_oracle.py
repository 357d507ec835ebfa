"""ctypes front end of the CPU oracle (``moe_rd_oracle.c``).

TEST INFRASTRUCTURE ONLY.  Imported by the tests, by the smoke check and by the
CPU-baseline / reference arm of the benchmark; the product package never
imports it.  PARITY UNPINNED: the reference project holds no golden vectors or
runnable CPU code for this path, so the oracle is the specification (see the
header of ``moe_rd_oracle.c``).

bf16 tensors cross this boundary as ``numpy.uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "libmoe_rd_oracle.so"
_lib = None

SCORE_FN = {"softmax": 0, "sigmoid": 1}
W_LAYOUT = {"HE": 0, "EH": 1}


def build(force: bool = False) -> Path:
    """Compile the oracle with the system C compiler (seconds)."""
    src = _DIR / "moe_rd_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-s", "-B", "-C", str(_DIR)], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return _SO


def _host_has_fma() -> bool:
    try:
        return " fma " in Path("/proc/cpuinfo").read_text().replace("\n", " ")
    except OSError:
        return False


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        # The Makefile adds -mfma only when this host has FMA; a library built
        # elsewhere must not be trusted on a host without it, so rebuild there.
        build(force=not _host_has_fma())
        L = ctypes.CDLL(str(_SO))
        vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
        L.moe_oracle_logits.argtypes = [vp, vp, i32, i32, vp, i64, i32, i32, vp]
        L.moe_oracle_logits.restype = None
        L.moe_oracle_logits_f64.argtypes = [vp, vp, i32, i32, vp, i64, i32, i32, vp]
        L.moe_oracle_logits_f64.restype = None
        L.moe_oracle_expf.argtypes = [f32]
        L.moe_oracle_expf.restype = f32
        L.moe_oracle_route.argtypes = [vp, vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, f32, f32, vp, vp]
        L.moe_oracle_route.restype = i32
        L.moe_oracle_dispatch.argtypes = [vp, i64, i32, i32, i64, vp, vp, vp, vp]
        L.moe_oracle_dispatch.restype = None
        L.moe_oracle_permute_bf16.argtypes = [vp, vp, i64, i32, i32, vp]
        L.moe_oracle_permute_bf16.restype = None
        L.moe_oracle_permute_fp8.argtypes = [vp, vp, i64, i32, i32, vp, vp]
        L.moe_oracle_permute_fp8.restype = None
        L.moe_oracle_f32_to_e4m3.argtypes = [f32]
        L.moe_oracle_f32_to_e4m3.restype = ctypes.c_uint8
        L.moe_oracle_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.moe_oracle_e4m3_to_f32.restype = f32
        L.moe_oracle_combine.argtypes = [vp, vp, vp, vp, i64, i32, i32, vp]
        L.moe_oracle_combine.restype = None
        L.moe_oracle_combine_add_rows.argtypes = [vp, vp, vp, i64, i32, vp]
        L.moe_oracle_combine_add_rows.restype = None
        L.moe_oracle_max_threads.restype = i32
        L.moe_oracle_set_threads.argtypes = [i32]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def _w(w):
    """Gate weight as (array, dtype code): float32 stays, uint16 means bf16 bits."""
    if w.dtype == np.float32:
        return np.ascontiguousarray(w), 0
    if w.dtype == np.uint16:
        return np.ascontiguousarray(w), 1
    raise TypeError("gate weight must be float32 or uint16 (bf16 bits)")


def logits(x_u16, w, *, w_layout="HE", logit_bias=None, f64=False):
    x = _c(x_u16, np.uint16)
    T, H = x.shape
    w, wd = _w(w)
    E = w.shape[1] if w_layout == "HE" else w.shape[0]
    assert (w.shape[0] if w_layout == "HE" else w.shape[1]) == H
    lb = _c(logit_bias, np.float32)
    z = np.empty((T, E), np.float64 if f64 else np.float32)
    fn = lib().moe_oracle_logits_f64 if f64 else lib().moe_oracle_logits
    fn(_p(x), _p(w), wd, W_LAYOUT[w_layout], _p(lb), T, H, E, _p(z))
    return z


def route(z, *, top_k, score_fn="softmax", select_bias=None, n_groups=1, topk_groups=1,
          group_topk=1, weight_from_key=False, renorm=True, routed_scale=1.0, norm_min=1e-20):
    z = _c(z, np.float32)
    T, E = z.shape
    sb = _c(select_bias, np.float32)
    ids = np.empty((T, top_k), np.int32)
    wts = np.empty((T, top_k), np.float32)
    rc = lib().moe_oracle_route(_p(z), _p(sb), T, E, top_k, SCORE_FN[score_fn], n_groups,
                                topk_groups, group_topk, int(weight_from_key), int(renorm),
                                routed_scale, norm_min, _p(ids), _p(wts))
    if rc != 0:
        raise ValueError("invalid routing parameters")
    return ids, wts


def dispatch(ids, E, capacity=0):
    ids = _c(ids, np.int32)
    T, K = ids.shape
    counts = np.empty(E, np.int32)
    offsets = np.empty(E + 1, np.int32)
    inv = np.empty((T, K), np.int32)
    drop = np.empty((T, K), np.uint8)
    lib().moe_oracle_dispatch(_p(ids), T, K, E, int(capacity), _p(counts), _p(offsets), _p(inv), _p(drop))
    return counts, offsets, inv, drop


def permute(x_u16, inv, *, quant="bf16", n_rows=None):
    """Rows in expert-major order.  Rows past offsets[E] stay zero."""
    x = _c(x_u16, np.uint16)
    inv = _c(inv, np.int32)
    T, H = x.shape
    K = inv.shape[1]
    R = T * K if n_rows is None else n_rows
    if quant == "bf16":
        rows = np.zeros((R, H), np.uint16)
        lib().moe_oracle_permute_bf16(_p(x), _p(inv), T, K, H, _p(rows))
        return rows, None
    assert quant == "fp8" and H % 128 == 0
    rows = np.zeros((R, H), np.uint8)
    scales = np.zeros((R, H // 128), np.float32)
    lib().moe_oracle_permute_fp8(_p(x), _p(inv), T, K, H, _p(rows), _p(scales))
    return rows, scales


def route_dispatch(x_u16, w, *, top_k, w_layout="HE", logit_bias=None, select_bias=None,
                   score_fn="softmax", n_groups=1, topk_groups=1, group_topk=1,
                   weight_from_key=False, renorm=True, routed_scale=1.0, norm_min=1e-20,
                   capacity=0, quant="bf16", given_logits=None, **_ignored):
    """The whole path on the CPU.  ``given_logits`` replaces the gate product
    (used to check everything downstream of a tensor-core gate bit for bit)."""
    z = given_logits if given_logits is not None else logits(x_u16, w, w_layout=w_layout, logit_bias=logit_bias)
    E = z.shape[1]
    ids, wts = route(z, top_k=top_k, score_fn=score_fn, select_bias=select_bias, n_groups=n_groups,
                     topk_groups=topk_groups, group_topk=group_topk, weight_from_key=weight_from_key,
                     renorm=renorm, routed_scale=routed_scale, norm_min=norm_min)
    counts, offsets, inv, drop = dispatch(ids, E, capacity)
    rows, scales = permute(x_u16, inv, quant=quant)
    return {"logits": z, "expert_ids": ids, "combine_weights": wts, "counts": counts,
            "offsets": offsets, "inverse_perm": inv, "drop_mask": drop,
            "permuted": rows, "scales": scales}


def ep_exchange(per_rank, E, world):
    """Single-process statement of the expert-parallel exchange.

    ``per_rank[r]`` is rank r's ``route_dispatch`` result.  Rank d owns experts
    [d*E/W, (d+1)*E/W); its buffer is expert-major and, inside an expert,
    ordered by (source rank, source slot order).  Returns for every rank d the
    rows, scales (or None), the per-(source, local expert) counts [W, E/W] and
    the local expert offsets [E/W + 1].
    """
    epr = E // world
    out = []
    for d in range(world):
        cnt = np.zeros((world, epr), np.int64)
        rows, scl = [], []
        for le in range(epr):
            e = d * epr + le
            for s in range(world):
                o = per_rank[s]["offsets"]
                cnt[s, le] = o[e + 1] - o[e]
                rows.append(per_rank[s]["permuted"][o[e]:o[e + 1]])
                if per_rank[s]["scales"] is not None:
                    scl.append(per_rank[s]["scales"][o[e]:o[e + 1]])
        offs = np.zeros(epr + 1, np.int64)
        offs[1:] = np.cumsum(cnt.sum(axis=0))
        out.append({"rows": np.concatenate(rows, axis=0),
                    "scales": np.concatenate(scl, axis=0) if scl else None,
                    "counts": cnt, "offsets": offs})
    return out


def ep_send_once_marks(per_rank, E, world, n_rows_buffer):
    """The marks of the send-once exchange, stated from the routing results alone.

    A token that has several kept pairs on one REMOTE rank sends its row there once, with the first of
    them; every later pair is a mark ``copy_of[row of that pair] = row of the first pair`` in the owner's
    array.  Rows are numbered as in ``ep_exchange`` (expert-major; inside an expert by source rank, then by
    the source's slot order).  Returns one int32 array [n_rows_buffer] per owner, -1 where no mark is.
    """
    epr = E // world
    kept = np.stack([np.diff(np.asarray(p["offsets"], dtype=np.int64)) for p in per_rank])  # [source, expert]
    marks = [np.full(n_rows_buffer, -1, np.int32) for _ in range(world)]
    for d in range(world):
        cnt = kept[:, d * epr:(d + 1) * epr]                       # [source, local expert]
        local_start = np.concatenate([[0], np.cumsum(cnt.sum(axis=0))])[:-1]
        before = np.cumsum(cnt, axis=0) - cnt                      # rows of lower source ranks
        for s in range(world):
            if s == d:
                continue
            ids = np.asarray(per_rank[s]["expert_ids"], dtype=np.int64)
            inv = np.asarray(per_rank[s]["inverse_perm"], dtype=np.int64)
            offs = np.asarray(per_rank[s]["offsets"], dtype=np.int64)
            for t in range(ids.shape[0]):
                first = -1
                for k in range(ids.shape[1]):
                    e = ids[t, k]
                    if e // epr != d or inv[t, k] < 0:
                        continue
                    le = e - d * epr
                    row = local_start[le] + before[s, le] + (inv[t, k] - offs[e])
                    if first < 0:
                        first = row
                    else:
                        marks[d][row] = first
    return marks


def combine(y_u16, inverse_perm, weights, shared_u16=None):
    """out[t] = shared[t] + sum_k w[t,k] * y[inverse_perm[t,k]] (bf16 bits in, bf16 bits out)."""
    y = _c(y_u16, np.uint16)
    inv = _c(inverse_perm, np.int32)
    w = _c(weights, np.float32)
    sh = _c(shared_u16, np.uint16)
    T, K = inv.shape
    H = y.shape[1]
    out = np.empty((T, H), np.uint16)
    lib().moe_oracle_combine(_p(y), _p(inv), _p(w), _p(sh), T, K, H, _p(out))
    return out


def combine_add_rows(y_u16, row_token, row_weight, n_rows, out_u16):
    """out[row_token[p]] += bf16(row_weight[p] * y[p]) for p < n_rows, rows in ascending order
    (bf16 bits; returns the updated copy of ``out_u16``)."""
    y = _c(y_u16, np.uint16)
    tok = _c(row_token, np.int32)
    wt = _c(row_weight, np.float32)
    out = np.array(out_u16, dtype=np.uint16, order="C", copy=True)
    lib().moe_oracle_combine_add_rows(_p(y), _p(tok), _p(wt), int(n_rows), y.shape[1], _p(out))
    return out


def row_meta(inverse_perm, weights, n_rows):
    """Forward permutation: token and combine weight of every permuted row
    (the reference's tok / pw, kernel.cu:2172-2177).  Rows nobody maps to keep
    token -1 and weight 0."""
    inv = np.asarray(inverse_perm, dtype=np.int64)
    T, K = inv.shape
    tok = np.full(n_rows, -1, dtype=np.int32)
    wt = np.zeros(n_rows, dtype=np.float32)
    t_idx = np.repeat(np.arange(T, dtype=np.int32), K).reshape(T, K)
    keep = inv >= 0
    tok[inv[keep]] = t_idx[keep]
    wt[inv[keep]] = np.asarray(weights, dtype=np.float32)[keep]
    return tok, wt


def expert_stats(offsets, row_weight):
    """Per-expert weight sum in the fixed order the statistics kernel states:
    element i of an expert's rows is added (fp32, ascending i) to partial i % 256,
    the partials are combined by the tree v[i] += v[i + off], off = 128..1;
    mean = sum / max(rows, 1); load = rows / max(all rows, 1).  (The reference
    accumulates wsum with atomics in no fixed order, kernel.cu:1903-1919.)"""
    offsets = np.asarray(offsets, dtype=np.int64)
    w = np.asarray(row_weight, dtype=np.float32)
    E = offsets.size - 1
    wsum = np.zeros(E, dtype=np.float32)
    mean = np.zeros(E, dtype=np.float32)
    load = np.zeros(E, dtype=np.float32)
    total = np.float32(max(int(offsets[E]), 1))
    for e in range(E):
        seg = w[offsets[e]:offsets[e + 1]]
        rows = seg.size
        pad = (-rows) % 256
        # padding with +0.0 leaves every partial unchanged except that -0.0 + 0.0 = +0.0,
        # which is also what a partial that starts from +0.0 gives
        m = np.concatenate([seg, np.zeros(pad, dtype=np.float32)]).reshape(-1, 256)
        acc = np.zeros(256, dtype=np.float32)
        for r in range(m.shape[0]):
            acc = (acc + m[r]).astype(np.float32)
        off = 128
        while off:
            acc[:off] = (acc[:off] + acc[off:2 * off]).astype(np.float32)
            off >>= 1
        wsum[e] = acc[0]
        mean[e] = np.float32(acc[0]) / np.float32(max(rows, 1))
        load[e] = np.float32(rows) / total
    return wsum, mean, load


def gemm_plan(offsets, a_base, a_row_bytes, w_base, w_expert_bytes, d_base, d_row_bytes, n, k,
              ident_base=0, ident_m=0):
    """Groups of the ragged expert GEMM as the reference's plan_kernel lays them
    out (moe_gemm.cu:613-638): (m, n, k, identity, a, b, d) per expert, with
    addresses as integers."""
    offsets = np.asarray(offsets, dtype=np.int64)
    out = []
    for e in range(offsets.size - 1):
        start, m = int(offsets[e]), int(offsets[e + 1] - offsets[e])
        ident = bool(ident_m > 0 and m == ident_m and ident_base)
        out.append(dict(m=m, n=n, k=k, identity=int(ident),
                        a=ident_base if ident else a_base + start * a_row_bytes,
                        b=w_base + e * w_expert_bytes, d=d_base + start * d_row_bytes))
    return out


def set_threads(n: int) -> None:
    lib().moe_oracle_set_threads(int(n))


def max_threads() -> int:
    return int(lib().moe_oracle_max_threads())

"""The workspace-free entry point, moe_rd_route_dispatch_noalloc.

Some users of the library may not allocate device memory at call time (their
host program owns the whole device-memory budget, or they froze their pool
after start-up), so they cannot provide the scratch buffer that
moe_rd_route_dispatch asks for.  This entry point keeps its scratch in a fixed
array inside the library instead.  The test drives it through the C ABI, twice
in a row on different problems (the second call finds the first call's leftovers
in the shared scratch), and requires exactly the outputs of the regular entry
point: integer outputs, row bytes and scales bit for bit, weights to 1e-6.

This file sorts last on purpose: with `pytest -x` every other test has already
run by the time it starts.
"""
import ctypes

import numpy as np
import pytest
import torch

from moe_rd import _cabi, workloads

pytestmark = pytest.mark.gpu

NOALLOC_MAX_BYTES = 32 << 20


def _setup(name, T, H):
    dev = torch.device("cuda:0")
    t, kw = workloads.make(name, T=T, H=H)
    x, w = t["x"].to(dev), t["w"].to(dev)
    bias = None if t["bias"] is None else t["bias"].to(dev)
    E, K = w.shape[1], kw["top_k"]
    fp8 = kw.get("rows_format", "bf16") == "fp8"
    mode = kw.get("bias_mode", "select")
    cap = int(kw.get("capacity", 0) or 0)
    out_rows = T * K if not cap else min(T * K, E * cap)
    p = _cabi.Params(
        T=T, H=H, E=E, K=K, n_groups=kw.get("n_groups", 1), topk_groups=kw.get("topk_groups", 1),
        group_topk=kw.get("group_topk", 1), score_fn=_cabi.SCORE_FN[kw.get("score_fn", "softmax")],
        weight_from_key=int(mode == "select_and_weight"), renorm=int(kw.get("renorm", True)),
        routed_scale=kw.get("routed_scale", 1.0), norm_min=1e-20, capacity=cap, out_rows=out_rows,
        rows_format=int(fp8), w_dtype=_cabi.W_DTYPE["fp32" if w.dtype == torch.float32 else "bf16"],
        w_layout=0, gate_impl=0, scatter_impl=0, flags=0)

    def outputs():
        o = dict(
            permuted=torch.zeros((out_rows, H), dtype=torch.uint8 if fp8 else torch.bfloat16, device=dev),
            scales=torch.zeros((out_rows, H // 128), dtype=torch.float32, device=dev) if fp8 else None,
            offsets=torch.zeros(E + 1, dtype=torch.int32, device=dev),
            inverse_perm=torch.zeros((T, K), dtype=torch.int32, device=dev),
            combine_weights=torch.zeros((T, K), dtype=torch.float32, device=dev),
            expert_ids=torch.zeros((T, K), dtype=torch.int32, device=dev),
            drop_mask=torch.zeros((T, K), dtype=torch.uint8, device=dev),
            counts=torch.zeros(E, dtype=torch.int32, device=dev))
        return o

    def buffers(o):
        def ptr(v):
            return None if v is None else ctypes.c_void_p(v.data_ptr())
        return _cabi.Buffers(
            x=ptr(x), gate_w=ptr(w), logit_bias=ptr(bias if mode == "logit" else None),
            select_bias=ptr(bias if mode in ("select", "select_and_weight") else None),
            permuted=ptr(o["permuted"]), scales=ptr(o["scales"]), offsets=ptr(o["offsets"]),
            inverse_perm=ptr(o["inverse_perm"]), combine_weights=ptr(o["combine_weights"]),
            expert_ids=ptr(o["expert_ids"]), drop_mask=ptr(o["drop_mask"]), router_logits=None,
            counts=ptr(o["counts"]))
    return dev, p, outputs, buffers, (x, w, bias)


def _compare(name, T, H, warm=True):
    L = _cabi.lib()
    dev, p, outputs, buffers, keep = _setup(name, T, H)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    # regular entry point, caller-provided workspace
    ref = outputs()
    ws_bytes = _cabi.workspace_bytes(p)
    assert ws_bytes <= NOALLOC_MAX_BYTES
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    b = buffers(ref)
    _cabi.check(L.moe_rd_route_dispatch(ctypes.byref(p), ctypes.byref(b), ctypes.c_void_p(ws.data_ptr()),
                                        ws_bytes, stream))
    # workspace-free entry point; the call itself must not take device memory from anyone
    got = outputs()
    b2 = buffers(got)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    held_before = torch.cuda.memory_allocated(dev)
    _cabi.check(L.moe_rd_route_dispatch_noalloc(ctypes.byref(p), ctypes.byref(b2), stream))
    torch.cuda.synchronize()
    if warm:  # the first call on a device may load the library's device image; later calls take nothing
        # (a device allocation comes in granules of 2 MiB or more; less free memory than before by a
        # granule would be one)
        assert torch.cuda.mem_get_info(dev)[0] > free_before - (1 << 20)
        assert torch.cuda.memory_allocated(dev) == held_before
    st = (ctypes.c_int32 * 8)()
    rc = L.moe_rd_read_status_noalloc(stream, st)
    assert rc == 0 and st[0] == 0, (rc, list(st))
    R = int(ref["offsets"][-1])
    assert R > 0
    for k in ("offsets", "inverse_perm", "expert_ids", "drop_mask", "counts"):
        assert torch.equal(got[k], ref[k]), k
    assert torch.equal(got["permuted"][:R].view(torch.uint8), ref["permuted"][:R].view(torch.uint8))
    if ref["scales"] is not None:
        assert torch.equal(got["scales"][:R].view(torch.int32), ref["scales"][:R].view(torch.int32))
    np.testing.assert_allclose(got["combine_weights"].cpu().numpy(), ref["combine_weights"].cpu().numpy(),
                               rtol=1e-6, atol=0)
    del keep


def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row():
    _compare("c4", 700, 1024, warm=False)   # tensor-core gate, group-limited routing, fp8 rows
    _compare("c3", 3000, 512)   # a different shape on the same scratch: capacity drops, bf16 rows
    _compare("c1", 512, 1024)   # fused GEMV gate


def test_noalloc_refuses_problems_beyond_its_scratch():
    L = _cabi.lib()
    p = _cabi.Params(T=400000, H=1024, E=256, K=8, n_groups=1, topk_groups=1, group_topk=1, score_fn=0,
                     weight_from_key=0, renorm=1, routed_scale=1.0, norm_min=1e-20, capacity=0,
                     out_rows=3200000, rows_format=0, w_dtype=1, w_layout=0, gate_impl=1, scatter_impl=0,
                     flags=0)
    assert _cabi.workspace_bytes(p) > NOALLOC_MAX_BYTES
    b = _cabi.Buffers()
    rc = L.moe_rd_route_dispatch_noalloc(ctypes.byref(p), ctypes.byref(b), None)
    assert rc == -10
    assert b"exceeds" in L.moe_rd_strerror(rc)

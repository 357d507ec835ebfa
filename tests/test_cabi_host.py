"""CPU-side checks of the C ABI: the library loads, exports every function that
include/moe_rd.h declares, validates parameters without touching a GPU, and the
Python operator refuses to run without CUDA (there is no CPU fallback)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from moe_rd import _cabi
import moe_rd

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "moe_rd.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_rd_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _cabi.lib()
    names = declared_functions()
    assert "moe_rd_route_dispatch" in names and "moe_rd_workspace_bytes" in names
    for n in names:
        assert hasattr(L, n), f"{n} declared in moe_rd.h but not exported"
    assert set(_cabi.EXPORTS) <= set(names)
    assert L.moe_rd_version() == 1


def params(**over):
    base = dict(T=1024, H=1024, E=8, K=2, n_groups=1, topk_groups=1, group_topk=1, score_fn=0,
                weight_from_key=0, renorm=1, routed_scale=1.0, norm_min=1e-20, capacity=0,
                out_rows=2048, rows_format=0, w_dtype=1, w_layout=0, gate_impl=0, scatter_impl=0, flags=0)
    base.update(over)
    return _cabi.Params(**base)


def test_struct_layout_matches_header():
    # int64 T, 11 x 4-byte fields, pad?, int64 capacity, int64 out_rows, 6 x int32
    assert ctypes.sizeof(_cabi.Params) == 8 + 4 * 11 + 4 + 16 + 24
    assert ctypes.sizeof(_cabi.Buffers) == 15 * ctypes.sizeof(ctypes.c_void_p)
    # moe_rd_gemm_group: 4 x int32, 3 pointers, 3 x int64
    assert ctypes.sizeof(_cabi.GemmGroup) == 16 + 24 + 24


def test_workspace_bytes_and_validation():
    n = _cabi.workspace_bytes(params())
    assert n % 256 == 0 and n >= 1024 * 8 * 4 + 1024 * 2 * 4
    assert _cabi.workspace_bytes(params(T=0, out_rows=0)) >= 512
    bad = [dict(H=1001), dict(E=0), dict(E=257), dict(K=0), dict(K=9), dict(K=33, E=64),
           dict(n_groups=3), dict(E=64, K=8, n_groups=8, topk_groups=0, group_topk=2),
           dict(E=64, K=8, n_groups=16, topk_groups=1, group_topk=2), dict(score_fn=7),
           dict(rows_format=1, H=1000), dict(capacity=-1), dict(T=-1), dict(gate_impl=9), dict(w_dtype=3),
           dict(flags=8), dict(flags=1, rows_format=1)]
    for o in bad:
        with pytest.raises(_cabi.MoeRdError):
            _cabi.workspace_bytes(params(**o))
            pytest.fail(f"accepted {o}")
    L = _cabi.lib()
    assert L.moe_rd_workspace_bytes(None, None) == -1
    for code in range(0, -11, -1):
        assert len(L.moe_rd_strerror(code)) > 1


def test_route_dispatch_rejects_null_buffers_before_any_cuda_call():
    L = _cabi.lib()
    p = params()
    b = _cabi.Buffers()
    assert L.moe_rd_route_dispatch(ctypes.byref(p), ctypes.byref(b), None, 0, None) == -1
    assert L.moe_rd_route_dispatch(ctypes.byref(p), None, None, 0, None) == -1


def test_residual_combine_validates_before_any_cuda_call():
    L = _cabi.lib()
    buf = (ctypes.c_char * 64)()
    a = ctypes.addressof(buf)
    a16 = (a + 15) & ~15
    ok = (ctypes.c_void_p(a16),) * 5
    assert L.moe_rd_combine_add_rows(7, 4, *ok, None) == L.moe_rd_combine_add_rows(12, 4, *ok, None) != 0   # H % 8
    assert L.moe_rd_combine_add_rows(64, -1, *ok, None) != 0
    assert L.moe_rd_combine_add_rows(64, 0, None, None, None, None, None, None) == 0                       # nothing to do
    assert L.moe_rd_combine_add_rows(64, 4, None, *ok[1:], None) == -1                                      # null
    assert L.moe_rd_combine_add_rows(64, 4, ctypes.c_void_p(a16 + 2), *ok[1:], None) not in (0, -1)         # alignment
    with pytest.raises((RuntimeError, NotImplementedError)):
        z = torch.zeros(4, 64, dtype=torch.bfloat16)
        moe_rd.combine_add_rows(z, torch.zeros(4, dtype=torch.int32), torch.zeros(4), torch.zeros(1, dtype=torch.int32), z)


def test_send_once_exchange_entries_validate_before_any_cuda_call():
    L = _cabi.lib()
    buf = (ctypes.c_char * 256)()
    a16 = ctypes.c_void_p((ctypes.addressof(buf) + 15) & ~15)
    two = (ctypes.c_void_p * 2)(a16, a16)
    p = params(scatter_impl=_cabi.SCATTER_IMPL["bulk"], E=8)
    common = (ctypes.byref(p), a16, a16, a16, a16, a16, 2)
    assert L.moe_rd_ep_scatter_once(*common, 0, two, None, None, a16, None) == -1            # no mark buffers
    assert L.moe_rd_ep_scatter_once(*common, 2, two, None, two, a16, None) == -2             # rank outside the world
    simt = params(scatter_impl=_cabi.SCATTER_IMPL["simt"], E=8)
    assert L.moe_rd_ep_scatter_once(ctypes.byref(simt), a16, a16, a16, a16, a16, 2, 0, two, None, two, a16,
                                    None) == -8                                              # bulk copies only
    assert L.moe_rd_ep_scatter_once(None, a16, a16, a16, a16, a16, 2, 0, two, None, two, a16, None) == -1
    # owner-side copies
    assert L.moe_rd_ep_replicate(ctypes.byref(p), None, None, a16, a16, 8, a16, None) == -1
    assert L.moe_rd_ep_replicate(ctypes.byref(p), a16, None, a16, a16, -1, a16, None) == -2
    fp8 = params(rows_format=_cabi.ROWS_FORMAT["fp8"], H=640)
    assert L.moe_rd_ep_replicate(ctypes.byref(fp8), a16, None, a16, a16, 8, a16, None) == -2   # scale rows not 16-byte multiples
    assert L.moe_rd_ep_replicate(ctypes.byref(p), ctypes.c_void_p(a16.value + 4), None, a16, a16, 8, a16, None) == -4
    assert L.moe_rd_ep_replicate(ctypes.byref(p), a16, None, a16, a16, 0, a16, None) == 0     # nothing to do


def test_no_cpu_path():
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    w = torch.zeros(64, 8, dtype=torch.bfloat16)
    with pytest.raises((RuntimeError, NotImplementedError)):
        moe_rd.route_dispatch(x, w, top_k=2)


def test_capacity_from_factor():
    assert moe_rd.capacity_from_factor(1.25, 32768, 8, 128) == 2560
    assert moe_rd.capacity_from_factor(1.0, 10, 2, 8) == 3


def test_workloads_shapes_and_determinism():
    from moe_rd import workloads
    t, kw = workloads.make("c4", T=16)
    assert t["x"].shape == (16, 7168) and t["w"].shape == (7168, 256) and t["bias"].shape == (256,)
    assert kw["n_groups"] == 8 and kw["rows_format"] == "fp8"
    t2, _ = workloads.make("c4", T=16)
    assert torch.equal(t["x"], t2["x"]) and torch.equal(t["w"], t2["w"])
    t3, _ = workloads.make("c5", T=16, rank=1)
    t4, _ = workloads.make("c5", T=16, rank=0)
    assert torch.equal(t3["w"], t4["w"]) and not torch.equal(t3["x"], t4["x"])
    assert workloads.algorithmic_bytes(16384, 4096, 8, 2, w_bytes=2, fp8=False, kept_rows=32768) == 537198628
    assert workloads.algorithmic_bytes(8192, 7168, 256, 8, w_bytes=2, fp8=True, kept_rows=65536) == 723518468
    assert workloads.algorithmic_bytes(512, 1024, 8, 2, w_bytes=4, fp8=False, kept_rows=1024) == 4235300

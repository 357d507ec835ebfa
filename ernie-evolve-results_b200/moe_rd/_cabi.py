"""ctypes view of libmoe_rd.so (the structs and entry points of include/moe_rd.h).

There is no CPU fallback: importing this module without the built library, or
calling into it without a CUDA device, raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libmoe_rd.so"

SCORE_FN = {"softmax": 0, "sigmoid": 1}
W_DTYPE = {"fp32": 0, "bf16": 1}
W_LAYOUT = {"HE": 0, "EH": 1}
ROWS_FORMAT = {"bf16": 0, "fp8": 1}
GATE_IMPL = {"auto": 0, "simt": 1, "umma": 2, "external": 3, "gemv": 4, "umma_one_cta": 5}
SCATTER_IMPL = {"auto": 0, "simt": 1, "bulk": 2, "none": 3}

EXPORTS = (
    "moe_rd_workspace_bytes", "moe_rd_route_dispatch", "moe_rd_route_dispatch_noalloc",
    "moe_rd_route_dispatch_timed", "moe_rd_read_status", "moe_rd_ep_unpack", "moe_rd_ep_plan", "moe_rd_combine",
    "moe_rd_combine_add_rows",
    "moe_rd_ep_scatter", "moe_rd_ep_scatter_once", "moe_rd_ep_replicate", "moe_rd_ep_combine", "moe_rd_read_status_noalloc", "moe_rd_gemm_plan", "moe_rd_expert_stats",
    "moe_rd_launch_count", "moe_rd_strerror", "moe_rd_last_cuda_error", "moe_rd_version",
)


class Params(ctypes.Structure):
    _fields_ = [
        ("T", ctypes.c_int64),
        ("H", ctypes.c_int32), ("E", ctypes.c_int32), ("K", ctypes.c_int32),
        ("n_groups", ctypes.c_int32), ("topk_groups", ctypes.c_int32), ("group_topk", ctypes.c_int32),
        ("score_fn", ctypes.c_int32), ("weight_from_key", ctypes.c_int32), ("renorm", ctypes.c_int32),
        ("routed_scale", ctypes.c_float), ("norm_min", ctypes.c_float),
        ("capacity", ctypes.c_int64), ("out_rows", ctypes.c_int64),
        ("rows_format", ctypes.c_int32), ("w_dtype", ctypes.c_int32), ("w_layout", ctypes.c_int32),
        ("gate_impl", ctypes.c_int32), ("scatter_impl", ctypes.c_int32), ("flags", ctypes.c_int32),
    ]


class Buffers(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "x", "gate_w", "logit_bias", "select_bias", "permuted", "scales", "offsets",
        "inverse_perm", "combine_weights", "expert_ids", "drop_mask", "router_logits", "counts",
        "row_token", "row_weight")]


class GemmGroup(ctypes.Structure):
    """moe_rd_gemm_group of include/moe_rd.h."""
    _fields_ = [("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32), ("identity", ctypes.c_int32),
                ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("d", ctypes.c_void_p),
                ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldd", ctypes.c_int64)]


FLAG_SKIP_IDENTITY_ROWS = 1
FLAG_TEST_GATE_STALL = 2
FLAG_SEPARATE_GATE_AND_ROUTING = 4


class MoeRdError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"moe_rd error {code}: {text}")
        self.code = code


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(
                f"{_LIB_PATH} is missing: build it with `python -m moe_rd._build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
        L = ctypes.CDLL(str(_LIB_PATH))
        L.moe_rd_workspace_bytes.argtypes = [ctypes.POINTER(Params), ctypes.POINTER(ctypes.c_size_t)]
        L.moe_rd_workspace_bytes.restype = ctypes.c_int
        L.moe_rd_route_dispatch.argtypes = [ctypes.POINTER(Params), ctypes.POINTER(Buffers),
                                            ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        L.moe_rd_route_dispatch.restype = ctypes.c_int
        L.moe_rd_route_dispatch_noalloc.argtypes = [ctypes.POINTER(Params), ctypes.POINTER(Buffers), ctypes.c_void_p]
        L.moe_rd_route_dispatch_noalloc.restype = ctypes.c_int
        L.moe_rd_route_dispatch_timed.argtypes = [ctypes.POINTER(Params), ctypes.POINTER(Buffers),
                                                  ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                                  ctypes.POINTER(ctypes.c_float)]
        L.moe_rd_route_dispatch_timed.restype = ctypes.c_int
        L.moe_rd_ep_unpack.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                       ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_ep_unpack.restype = ctypes.c_int
        L.moe_rd_ep_plan.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_ep_plan.restype = ctypes.c_int
        L.moe_rd_ep_scatter.argtypes = [ctypes.POINTER(Params), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                        ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_ep_scatter.restype = ctypes.c_int
        L.moe_rd_ep_scatter_once.argtypes = [ctypes.POINTER(Params), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                             ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                             ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_ep_scatter_once.restype = ctypes.c_int
        L.moe_rd_ep_replicate.argtypes = [ctypes.POINTER(Params), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_ep_replicate.restype = ctypes.c_int
        L.moe_rd_combine.argtypes = [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_combine.restype = ctypes.c_int
        L.moe_rd_combine_add_rows.argtypes = [ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_combine_add_rows.restype = ctypes.c_int
        L.moe_rd_read_status_noalloc.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
        L.moe_rd_read_status_noalloc.restype = ctypes.c_int
        L.moe_rd_ep_combine.argtypes = [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p]
        L.moe_rd_ep_combine.restype = ctypes.c_int
        L.moe_rd_gemm_plan.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                       ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                       ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_gemm_plan.restype = ctypes.c_int
        L.moe_rd_expert_stats.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p,
                                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        L.moe_rd_expert_stats.restype = ctypes.c_int
        L.moe_rd_read_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
        L.moe_rd_read_status.restype = ctypes.c_int
        L.moe_rd_launch_count.argtypes = []
        L.moe_rd_launch_count.restype = ctypes.c_int64
        L.moe_rd_strerror.argtypes = [ctypes.c_int]
        L.moe_rd_strerror.restype = ctypes.c_char_p
        L.moe_rd_last_cuda_error.argtypes = []
        L.moe_rd_last_cuda_error.restype = ctypes.c_char_p
        L.moe_rd_version.argtypes = []
        L.moe_rd_version.restype = ctypes.c_int
        _lib = L
    return _lib


def check(code: int) -> None:
    if code != 0:
        L = lib()
        text = L.moe_rd_strerror(code).decode()
        if code == -7:
            text += ": " + L.moe_rd_last_cuda_error().decode()
        raise MoeRdError(code, text)


def workspace_bytes(params: Params) -> int:
    n = ctypes.c_size_t(0)
    check(lib().moe_rd_workspace_bytes(ctypes.byref(params), ctypes.byref(n)))
    return int(n.value)


def launch_count() -> int:
    return int(lib().moe_rd_launch_count())

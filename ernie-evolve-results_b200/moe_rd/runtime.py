"""A fixed-shape session over the C ABI: outputs and workspace are allocated
once (the reference allocates one arena per call, kernel.cu:4202-4268; a
serving loop with a fixed token budget can keep it), and every ``run`` only
enqueues kernels on the current stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _cabi
from . import RouteDispatchResult


class Session:
    def __init__(self, T: int, H: int, E: int, K: int, *, device, w_dtype=torch.bfloat16,
                 w_layout: str = "HE", score_fn: str = "softmax", bias_mode: str = "select",
                 n_groups: int = 1, topk_groups: int = 1, group_topk: int = 1, renorm: bool = True,
                 routed_scale: float = 1.0, norm_min: float = 1e-20, capacity: int = 0,
                 rows_format: str = "bf16", gate_impl: str = "auto", scatter_impl: str = "auto",
                 return_logits: bool = False, top_k: Optional[int] = None, flags: int = 0):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("moe_rd has no CPU path")
        self.T, self.H, self.E, self.K = T, H, E, K
        self.bias_mode = bias_mode
        self.fp8 = rows_format == "fp8"
        out_rows = T * K if not capacity else min(T * K, E * capacity)
        d = self.device
        self.rows_moved_here = scatter_impl != "none"  # "none": rows leave through moe_rd.ep instead
        self.permuted = (torch.empty((out_rows, H), dtype=torch.uint8 if self.fp8 else torch.bfloat16, device=d)
                         if self.rows_moved_here else None)
        self.scales = (torch.empty((out_rows, H // 128), dtype=torch.float32, device=d)
                       if self.fp8 and self.rows_moved_here else None)
        self.offsets = torch.empty(E + 1, dtype=torch.int32, device=d)
        self.inverse_perm = torch.empty((T, K), dtype=torch.int32, device=d)
        self.combine_weights = torch.empty((T, K), dtype=torch.float32, device=d)
        self.expert_ids = torch.empty((T, K), dtype=torch.int32, device=d)
        self.drop_mask = torch.empty((T, K), dtype=torch.uint8, device=d)
        self.counts = torch.empty(E, dtype=torch.int32, device=d)
        self.router_logits = torch.empty((T, E), dtype=torch.float32, device=d) if return_logits else None
        self.params = _cabi.Params(
            T=T, H=H, E=E, K=K, n_groups=n_groups, topk_groups=topk_groups, group_topk=group_topk,
            score_fn=_cabi.SCORE_FN[score_fn], weight_from_key=int(bias_mode == "select_and_weight"),
            renorm=int(renorm), routed_scale=routed_scale, norm_min=norm_min, capacity=int(capacity or 0),
            out_rows=out_rows, rows_format=_cabi.ROWS_FORMAT[rows_format],
            w_dtype=_cabi.W_DTYPE["fp32" if w_dtype == torch.float32 else "bf16"],
            w_layout=_cabi.W_LAYOUT[w_layout], gate_impl=_cabi.GATE_IMPL[gate_impl],
            scatter_impl=_cabi.SCATTER_IMPL[scatter_impl], flags=int(flags))
        self.ws_bytes = _cabi.workspace_bytes(self.params)
        self.workspace = torch.empty(self.ws_bytes, dtype=torch.uint8, device=d)

    def _buffers(self, x, w, bias):
        def ptr(t):
            return None if t is None else ctypes.c_void_p(t.data_ptr())
        lb = bias if (bias is not None and self.bias_mode == "logit") else None
        sb = bias if (bias is not None and self.bias_mode in ("select", "select_and_weight")) else None
        return _cabi.Buffers(
            x=ptr(x), gate_w=ptr(w), logit_bias=ptr(lb), select_bias=ptr(sb), permuted=ptr(self.permuted),
            scales=ptr(self.scales), offsets=ptr(self.offsets), inverse_perm=ptr(self.inverse_perm),
            combine_weights=ptr(self.combine_weights), expert_ids=ptr(self.expert_ids),
            drop_mask=ptr(self.drop_mask), router_logits=ptr(self.router_logits), counts=ptr(self.counts),
            row_token=None, row_weight=None)

    def _check_inputs(self, x, w):
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and tuple(x.shape) == (self.T, self.H)):
            raise ValueError("x must be a contiguous CUDA bf16 tensor of the session's [T, H]")
        if not (w.is_cuda and w.is_contiguous()):
            raise ValueError("gate weight must be a contiguous CUDA tensor")

    def run(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> RouteDispatchResult:
        """Enqueue one pass on the current stream; results alias the session's buffers."""
        self._check_inputs(x, w)
        b = self._buffers(x, w, bias)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _cabi.check(_cabi.lib().moe_rd_route_dispatch(
            ctypes.byref(self.params), ctypes.byref(b), ctypes.c_void_p(self.workspace.data_ptr()),
            self.ws_bytes, stream))
        return self.result()

    def capture(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> "torch.cuda.CUDAGraph":
        """Record one pass into a CUDA graph and return it; ``graph.replay()`` repeats the pass on the same
        input and output buffers (refill ``x`` / ``w`` / ``bias`` in place between replays).  The call only
        enqueues kernels and one memset on the given stream - no allocation, no host synchronisation, the
        tensor maps are kernel parameters - so it captures as it is, programmatic launch dependencies between
        its kernels included; a replay pays one submission instead of four or five launches, which is what
        matters for the launch-bound small shapes."""
        self.run(x, w, bias)                    # one-time function attributes are set outside the capture
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.run(x, w, bias)
        self._captured_inputs = (x, w, bias)    # the graph holds their addresses
        return graph

    def run_timed(self, x, w, bias=None):
        """One pass with per-stage device times in ms: (gate, route, scan, positions, scatter). Synchronises."""
        self._check_inputs(x, w)
        b = self._buffers(x, w, bias)
        ms = (ctypes.c_float * 5)()
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _cabi.check(_cabi.lib().moe_rd_route_dispatch_timed(
            ctypes.byref(self.params), ctypes.byref(b), ctypes.c_void_p(self.workspace.data_ptr()),
            self.ws_bytes, stream, ms))
        return tuple(float(v) for v in ms)

    def result(self) -> RouteDispatchResult:
        return RouteDispatchResult(self.permuted, self.offsets, self.inverse_perm, self.combine_weights,
                                   self.scales, self.drop_mask, self.expert_ids, self.router_logits, self.counts)

    def status(self):
        """Device status block of the last run (synchronises). Raises on a failed device check."""
        st = (ctypes.c_int32 * 8)()
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        rc = _cabi.lib().moe_rd_read_status(ctypes.c_void_p(self.workspace.data_ptr()), stream, st)
        vals = [int(v) for v in st]
        if rc != 0:
            raise _cabi.MoeRdError(rc, f"device status {vals}")
        return vals

"""moe_rd — MoE sparse routing and dispatch on B200 (sm_100a).

Host-side mirror of the operator boundary of the reference's
``sol-execbench/029_moe_sparse_routing_and_dispatch`` (``kernel.cu::run``,
kernel.cu:4067-4077): a Python callable that takes hidden states, the router
(gate) weight and a bias, and returns expert-major permuted token rows,
per-expert offsets, the inverse permutation and the combine weights.  It is
registered as the torch custom op ``torch.ops.moe_rd.route_dispatch`` (CUDA
only) on top of the C ABI in ``include/moe_rd.h``.  There is no CPU fallback
and no alternative backend: without ``libmoe_rd.so`` or without a CUDA device
every call raises.
"""
from __future__ import annotations

import ctypes
import math
from typing import NamedTuple, Optional

import torch

from . import _cabi
from ._cabi import MoeRdError  # noqa: F401

__all__ = ["route_dispatch", "combine", "combine_add_rows", "gemm_plan", "expert_stats", "RouteDispatchResult", "ExpertStats",
           "MoeRdError", "capacity_from_factor"]


class RouteDispatchResult(NamedTuple):
    permuted: torch.Tensor                # [T*K, H] bf16, or uint8 viewable as float8_e4m3fn
    offsets: torch.Tensor                 # [E+1] int32, offsets[E] = kept pairs
    inverse_perm: torch.Tensor            # [T, K] int32, -1 = dropped
    combine_weights: torch.Tensor         # [T, K] fp32
    scales: Optional[torch.Tensor]        # [T*K, H/128] fp32 (fp8 rows only)
    drop_mask: torch.Tensor               # [T, K] uint8
    expert_ids: torch.Tensor              # [T, K] int32
    router_logits: Optional[torch.Tensor]  # [T, E] fp32 when requested
    counts: torch.Tensor                  # [E] int32 pairs per expert before dropping
    row_token: Optional[torch.Tensor] = None   # [T*K] int32 token of each permuted row, when requested
    row_weight: Optional[torch.Tensor] = None  # [T*K] fp32 combine weight of each permuted row, when requested


class ExpertStats(NamedTuple):
    weight_sum: torch.Tensor   # [E] fp32, sum of the combine weights of the expert's kept rows (fixed order)
    mean_weight: torch.Tensor  # [E] fp32, weight_sum / max(rows, 1)
    load: torch.Tensor         # [E] fp32, rows / max(all kept rows, 1)


def capacity_from_factor(factor: float, T: int, K: int, E: int) -> int:
    """Rows kept per expert: ceil(factor * T * K / E)."""
    return int(math.ceil(factor * T * K / E))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_BIAS_MODES = ("none", "logit", "select", "select_and_weight")


def _impl(x, gate_weight, logit_bias, select_bias, given_logits, top_k, score_fn, n_groups,
          topk_groups, group_topk, weight_from_key, renorm, routed_scale, norm_min, capacity,
          rows_format, w_layout, gate_impl, scatter_impl, return_logits, return_row_meta, flags):
    """CUDA implementation of ``moe_rd::route_dispatch`` (enqueue only, no host sync)."""
    if not x.is_cuda:
        raise RuntimeError("moe_rd.route_dispatch has no CPU path: hidden_states must be a CUDA tensor")
    if x.dtype != torch.bfloat16:
        raise TypeError("hidden_states must be bfloat16")
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    T, H = x2.shape
    dev = x2.device
    external = given_logits is not None
    if external:
        E = given_logits.shape[-1]
        given_logits = given_logits.to(torch.float32).contiguous()
        w = None
        w_dtype = _cabi.W_DTYPE["bf16"]
    else:
        w = gate_weight.contiguous()
        if w.dtype == torch.float32:
            w_dtype = _cabi.W_DTYPE["fp32"]
        elif w.dtype == torch.bfloat16:
            w_dtype = _cabi.W_DTYPE["bf16"]
        else:
            raise TypeError("gate_weight must be float32 or bfloat16")
        if w.dim() != 2:
            raise ValueError("gate_weight must be 2-D")
        wh, we = (w.shape[0], w.shape[1]) if w_layout == 0 else (w.shape[1], w.shape[0])
        if wh != H:
            raise ValueError(f"gate_weight does not match hidden size {H}")
        E = we
    K = int(top_k)
    for b in (logit_bias, select_bias):
        if b is not None and (b.dtype != torch.float32 or b.numel() != E or not b.is_cuda):
            raise ValueError("bias must be a CUDA float32 tensor of E elements")

    out_rows = T * K
    if capacity > 0:
        out_rows = min(out_rows, E * capacity)
    fp8 = rows_format == _cabi.ROWS_FORMAT["fp8"]
    move_rows = scatter_impl != _cabi.SCATTER_IMPL["none"]
    with torch.cuda.device(dev):
        permuted = torch.empty((out_rows if move_rows else 0, H), dtype=torch.uint8 if fp8 else torch.bfloat16,
                               device=dev)
        scales = torch.empty((out_rows if move_rows else 0, H // 128), dtype=torch.float32, device=dev) if fp8 else None
        offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        inv = torch.empty((T, K), dtype=torch.int32, device=dev)
        weights = torch.empty((T, K), dtype=torch.float32, device=dev)
        ids = torch.empty((T, K), dtype=torch.int32, device=dev)
        drop = torch.empty((T, K), dtype=torch.uint8, device=dev)
        counts = torch.empty(E, dtype=torch.int32, device=dev)
        row_token = torch.empty(out_rows, dtype=torch.int32, device=dev) if return_row_meta else None
        row_weight = torch.empty(out_rows, dtype=torch.float32, device=dev) if return_row_meta else None
        if external:
            logits = given_logits
        elif return_logits:
            logits = torch.empty((T, E), dtype=torch.float32, device=dev)
        else:
            logits = None

        p = _cabi.Params(
            T=T, H=H, E=E, K=K, n_groups=n_groups, topk_groups=topk_groups, group_topk=group_topk,
            score_fn=score_fn, weight_from_key=int(weight_from_key), renorm=int(renorm),
            routed_scale=routed_scale, norm_min=norm_min, capacity=capacity, out_rows=out_rows,
            rows_format=rows_format, w_dtype=w_dtype, w_layout=w_layout,
            gate_impl=_cabi.GATE_IMPL["external"] if external else gate_impl,
            scatter_impl=scatter_impl, flags=int(flags))
        ws_bytes = _cabi.workspace_bytes(p)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        bufs = _cabi.Buffers(
            x=_ptr(x2), gate_w=_ptr(w), logit_bias=_ptr(logit_bias), select_bias=_ptr(select_bias),
            permuted=_ptr(permuted), scales=_ptr(scales), offsets=_ptr(offsets), inverse_perm=_ptr(inv),
            combine_weights=_ptr(weights), expert_ids=_ptr(ids), drop_mask=_ptr(drop),
            router_logits=_ptr(logits), counts=_ptr(counts), row_token=_ptr(row_token),
            row_weight=_ptr(row_weight))
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _cabi.check(_cabi.lib().moe_rd_route_dispatch(
            ctypes.byref(p), ctypes.byref(bufs), ctypes.c_void_p(ws.data_ptr()), ws_bytes, stream))
        # ws goes back to the caching allocator here; reuse is ordered on this stream
    empty = torch.empty(0, device=dev)
    return [permuted, offsets, inv, weights, scales if scales is not None else empty, drop, ids,
            logits if (logits is not None and not external) else empty, counts,
            row_token if row_token is not None else empty, row_weight if row_weight is not None else empty]


_SCHEMA = ("route_dispatch(Tensor hidden_states, Tensor? gate_weight, Tensor? logit_bias, "
           "Tensor? select_bias, Tensor? given_logits, int top_k, int score_fn, int n_groups, "
           "int topk_groups, int group_topk, bool weight_from_key, bool renorm, float routed_scale, "
           "float norm_min, int capacity, int rows_format, int w_layout, int gate_impl, "
           "int scatter_impl, bool return_logits, bool return_row_meta, int flags) -> Tensor[]")

_torch_lib = torch.library.Library("moe_rd", "DEF")
_torch_lib.define(_SCHEMA)
_torch_lib.impl("route_dispatch", _impl, "CUDA")


def route_dispatch(hidden_states: torch.Tensor, gate_weight: Optional[torch.Tensor],
                   bias: Optional[torch.Tensor] = None, *, top_k: int,
                   score_fn: str = "softmax", bias_mode: str = "select",
                   n_groups: int = 1, topk_groups: int = 1, group_topk: int = 1,
                   renorm: bool = True, routed_scale: float = 1.0, norm_min: float = 1e-20,
                   capacity_factor: Optional[float] = None, capacity: Optional[int] = None,
                   rows_format: str = "bf16", w_layout: str = "HE", gate_impl: str = "auto",
                   scatter_impl: str = "auto", return_logits: bool = False,
                   given_logits: Optional[torch.Tensor] = None, return_row_meta: bool = False,
                   skip_identity_rows: bool = False) -> RouteDispatchResult:
    """Route tokens to experts and build the expert-major dispatch buffers.

    hidden_states: [..., H] bf16 (CUDA).  gate_weight: [H, E] (``w_layout="HE"``)
    or [E, H] (``"EH"``, the reference's layout, kernel.cu:4324), fp32 or bf16.
    bias: [E] fp32, used according to ``bias_mode``:
      "logit"             added to the logits before scoring;
      "select"            added to the scores for selection only;
      "select_and_weight" added to the scores for selection and kept in the
                          combine weights, the reference's behaviour
                          (kernel.cu:1865-1866, 1891, 1909).
    capacity / capacity_factor: rows kept per expert; later pairs (token order)
    are dropped.  rows_format "fp8" quantises rows to e4m3 with one fp32 scale
    per 128 elements.  ``given_logits`` skips the gate product.
    ``return_row_meta`` also returns the forward permutation (token and combine
    weight of every permuted row; the reference's ``tok`` / ``pw``,
    kernel.cu:2172-2177).  ``skip_identity_rows`` (bf16 rows) leaves the rows of
    an expert that received every token unwritten - they would be a copy of
    ``hidden_states`` - for ``gemm_plan`` to aim that expert at ``hidden_states``
    (the reference's identity shortcut, kernel.cu:2089-2108).
    """
    if bias_mode not in _BIAS_MODES:
        raise ValueError(f"bias_mode must be one of {_BIAS_MODES}")
    logit_bias = bias if (bias is not None and bias_mode == "logit") else None
    select_bias = bias if (bias is not None and bias_mode in ("select", "select_and_weight")) else None
    T = hidden_states.numel() // hidden_states.shape[-1]
    if given_logits is not None:
        E = given_logits.shape[-1]
    else:
        E = gate_weight.shape[1] if w_layout == "HE" else gate_weight.shape[0]
    if capacity is None:
        capacity = capacity_from_factor(capacity_factor, T, top_k, E) if capacity_factor else 0
    out = torch.ops.moe_rd.route_dispatch(
        hidden_states, gate_weight, logit_bias, select_bias, given_logits, top_k,
        _cabi.SCORE_FN[score_fn], n_groups, topk_groups, group_topk,
        bias_mode == "select_and_weight", renorm, float(routed_scale), float(norm_min),
        int(capacity), _cabi.ROWS_FORMAT[rows_format], _cabi.W_LAYOUT[w_layout],
        _cabi.GATE_IMPL[gate_impl], _cabi.SCATTER_IMPL[scatter_impl], return_logits, return_row_meta,
        _cabi.FLAG_SKIP_IDENTITY_ROWS if skip_identity_rows else 0)
    permuted, offsets, inv, weights, scales, drop, ids, logits, counts, row_token, row_weight = out
    if given_logits is not None:
        logits = given_logits
    elif not return_logits:
        logits = None
    return RouteDispatchResult(permuted, offsets, inv, weights,
                               scales if rows_format == "fp8" else None, drop, ids, logits, counts,
                               row_token if return_row_meta else None, row_weight if return_row_meta else None)


def _combine_impl(y, inverse_perm, combine_weights, shared):
    if not y.is_cuda:
        raise RuntimeError("moe_rd.combine has no CPU path")
    if y.dtype != torch.bfloat16 or inverse_perm.dtype != torch.int32 or combine_weights.dtype != torch.float32:
        raise TypeError("combine expects y bf16, inverse_perm int32, combine_weights float32")
    y = y.contiguous()
    inv = inverse_perm.contiguous()
    w = combine_weights.contiguous()
    T, K = inv.shape
    H = y.shape[-1]
    sh = None if shared is None else shared.reshape(T, H).contiguous()
    with torch.cuda.device(y.device):
        out = torch.empty((T, H), dtype=torch.bfloat16, device=y.device)
        stream = ctypes.c_void_p(torch.cuda.current_stream(y.device).cuda_stream)
        _cabi.check(_cabi.lib().moe_rd_combine(T, H, K, _ptr(y), _ptr(inv), _ptr(w), _ptr(sh), _ptr(out), stream))
    return out


_torch_lib.define("combine(Tensor y, Tensor inverse_perm, Tensor combine_weights, Tensor? shared) -> Tensor")
_torch_lib.impl("combine", _combine_impl, "CUDA")


def combine(y: torch.Tensor, inverse_perm: torch.Tensor, combine_weights: torch.Tensor,
            shared: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = shared[t] + sum_k combine_weights[t,k] * y[inverse_perm[t,k]]  (bf16 in, bf16 out).

    The inverse of ``route_dispatch``'s permutation with the routing weights
    applied: ``y`` holds the expert outputs in expert-major row order.  Mirrors
    the reference's combine_kernel (kernel.cu:2365-2428)."""
    return torch.ops.moe_rd.combine(y, inverse_perm, combine_weights, shared)


def _combine_add_rows_impl(y, row_token, row_weight, n_rows, out):
    if not y.is_cuda:
        raise RuntimeError("moe_rd.combine_add_rows has no CPU path")
    if (y.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or row_token.dtype != torch.int32
            or row_weight.dtype != torch.float32 or n_rows.dtype != torch.int32):
        raise TypeError("combine_add_rows expects y/out bf16, row_token/n_rows int32, row_weight float32")
    if not (y.is_contiguous() and out.is_contiguous() and row_token.is_contiguous() and row_weight.is_contiguous()):
        raise ValueError("combine_add_rows updates out in place and takes contiguous tensors")
    H = y.shape[-1]
    max_rows = min(y.shape[0], row_token.numel(), row_weight.numel())
    if out.shape[-1] != H or n_rows.numel() < 1:
        raise ValueError("combine_add_rows: out must be [T,H] like y's rows, n_rows a device int32 scalar")
    with torch.cuda.device(y.device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(y.device).cuda_stream)
        _cabi.check(_cabi.lib().moe_rd_combine_add_rows(H, max_rows, _ptr(y), _ptr(row_token), _ptr(row_weight),
                                                        _ptr(n_rows), _ptr(out), stream))


_torch_lib.define("combine_add_rows(Tensor y, Tensor row_token, Tensor row_weight, Tensor n_rows, "
                  "Tensor(a!) out) -> ()")
_torch_lib.impl("combine_add_rows", _combine_add_rows_impl, "CUDA")


def combine_add_rows(y: torch.Tensor, row_token: torch.Tensor, row_weight: torch.Tensor, n_rows: torch.Tensor,
                     out: torch.Tensor) -> torch.Tensor:
    """out[row_token[p]] += bf16(row_weight[p] * y[p]) for p < n_rows, in place; returns ``out``.

    The residual combine of a pipeline whose expert GEMM already reduced most outputs into ``out``
    (the reference's raddleft_kernel, kernel.cu:2451-2486).  ``row_token`` / ``row_weight`` are what
    ``route_dispatch(..., return_row_meta=True)`` returns; ``n_rows`` is a DEVICE int32 tensor (for
    example ``offsets[-1:]``), so the number of live rows is never read back.  The adds are bf16
    reductions in no fixed order: bit-exact when a token receives at most one row."""
    torch.ops.moe_rd.combine_add_rows(y, row_token, row_weight, n_rows, out)
    return out


def gemm_plan(offsets: torch.Tensor, rows: torch.Tensor, expert_weights: torch.Tensor, out: torch.Tensor,
              identity_source: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Device-side plan of the ragged expert GEMM ``out[rows of e] = rows[rows of e] @ expert_weights[e]``.

    Returns a uint8 tensor [E, sizeof(moe_rd_gemm_group)] holding one
    ``moe_rd_gemm_group`` per expert (problem shape, A / B / D pointers, pitches),
    built on the current stream from ``offsets`` without a host synchronisation;
    ``decode_gemm_plan`` reads it back.  With ``identity_source`` (the un-permuted
    hidden states), an expert that holds every token reads it instead of its
    slice of ``rows``.  Mirrors the reference's plan_kernel (moe_gemm.cu:613-638).
    """
    if not offsets.is_cuda or offsets.dtype != torch.int32:
        raise TypeError("offsets must be a CUDA int32 tensor")
    E = offsets.numel() - 1
    if expert_weights.shape[0] != E:
        raise ValueError("expert_weights must have one leading slice per expert")
    k = rows.shape[-1]
    n = out.shape[-1]
    ident_m = 0 if identity_source is None else identity_source.numel() // identity_source.shape[-1]
    with torch.cuda.device(offsets.device):
        plan = torch.empty((E, ctypes.sizeof(_cabi.GemmGroup)), dtype=torch.uint8, device=offsets.device)
        stream = ctypes.c_void_p(torch.cuda.current_stream(offsets.device).cuda_stream)
        _cabi.check(_cabi.lib().moe_rd_gemm_plan(
            _ptr(offsets), E, _ptr(rows), rows.stride(0) * rows.element_size(), _ptr(identity_source), ident_m,
            _ptr(expert_weights), expert_weights.stride(0) * expert_weights.element_size(), _ptr(out),
            out.stride(0) * out.element_size(), n, k, _ptr(plan), stream))
    return plan


def decode_gemm_plan(plan: torch.Tensor):
    """Host copy of a ``gemm_plan`` result as a list of ``_cabi.GemmGroup`` (synchronises)."""
    raw = plan.cpu().numpy().tobytes()
    size = ctypes.sizeof(_cabi.GemmGroup)
    return [_cabi.GemmGroup.from_buffer_copy(raw[i * size:(i + 1) * size]) for i in range(plan.shape[0])]


def expert_stats(offsets: torch.Tensor, row_weight: torch.Tensor) -> ExpertStats:
    """Per-expert sum and mean of the combine weights of the kept rows, and the
    share of rows each expert received; the sums are added in a fixed order, so
    repeated runs give the same bits (the reference's wsum / counts,
    kernel.cu:1903-1919, made outputs)."""
    if not offsets.is_cuda or offsets.dtype != torch.int32 or row_weight.dtype != torch.float32:
        raise TypeError("expert_stats expects CUDA int32 offsets and float32 row weights")
    E = offsets.numel() - 1
    with torch.cuda.device(offsets.device):
        ws, mw, ld = (torch.empty(E, dtype=torch.float32, device=offsets.device) for _ in range(3))
        stream = ctypes.c_void_p(torch.cuda.current_stream(offsets.device).cuda_stream)
        _cabi.check(_cabi.lib().moe_rd_expert_stats(_ptr(offsets), _ptr(row_weight.contiguous()), E, _ptr(ws), _ptr(mw),
                                                    _ptr(ld), stream))
    return ExpertStats(ws, mw, ld)

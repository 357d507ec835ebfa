"""The five benchmark/parity workloads as seeded synthetic inputs.

No dataset is involved: every tensor is drawn from ``torch.Generator`` on the
CPU (fp32 draw, then cast) so that the GPU path and a CPU checker see the same
bits.  Shapes, dtypes and distributions follow the target configurations:

c1  T=512   H=1024 E=8   top-2 softmax renormalised, fp32 gate weight, bf16 rows
c2  T=16384 H=4096 E=8   top-2 softmax renormalised, bf16 gate weight, bf16 rows
c3  T=32768 H=2048 E=128 top-8 softmax, Zipf(1.1) logit bias scaled to 0..2,
    capacity factor 1.25 with token-order drops, bf16 rows
c4  T=8192  H=7168 E=256 sigmoid + selection-only bias U(-0.1,0.1), 8 groups,
    keep top-4 groups by the sum of each group's top-2, top-8 experts, weights
    normalised and scaled by 2.5, fp8-e4m3 rows with one scale per 128 elements
c5  c4 per rank (T=8192 tokens per rank), experts sharded over the ranks
ref the reference kernel's own problem (kernel.cu:1582-1583, 4324, 4347): T=8192
    H=8192 E=64 top-8, fp32 gate weight in [E,H] layout drawn randn/sqrt(H), softmax,
    a randn correction bias added to the scores for selection AND kept in the
    weights (kernel.cu:1865-1866, 1891, 1909; input draws as kernel.cu:1291-1300
    describes them), bf16 rows
"""
from __future__ import annotations

import math
from typing import Optional

import torch

SPECS = {
    "c1": dict(T=512, H=1024, E=8, K=2, w_dtype=torch.float32, w_std=0.02, seed=1001),
    "c2": dict(T=16384, H=4096, E=8, K=2, w_dtype=torch.bfloat16, w_std=0.02, seed=1002),
    "c3": dict(T=32768, H=2048, E=128, K=8, w_dtype=torch.bfloat16, w_std=0.02, seed=1003),
    "c4": dict(T=8192, H=7168, E=256, K=8, w_dtype=torch.bfloat16, w_std=0.006, seed=1004),
    "c5": dict(T=8192, H=7168, E=256, K=8, w_dtype=torch.bfloat16, w_std=0.006, seed=1005),
    "ref": dict(T=8192, H=8192, E=64, K=8, w_dtype=torch.float32, w_std=None, seed=1029),
}


def make(name: str, *, T: Optional[int] = None, rank: int = 0, H: Optional[int] = None):
    """Returns (tensors, kwargs): CPU tensors ``x``, ``w``, ``bias`` and the
    keyword arguments of ``moe_rd.route_dispatch`` for this workload.  ``T`` and
    ``H`` shrink the problem for parity cases; ``rank`` reseeds the tokens of an
    expert-parallel rank (the gate weight and bias are the same on every rank).
    """
    s = SPECS[name]
    T = s["T"] if T is None else T
    H = s["H"] if H is None else H
    E, K = s["E"], s["K"]
    gw = torch.Generator(device="cpu").manual_seed(s["seed"])
    w_std = s["w_std"] if s["w_std"] is not None else 1.0 / math.sqrt(H)
    w = (torch.randn(H, E, generator=gw, dtype=torch.float32) * w_std).to(s["w_dtype"])
    bias = None
    kw = dict(top_k=K, w_layout="HE")
    if name == "ref":
        w = w.t().contiguous()  # [E,H], the reference's layout
        bias = torch.randn(E, generator=gw, dtype=torch.float32)
        kw.update(w_layout="EH", score_fn="softmax", bias_mode="select_and_weight", renorm=True)
    elif name == "c3":
        r = torch.randperm(E, generator=gw).to(torch.float32) + 1.0
        bias = (2.0 * r.pow(-1.1)).to(torch.float32)
        kw.update(score_fn="softmax", bias_mode="logit", renorm=True,
                  capacity=int(math.ceil(1.25 * T * K / E)))
    elif name in ("c4", "c5"):
        bias = (torch.rand(E, generator=gw, dtype=torch.float32) * 0.2 - 0.1)
        kw.update(score_fn="sigmoid", bias_mode="select", n_groups=8, topk_groups=4, group_topk=2,
                  renorm=True, routed_scale=2.5, rows_format="fp8")
    else:
        kw.update(score_fn="softmax", renorm=True)
    gx = torch.Generator(device="cpu").manual_seed(s["seed"] + 100 * rank + 7919)
    x = torch.randn(T, H, generator=gx, dtype=torch.float32).to(torch.bfloat16)
    return dict(x=x, w=w, bias=bias), kw


def algorithmic_bytes(T: int, H: int, E: int, K: int, *, w_bytes: int, fp8: bool, kept_rows: int) -> int:
    """Bytes the path must move: x read twice (gate pass and dispatch pass), the
    gate weight once, every output once; scratch and cache hits earn nothing."""
    row_bytes = H * (1 if fp8 else 2)
    scale_bytes = (H // 128) * 4 if fp8 else 0
    return 2 * T * H * 2 + H * E * w_bytes + kept_rows * (row_bytes + scale_bytes) + T * K * 8 + (E + 1) * 4


def oracle_kwargs(kw: dict, bias) -> dict:
    """Translate ``route_dispatch`` keywords into the CPU checker's keywords."""
    o = dict(top_k=kw["top_k"], w_layout=kw.get("w_layout", "HE"), score_fn=kw.get("score_fn", "softmax"),
             n_groups=kw.get("n_groups", 1), topk_groups=kw.get("topk_groups", 1),
             group_topk=kw.get("group_topk", 1), renorm=kw.get("renorm", True),
             routed_scale=kw.get("routed_scale", 1.0), norm_min=kw.get("norm_min", 1e-20),
             capacity=kw.get("capacity", 0) or 0, quant=kw.get("rows_format", "bf16"))
    mode = kw.get("bias_mode", "select")
    b = None if bias is None else bias.numpy()
    o["logit_bias"] = b if mode == "logit" else None
    o["select_bias"] = b if mode in ("select", "select_and_weight") else None
    o["weight_from_key"] = mode == "select_and_weight"
    return o

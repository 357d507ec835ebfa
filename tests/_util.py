"""Shared helpers of the parity tests: run the CUDA path through the public
callable (which goes through the C ABI) and compare with the CPU oracle."""
from __future__ import annotations

import numpy as np
import torch

from oracle import cpu_oracle
from moe_rd import workloads


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def w_for_oracle(w: torch.Tensor) -> np.ndarray:
    return w.numpy() if w.dtype == torch.float32 else bf16_bits(w)


def run_oracle(tensors, kw, given_logits=None):
    ok = workloads.oracle_kwargs(kw, tensors.get("bias"))
    w = tensors.get("w")
    return cpu_oracle.route_dispatch(bf16_bits(tensors["x"]), None if w is None else w_for_oracle(w),
                                     given_logits=given_logits, **ok)


def run_gpu(tensors, kw, **extra):
    import moe_rd
    dev = torch.device("cuda:0")
    x = tensors["x"].to(dev)
    w = None if tensors.get("w") is None else tensors["w"].to(dev)
    b = None if tensors.get("bias") is None else tensors["bias"].to(dev)
    args = dict(kw)
    args.update(extra)
    if "given_logits" in args and args["given_logits"] is not None:
        args["given_logits"] = args["given_logits"].to(dev)
    res = moe_rd.route_dispatch(x, w, b, **args)
    torch.cuda.synchronize()
    return res


def to_np(res):
    d = {}
    for k, v in res._asdict().items():
        if v is None:
            d[k] = None
        elif v.dtype == torch.bfloat16:
            d[k] = v.cpu().view(torch.int16).numpy().view(np.uint16)
        else:
            d[k] = v.cpu().numpy()
    return d


def assert_parity(got: dict, ref: dict, *, weight_rtol=1e-6, exact_weights=True):
    """Bit-exact: expert ids, counts, offsets, inverse permutation, drop mask,
    row copies (bf16 or fp8 bytes) and fp8 scales.  Combine weights: 1e-6
    relative (and, where the gate order is fixed, bit-exact as well)."""
    E = ref["offsets"].shape[0] - 1
    np.testing.assert_array_equal(got["expert_ids"], ref["expert_ids"], err_msg="expert_ids")
    np.testing.assert_array_equal(got["counts"], ref["counts"], err_msg="counts")
    np.testing.assert_array_equal(got["offsets"], ref["offsets"], err_msg="offsets")
    np.testing.assert_array_equal(got["inverse_perm"], ref["inverse_perm"], err_msg="inverse_perm")
    np.testing.assert_array_equal(got["drop_mask"], ref["drop_mask"], err_msg="drop_mask")
    R = int(ref["offsets"][E])
    np.testing.assert_array_equal(got["permuted"][:R], ref["permuted"][:R], err_msg="permuted rows")
    if ref["scales"] is not None:
        np.testing.assert_array_equal(got["scales"][:R].view(np.uint32), ref["scales"][:R].view(np.uint32),
                                      err_msg="fp8 scales")
    np.testing.assert_allclose(got["combine_weights"], ref["combine_weights"], rtol=weight_rtol, atol=0,
                               err_msg="combine_weights")
    if exact_weights:
        np.testing.assert_array_equal(got["combine_weights"].view(np.uint32),
                                      ref["combine_weights"].view(np.uint32), err_msg="combine_weights bits")


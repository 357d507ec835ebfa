"""The call is stream-ordered without allocation or host synchronisation, so it can be recorded into a CUDA
graph: a replay on refilled input buffers must give exactly what the plain call gives."""
import numpy as np
import pytest
import torch

from moe_rd import workloads
from moe_rd.runtime import Session
import _util

pytestmark = pytest.mark.gpu

KEYS = ("score_fn", "bias_mode", "n_groups", "topk_groups", "group_topk", "renorm", "routed_scale", "capacity",
        "rows_format", "w_layout")


def _snapshot(res):
    return {k: (None if v is None else v.clone()) for k, v in res._asdict().items()}


@pytest.mark.parametrize("name,T,H", [("c1", 512, 1024),      # fused GEMV gate (memset + 3 kernels)
                                      ("c4", 2048, 7168),     # two-CTA tcgen05 gate, fp8 rows
                                      ("ref", 4096, 2048),    # weight split + tcgen05 gate + fold
                                      ("c3", 24100, 512)])    # gate and routing in one kernel, capacity drops
def test_graph_replay_equals_plain_call(name, T, H):
    dev = torch.device("cuda:0")
    t, kw = workloads.make(name, T=T, H=H)
    if name == "c3":
        kw = dict(kw, capacity=int(np.ceil(1.25 * T * kw["top_k"] / 128)))
    spec = workloads.SPECS[name]
    sess = Session(T, H, spec["E"], spec["K"], device=dev, w_dtype=t["w"].dtype,
                   **{k: v for k, v in kw.items() if k in KEYS})
    x = t["x"].to(dev)
    w = t["w"].to(dev)
    b = None if t["bias"] is None else t["bias"].to(dev)
    graph = sess.capture(x, w, b)
    # new tokens in the same buffer: the graph must read them, not what it saw while recording
    x.copy_(workloads.make(name, T=T, H=H, rank=3)[0]["x"])
    graph.replay()
    torch.cuda.synchronize()
    assert sess.status()[0] == 0
    replayed = _snapshot(sess.result())
    plain = _snapshot(sess.run(x, w, b))
    torch.cuda.synchronize()
    R = int(plain["offsets"][-1])
    for k, v in plain.items():
        if v is None:
            continue
        a, c = (replayed[k][:R], v[:R]) if k in ("permuted", "scales") else (replayed[k], v)
        assert torch.equal(a.view(torch.uint8) if a.dtype == torch.bfloat16 else a,
                           c.view(torch.uint8) if c.dtype == torch.bfloat16 else c), k
    # and it is the right answer, not merely the same one
    ref = _util.run_oracle(dict(t, x=x.cpu()), kw, given_logits=None) if name == "c1" else None
    if ref is not None:
        np.testing.assert_array_equal(plain["expert_ids"].cpu().numpy(), ref["expert_ids"])
        np.testing.assert_array_equal(plain["inverse_perm"].cpu().numpy(), ref["inverse_perm"])

"""The expert-parallel peer-store exchange with every rank's buffers on ONE GPU.

The exchange kernels take plain device pointers for the owners' buffers, so W
ranks can be played one after another in one process on one device: rank r
routes its own tokens, the kept counts of all ranks are stacked (what the
all-gather delivers), every rank runs the plan kernel and then its scatter
kernel into the W receive buffers, and every owner runs the replicate kernel.
No kernel waits on another, so running them in sequence is the same
computation.  Each owner's buffer must equal, bit for bit, the single-process
statement of the exchange in the CPU oracle - with every pair carrying its row
and with the send-once form (a token crosses to a rank once, later pairs are
copied by the owner), in both fp8 layouts and for bf16 rows, twice in a row
(the marks must be back at -1)."""
import ctypes

import numpy as np
import pytest
import torch

from moe_rd import _cabi, workloads
from moe_rd.runtime import Session
from oracle import cpu_oracle
import _util

pytestmark = pytest.mark.gpu
E, K = 256, 8


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _ptr_array(ts):
    return (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


@pytest.mark.parametrize("world,fmt,layout,once", [(2, "fp8", "packed", True), (4, "fp8", "packed", True),
                                                  (8, "fp8", "separate", True), (4, "fp8", "packed", False),
                                                  (2, "bf16", "separate", True), (4, "bf16", "separate", False)])
def test_exchange_of_w_ranks_on_one_device(world, fmt, layout, once):
    dev = torch.device("cuda:0")
    H, T0 = 1024, 300
    L = _cabi.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    fp8 = fmt == "fp8"
    epr = E // world
    sessions, inputs, oracle_in = [], [], []
    for r in range(world):
        T = T0 + 64 * r                       # ragged: ranks hold different token counts
        t, kw = workloads.make("c5", T=T, H=H, rank=r)
        kw = dict(kw, rows_format=fmt)
        s = Session(T, H, E, K, device=dev, score_fn="sigmoid", bias_mode="select", n_groups=8, topk_groups=4,
                    group_topk=2, routed_scale=2.5, rows_format=fmt, return_logits=True, scatter_impl="none")
        sessions.append(s)
        inputs.append((t["x"].to(dev), t["w"].to(dev), t["bias"].to(dev)))
        oracle_in.append((t, kw))
    max_rows = world * (T0 + 64 * world) * K
    nb = H // 128
    pitch = (H + nb * 4) if (fp8 and layout == "packed") else (H if fp8 else 2 * H)
    rows = [torch.zeros(max_rows * pitch, dtype=torch.uint8, device=dev) for _ in range(world)]
    scales = ([torch.zeros((max_rows, nb), dtype=torch.float32, device=dev) for _ in range(world)]
              if fp8 and layout == "separate" else None)
    copy_of = [torch.full((max_rows,), -1, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    plans = [dict(dest_base=torch.empty(E, dtype=torch.int32, device=dev),
                  cnt=torch.empty((world, epr), dtype=torch.int32, device=dev),
                  local_offsets=torch.empty(epr + 1, dtype=torch.int32, device=dev)) for _ in range(world)]
    sent_rows = marks = 0
    for step in range(2):
        for s, (x, w, b) in zip(sessions, inputs):
            s.run(x, w, b)
        kept_all = torch.stack([(s.offsets[1:] - s.offsets[:-1]) for s in sessions]).contiguous()
        for r in range(world):
            p = plans[r]
            _cabi.check(L.moe_rd_ep_plan(_ptr(kept_all), world, r, E, max_rows, _ptr(p["dest_base"]), _ptr(p["cnt"]),
                                         _ptr(p["local_offsets"]), _ptr(status), stream))
        for r, (s, (x, w, b)) in enumerate(zip(sessions, inputs)):
            params = _cabi.Params.from_buffer_copy(s.params)
            params.scatter_impl = _cabi.SCATTER_IMPL["bulk"]
            args = (ctypes.byref(params), _ptr(x), _ptr(s.expert_ids), _ptr(s.inverse_perm), _ptr(s.offsets),
                    _ptr(plans[r]["dest_base"]), world)
            peers = (_ptr_array(rows), None if scales is None else _ptr_array(scales))
            if once:
                _cabi.check(L.moe_rd_ep_scatter_once(*args, r, *peers, _ptr_array(copy_of), _ptr(status), stream))
            else:
                _cabi.check(L.moe_rd_ep_scatter(*args, *peers, _ptr(status), stream))
        if once and step == 0:
            torch.cuda.synchronize()
            marks = sum(int((c >= 0).sum()) for c in copy_of)
            marks_seen = [c.cpu().numpy() for c in copy_of]
        for r in range(world):
            if once:
                params = _cabi.Params.from_buffer_copy(sessions[r].params)
                n_rows = ctypes.c_void_p(plans[r]["local_offsets"].data_ptr() + 4 * epr)
                _cabi.check(L.moe_rd_ep_replicate(ctypes.byref(params), _ptr(rows[r]),
                                                  None if scales is None else _ptr(scales[r]), _ptr(copy_of[r]),
                                                  n_rows, max_rows, _ptr(status), stream))
        torch.cuda.synchronize()
        assert int(status[0]) == 0, status.tolist()
        for c in copy_of:
            assert int((c >= 0).sum()) == 0      # every mark consumed and reset
        if step == 0:
            for rbuf in rows:                    # the second round must not live on the first one's bytes
                rbuf.zero_()
            continue
        per = [_util.run_oracle(t, kw, given_logits=s.router_logits.cpu().numpy())
               for (t, kw), s in zip(oracle_in, sessions)]
        ref = cpu_oracle.ep_exchange(per, E, world)
        for d in range(world):
            n = ref[d]["rows"].shape[0]
            sent_rows += n
            assert int(plans[d]["local_offsets"][-1]) == n
            np.testing.assert_array_equal(plans[d]["cnt"].cpu().numpy(), ref[d]["counts"])
            img = rows[d].view(max_rows, pitch)[:n].cpu()
            if fp8:
                np.testing.assert_array_equal(img[:, :H].numpy(), ref[d]["rows"])
                got_s = (img[:, H:].contiguous().view(torch.float32) if layout == "packed" else scales[d][:n].cpu())
                np.testing.assert_array_equal(got_s.numpy().view(np.uint32), ref[d]["scales"].view(np.uint32))
            else:
                np.testing.assert_array_equal(img.contiguous().view(torch.int16).numpy().view(np.uint16),
                                              ref[d]["rows"])
    if once:
        # one mark for every kept pair beyond a token's first on a REMOTE rank, none for the rank itself
        expected = 0
        for r, o in enumerate(per):
            owner = o["expert_ids"] // epr
            kept = o["inverse_perm"] >= 0
            for d in range(world):
                if d != r:
                    expected += int(np.maximum(((owner == d) & kept).sum(axis=1) - 1, 0).sum())
        assert marks == expected, (marks, expected)
        # and each mark names the row of the token's first pair on that rank
        for got, want in zip(marks_seen, cpu_oracle.ep_send_once_marks(per, E, world, max_rows)):
            np.testing.assert_array_equal(got, want)
        # group-limited routing: 8 experts from at most 4 groups; with 32 experts per group a rank owns
        # 8 / world groups, so a good part of the remote pairs repeat a rank
        assert marks > 0.2 * sent_rows * (world - 1) / world, (marks, sent_rows)

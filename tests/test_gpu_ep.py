"""Expert-parallel dispatch (and, for the fused form, the combine that pulls
rows back) on real GPUs (needs >= 2): every rank routes its
own seeded tokens, the ranks exchange counts, rows and scales over NCCL, and
each rank's expert-major buffer must equal, bit for bit, the single-process
statement of the exchange in the CPU oracle (fp8 rows and scales; tensor-core
gate, so the oracle is given each rank's GPU logits)."""
import datetime
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T0, H, mode, q):
    try:
        sys.path[:0] = [str(ROOT), str(ROOT / "ernie-evolve-results_b200"), str(ROOT / "tests")]
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=120))
        from moe_rd import workloads
        from moe_rd.runtime import Session
        from moe_rd.ep import ExpertParallel, ExpertParallelFused
        from oracle import cpu_oracle
        import _util
        E, K = 256, 8
        T = T0 + 64 * rank  # ragged: ranks hold different token counts
        t, kw = workloads.make("c5", T=T, H=H, rank=rank)
        fused = mode.startswith("fused")
        sess = Session(T, H, E, K, device=dev, score_fn="sigmoid", bias_mode="select", n_groups=8, topk_groups=4,
                       group_topk=2, routed_scale=2.5, rows_format="fp8", return_logits=True,
                       scatter_impl="none" if fused else "auto")
        cls = ExpertParallelFused if fused else ExpertParallel
        kwargs = dict(bulk=True) if mode == "fused_bulk" else {}
        if mode == "fused_symm_sync":
            kwargs = dict(sync="symm")
        ep = cls(sess, max_recv_rows=world * (T0 + 64 * world) * K, **kwargs)
        x, w, b = t["x"].to(dev), t["w"].to(dev), t["bias"].to(dev)
        for _ in range(2):  # twice: buffers are reused
            sess.run(x, w, b)
            out = ep.exchange(x) if fused else ep.exchange()
        torch.cuda.synchronize()
        sess.status()
        # every rank's GPU logits, so that the oracle can restate all ranks
        z = sess.router_logits.cpu()
        sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        gathered = [None] * world
        dist.all_gather_object(gathered, z.numpy())
        per = []
        for r in range(world):
            tr, kwr = workloads.make("c5", T=T0 + 64 * r, H=H, rank=r)
            per.append(_util.run_oracle(tr, kwr, given_logits=gathered[r]))
        ref = cpu_oracle.ep_exchange(per, E, world)[rank]
        n = int(out.offsets[-1].item())
        assert n == ref["rows"].shape[0]
        np.testing.assert_array_equal(out.counts.cpu().numpy(), ref["counts"])
        np.testing.assert_array_equal(out.offsets.cpu().numpy(), ref["offsets"])
        np.testing.assert_array_equal(out.rows[:n].cpu().numpy(), ref["rows"])
        np.testing.assert_array_equal(out.scales[:n].cpu().numpy().view(np.uint32), ref["scales"].view(np.uint32))
        assert int(ep.status[0].item()) == 0
        if fused:
            # Return path: every owner turns its received fp8 bytes into bf16 "expert
            # outputs"; each source rank pulls its rows back over NVLink and combines
            # them.  Expected: the local combine of this rank's own quantised rows.
            y = ep.expert_output_buffer()
            y[:n] = out.rows[:n].to(torch.float32).to(torch.bfloat16)
            got = ep.combine()
            got = ep.combine()  # twice: the barriers keep the buffers consistent
            torch.cuda.synchronize()
            mine = per[rank]
            y_local = torch.from_numpy(mine["permuted"].astype(np.float32)).to(torch.bfloat16)
            y_bits = y_local.view(torch.int16).numpy().view(np.uint16)
            ref_out = cpu_oracle.combine(y_bits, mine["inverse_perm"], mine["combine_weights"])
            np.testing.assert_array_equal(got.cpu().view(torch.int16).numpy().view(np.uint16), ref_out)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-1500:]}"))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("mode", ["nccl", "fused", "fused_bulk", "fused_symm_sync"])
def test_expert_parallel_exchange_matches_oracle(mode):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 300, 1024, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, "ok") for r in range(world)], res

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
        kwargs = {"fused": dict(bulk=False), "fused_bulk": dict(bulk=True),  # rows + scales as one copy per pair
                  "fused_bulk_separate": dict(bulk=True, layout="separate")}.get(mode, {})
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
            ep.check()
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


def _full_size_worker(rank, world, port, q):
    """T=8192 tokens per rank, H=7168, 256 experts, fp8 rows: the measured
    configuration.  The oracle restates this rank's own dispatch at full size; the
    exchange is checked through a property that does not need every rank's rows on
    the host: the one-kernel peer-store exchange must deliver, bit for bit, what
    the NCCL all-to-all plus reorder delivers (that form is compared with the
    oracle's statement of the exchange in the small cases above)."""
    try:
        sys.path[:0] = [str(ROOT), str(ROOT / "ernie-evolve-results_b200"), str(ROOT / "tests")]
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=300))
        from moe_rd import workloads
        from moe_rd.runtime import Session
        from moe_rd.ep import ExpertParallel, ExpertParallelFused
        import _util
        spec = workloads.SPECS["c5"]
        T, H, E, K = spec["T"], spec["H"], spec["E"], spec["K"]
        t, kw = workloads.make("c5", rank=rank)
        common = dict(device=dev, score_fn="sigmoid", bias_mode="select", n_groups=8, topk_groups=4, group_topk=2,
                      routed_scale=2.5, rows_format="fp8", return_logits=True)
        x, w, b = t["x"].to(dev), t["w"].to(dev), t["bias"].to(dev)
        local = Session(T, H, E, K, **common)
        a2a = ExpertParallel(local, max_recv_rows=2 * T * K)
        local.run(x, w, b)
        ref = a2a.exchange()
        n = int(ref.offsets[-1].item())
        # this rank's dispatch against the oracle (given the GPU's logits: tensor-core gate)
        mine = _util.run_oracle(t, kw, given_logits=local.router_logits.cpu().numpy())
        _util.assert_parity(_util.to_np(local.result()), mine)
        ref_rows, ref_scales = ref.rows[:n].clone(), ref.scales[:n].clone()
        ref_offs, ref_cnt = ref.offsets.clone(), ref.counts.clone()
        del a2a
        remote = Session(T, H, E, K, scatter_impl="none", **common)
        for layout in ("packed", "separate"):
            ep = ExpertParallelFused(remote, max_recv_rows=2 * T * K, bulk=True, layout=layout)
            for _ in range(2):
                remote.run(x, w, b)
                out = ep.exchange(x)
            torch.cuda.synchronize()
            ep.check()
            assert int(out.offsets[-1].item()) == n
            assert torch.equal(out.offsets, ref_offs) and torch.equal(out.counts, ref_cnt)
            assert torch.equal(out.rows[:n], ref_rows), layout
            assert torch.equal(out.scales[:n].contiguous().view(torch.int32), ref_scales.view(torch.int32)), layout
            del ep, out
            torch.cuda.empty_cache()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-1500:]}"))


def _small_buffer_worker(rank, world, port, q):
    """A receive buffer far too small for the routed rows: the plan kernel must
    record it (id 202) on every rank, the rows that do not fit must be skipped -
    nothing is stored outside a buffer - and the call must stay usable."""
    try:
        sys.path[:0] = [str(ROOT), str(ROOT / "ernie-evolve-results_b200"), str(ROOT / "tests")]
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=120))
        from moe_rd import workloads, MoeRdError
        from moe_rd.runtime import Session
        from moe_rd.ep import ExpertParallelFused
        T, H, E, K = 512, 1024, 256, 8
        t, kw = workloads.make("c5", T=T, H=H, rank=rank)
        x, w, b = t["x"].to(dev), t["w"].to(dev), t["bias"].to(dev)
        sess = Session(T, H, E, K, device=dev, score_fn="sigmoid", bias_mode="select", n_groups=8, topk_groups=4,
                       group_topk=2, routed_scale=2.5, rows_format="fp8", scatter_impl="none")
        for bulk in (True, False):
            cap = 96  # rows; about T*K = 4096 are bound for every rank
            ep = ExpertParallelFused(sess, max_recv_rows=cap, bulk=bulk)
            sess.run(x, w, b)
            out = ep.exchange(x)
            torch.cuda.synchronize()
            try:
                ep.check()
                raise AssertionError("an undersized receive buffer was not reported")
            except MoeRdError as err:
                assert "202" in str(err), str(err)
            assert int(out.offsets[-1].item()) <= cap
            assert int((ep.dest_base < 0).sum().item()) > 0  # experts without a destination
            got = ep.combine()  # the return path skips the same pairs; it must not read out of bounds
            torch.cuda.synchronize()
            assert got.shape == (T, H)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-1500:]}"))


def _run(target, args_of_rank, world, timeout=900):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=args_of_rank(r) + (q,)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=timeout) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, "ok") for r in range(world)], res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("mode", ["nccl", "fused", "fused_bulk", "fused_bulk_separate"])
def test_expert_parallel_exchange_matches_oracle(mode):
    world = torch.cuda.device_count()  # every visible GPU (256 experts divide over 2, 4 and 8)
    world = 8 if world >= 8 else 4 if world >= 4 else 2
    port = _free_port()
    _run(_worker, lambda r: (r, world, port, 300, 1024, mode), world)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_expert_parallel_full_size_peer_stores_equal_all_to_all():
    world = torch.cuda.device_count()
    world = 8 if world >= 8 else 4 if world >= 4 else 2
    port = _free_port()
    _run(_full_size_worker, lambda r: (r, world, port), world, timeout=1500)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_undersized_receive_buffer_is_reported_and_nothing_is_stored_past_it():
    world = 2
    port = _free_port()
    _run(_small_buffer_worker, lambda r: (r, world, port), world)

"""Host-side logic of the expert-parallel exchange on CPU ranks (gloo,
world_size 2 and 4): counts first, then rows by all-to-all with the split sizes
derived from the counts.  Every rank checks what it received, reordered to
expert-major, against the single-process statement of the exchange in the CPU
oracle.  Also: a rank that disappears makes the others fail with an error
instead of hanging (short process-group timeout)."""
import datetime
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _per_rank_results(world, E, T0):
    sys.path[:0] = [str(ROOT), str(ROOT / "ernie-evolve-results_b200"), str(ROOT / "tests")]
    from moe_rd import workloads
    import _util
    out = []
    for r in range(world):
        t, kw = workloads.make("c4", T=T0 + 7 * r, H=256, rank=r)
        out.append(_util.run_oracle(t, kw))
    return out


def _worker(rank, world, port, T0, q):
    try:
        sys.path[:0] = [str(ROOT), str(ROOT / "ernie-evolve-results_b200"), str(ROOT / "tests")]
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=60))
        from moe_rd import ep
        from oracle import cpu_oracle
        E = 256
        per = _per_rank_results(world, E, T0)
        mine = per[rank]
        offs = torch.from_numpy(mine["offsets"].astype(np.int32))
        kept = offs[1:] - offs[:-1]
        cnt, send_splits, recv_splits = ep.exchange_plan(kept, world)
        rows = torch.from_numpy(mine["permuted"])
        scales = torch.from_numpy(mine["scales"])
        n_recv = sum(recv_splits)
        got_rows = torch.empty((n_recv, rows.shape[1]), dtype=rows.dtype)
        got_scales = torch.empty((n_recv, scales.shape[1]), dtype=scales.dtype)
        ep.exchange_rows(rows, send_splits, recv_splits, got_rows)
        ep.exchange_rows(scales, send_splits, recv_splits, got_scales)
        ref = cpu_oracle.ep_exchange(per, E, world)[rank]
        np.testing.assert_array_equal(cnt.numpy(), ref["counts"])
        # reorder [source][expert] -> [expert][source] (what moe_rd_ep_unpack does on the GPU)
        epr = E // world
        c = cnt.numpy()
        src_start = np.concatenate([[0], np.cumsum(c.reshape(-1))])
        order = []
        for le in range(epr):
            for s in range(world):
                k = s * epr + le
                order.extend(range(src_start[k], src_start[k + 1]))
        np.testing.assert_array_equal(got_rows.numpy()[order], ref["rows"])
        np.testing.assert_array_equal(got_scales.numpy()[order], ref["scales"])
        assert n_recv == ref["rows"].shape[0] == ref["offsets"][-1]
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q.put((rank, f"{type(e).__name__}: {e}"))


@pytest.mark.parametrize("world", [2, 4])
def test_counts_then_rows_exchange_matches_oracle(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 40, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(r, "ok") for r in range(world)], res


def _worker_missing_rank(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=5))
        sys.path[:0] = [str(ROOT / "ernie-evolve-results_b200")]
        from moe_rd import ep
        if rank == 1:
            q.put((rank, "left"))   # leaves between steps, nothing in flight
            q.close()
            q.join_thread()
            os._exit(0)
        kept = torch.ones(8, dtype=torch.int32)
        try:
            ep.exchange_plan(kept, world)
            q.put((rank, "no error"))
        except Exception as e:
            q.put((rank, "error:" + type(e).__name__))
    except Exception as e:  # pragma: no cover
        q.put((rank, f"setup {type(e).__name__}: {e}"))
    q.close()
    q.join_thread()
    os._exit(0)


def test_missing_rank_surfaces_as_error_not_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_missing_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res[1] == "left"
    assert res[0].startswith("error:"), res

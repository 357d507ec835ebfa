"""Expert-parallel dispatch across the GPUs of one box.

Tokens shard by rank, experts shard by rank: rank d owns experts
[d*E/W, (d+1)*E/W).  Every rank routes its own tokens against all E experts
(``moe_rd.route_dispatch`` / ``Session.run``), which leaves its rows
expert-major, i.e. destination-rank-major.  The exchange then is

  1. counts first: an all-to-all of the kept rows per (destination, expert);
  2. rows (and fp8 scales) by NCCL all-to-all with the split sizes from (1);
  3. a local reorder from [source][expert] to [expert][source]
     (``moe_rd_ep_unpack``), so that an expert's rows are contiguous and ordered
     by (source rank, source slot order).

The reference has no expert parallelism; the counts-then-rows shape follows its
row-sharded embedding exchange (nanogpt-speedrun/track-1,
track_1_short/sharded_rows.py:72-103; rows and scales as two exchanges,
ngram_table.py:343-360).
"""
from __future__ import annotations

import ctypes
from typing import NamedTuple, Optional

import torch
import torch.distributed as dist

from . import _cabi


class EPResult(NamedTuple):
    rows: torch.Tensor             # [capacity, H] expert-major; first offsets[-1] rows valid
    scales: Optional[torch.Tensor]
    offsets: torch.Tensor          # [E/W + 1] int32 (device)
    counts: torch.Tensor           # [W, E/W] int32 (device): rows from source s for local expert le
    recv_rows: int                 # rows received (host int)
    sent_off_rank_bytes: int       # bytes this rank sent to other ranks


def exchange_plan(kept: torch.Tensor, world: int, group=None):
    """Counts first.  ``kept`` [E] = rows this rank dispatched per expert.
    Returns (cnt [W, E/W] as received, send_splits, recv_splits) with the
    splits as host lists.  Works on any backend (NCCL on device tensors, gloo
    on CPU tensors); synchronises the host once to read the sizes."""
    epr = kept.numel() // world
    send = kept.reshape(world, epr).contiguous()
    cnt = torch.empty_like(send)
    dist.all_to_all_single(cnt, send, group=group)
    sizes = torch.stack([send.sum(dim=1), cnt.sum(dim=1)]).cpu()
    return cnt, [int(v) for v in sizes[0]], [int(v) for v in sizes[1]]


def exchange_rows(rows: torch.Tensor, send_splits, recv_splits, out: torch.Tensor, group=None):
    """Rows by all-to-all; ``out`` must hold sum(recv_splits) rows."""
    n_send, n_recv = sum(send_splits), sum(recv_splits)
    dist.all_to_all_single(out[:n_recv], rows[:n_send], recv_splits, send_splits, group=group)
    return n_recv


class ExpertParallel:
    """Receive buffers are sized once for the worst case (every rank sends all of
    its T*K rows here), so no allocation happens per exchange."""

    def __init__(self, session, group=None, max_recv_rows: Optional[int] = None):
        self.sess = session
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        E = session.E
        if E % self.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.epr = E // self.world
        dev = session.device
        send_rows = session.permuted.shape[0]
        self.max_rows = int(max_recv_rows if max_recv_rows is not None else self.world * send_rows)
        H = session.H
        self.recv_rows = torch.empty((self.max_rows, H), dtype=session.permuted.dtype, device=dev)
        self.out_rows = torch.empty_like(self.recv_rows)
        if session.scales is not None:
            nb = session.scales.shape[1]
            self.recv_scales = torch.empty((self.max_rows, nb), dtype=torch.float32, device=dev)
            self.out_scales = torch.empty_like(self.recv_scales)
        else:
            self.recv_scales = self.out_scales = None
        self.local_offsets = torch.empty(self.epr + 1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(8, dtype=torch.int32, device=dev)

    def exchange(self, result=None) -> EPResult:
        r = result if result is not None else self.sess.result()
        offs = r.offsets
        kept = offs[1:] - offs[:-1]
        cnt, send_splits, recv_splits = exchange_plan(kept, self.world, self.group)
        n_recv = sum(recv_splits)
        if n_recv > self.max_rows:
            raise RuntimeError(f"expert-parallel receive buffer too small: {n_recv} > {self.max_rows}")
        exchange_rows(r.permuted, send_splits, recv_splits, self.recv_rows, self.group)
        if r.scales is not None:
            exchange_rows(r.scales, send_splits, recv_splits, self.recv_scales, self.group)
        row_bytes = r.permuted.shape[1] * r.permuted.element_size()
        dev = self.recv_rows.device
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

        def ptr(t):
            return None if t is None else ctypes.c_void_p(t.data_ptr())
        _cabi.check(_cabi.lib().moe_rd_ep_unpack(
            ptr(cnt), self.world, self.epr, ptr(self.recv_rows), ptr(self.recv_scales if r.scales is not None else None),
            ptr(self.out_rows), ptr(self.out_scales if r.scales is not None else None), ptr(self.local_offsets),
            row_bytes, 0 if r.scales is None else r.scales.shape[1], self.max_rows, ptr(self.status), stream))
        scale_bytes = 0 if r.scales is None else r.scales.shape[1] * 4
        off_rank = (sum(send_splits) - send_splits[self.rank]) * (row_bytes + scale_bytes)
        return EPResult(self.out_rows, self.out_scales if r.scales is not None else None, self.local_offsets, cnt,
                        n_recv, off_rank)


class ExpertParallelFused:
    """Expert-parallel dispatch without a send buffer: after the counts are
    gathered, ONE kernel reads each token row once and stores it straight into
    the owner's expert-major buffer over NVLink (peer stores, no multicast),
    already at its final row, so there is no receive-side reorder.
    Use a ``Session(..., scatter_impl="none")``.

    The receive buffers live in symmetric memory (torch's intra-node peer
    mapping) and are sized once, ``max_recv_rows`` rows on every rank (default:
    the worst case, every rank sending all its rows here).  ``exchange``
    synchronises nothing on the host: all-gather of the counts (NCCL; it is also
    the barrier that protects the previous step's buffers), plan kernel, scatter
    kernel, and a one-element all-reduce that orders every rank's stores before
    anyone reads its buffer.  NCCL's collectives end with an error, through the
    process group's timeout, when a rank never arrives; no kernel here waits on
    another rank.

    ``layout``: "packed" (fp8 rows moved by bulk copies, the default there): a
    received row is H bytes followed by its H/128 scales, so a pair crosses
    NVLink as one copy; ``rows`` and ``scales`` are strided views of that
    buffer.  "separate": rows and scales in two dense buffers (two copies per
    pair).  Both hold the same values.

    ``send_once`` (default with bulk copies): a token with several experts on one
    remote rank crosses NVLink once.  The first of its pairs there carries the
    row; for the others the sender stores a 4-byte mark in the owner's memory
    and, after the barrier, the owner copies the row inside its own buffer
    (``moe_rd_ep_replicate``).  The buffers end up bit for bit the same; with
    group-limited routing the NVLink bytes drop to a half (8 ranks) or a quarter
    (2 ranks).  ``send_once=False``: every pair carries its row.

    If the rows bound for some rank exceed ``max_recv_rows``, the plan kernel
    records it (``check()`` raises) and the experts that do not fit receive
    nothing; no store or load leaves a buffer.
    """

    def __init__(self, session, group=None, max_recv_rows: Optional[int] = None,
                 bulk: Optional[bool] = None, layout: Optional[str] = None, send_once: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem
        # Whole-row bulk copies (cp.async.bulk through shared memory) measured ~7 % more NVLink
        # bandwidth than 16-byte stores; they need 16-byte aligned scale rows (H % 512 == 0).
        H = session.H
        img = (H + (H // 128) * 4 + 127) // 128 * 128
        ok = (H % 512 == 0 and 2 * img <= 200 * 1024) if session.fp8 else (H * 4 + 64 <= 200 * 1024)
        if bulk and not ok:
            raise ValueError("bulk expert-parallel scatter is not available for this row size")
        self.bulk = ok if bulk is None else bulk
        if layout is None:
            layout = "packed" if (self.bulk and session.fp8) else "separate"
        if layout not in ("packed", "separate"):
            raise ValueError("layout must be 'packed' or 'separate'")
        if layout == "packed" and not (self.bulk and session.fp8):
            raise ValueError("the packed layout needs fp8 rows moved by bulk copies")
        self.layout = layout
        self.sess = session
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        E, K, T, H = session.E, session.K, session.T, session.H
        if E % self.world or self.world > 8:
            raise ValueError("experts must divide evenly over at most 8 ranks")
        self.epr = E // self.world
        dev = session.device
        self.fp8 = session.fp8
        self.row_bytes = H * (1 if self.fp8 else 2)
        self.nb = H // 128 if self.fp8 else 0
        per_rank = T * K if not session.params.capacity else min(T * K, E * session.params.capacity)
        self.max_rows = int(max_recv_rows if max_recv_rows is not None else self.world * per_rank)
        if layout == "packed":
            pitch = self.row_bytes + self.nb * 4
            self.buf = symm_mem.empty(self.max_rows * pitch, dtype=torch.uint8, device=dev)
            self.hdl = symm_mem.rendezvous(self.buf, self.group)
            ptrs = [int(p) for p in self.hdl.buffer_ptrs]
            self.peer_rows = (ctypes.c_void_p * self.world)(*ptrs)
            self.peer_scales = None
            img2d = self.buf.view(self.max_rows, pitch)
            self.rows = img2d[:, :H]
            self.scales = img2d[:, H:].view(torch.float32)
        else:
            rows_bytes = (self.max_rows * self.row_bytes + 255) // 256 * 256
            total = rows_bytes + self.max_rows * self.nb * 4
            self.buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
            self.hdl = symm_mem.rendezvous(self.buf, self.group)
            ptrs = [int(p) for p in self.hdl.buffer_ptrs]
            self.peer_rows = (ctypes.c_void_p * self.world)(*ptrs)
            self.peer_scales = (ctypes.c_void_p * self.world)(*[p + rows_bytes for p in ptrs])
            rows_u8 = self.buf[: self.max_rows * self.row_bytes]
            self.rows = (rows_u8 if self.fp8 else rows_u8.view(torch.bfloat16)).view(self.max_rows, H)
            self.scales = (self.buf[rows_bytes: rows_bytes + self.max_rows * self.nb * 4].view(torch.float32)
                           .view(self.max_rows, self.nb)) if self.fp8 else None
        # send-once: a token with several experts on one remote rank crosses NVLink once; the owner copies
        # the row for the later pairs locally (4-byte marks in copy_of, then moe_rd_ep_replicate)
        if send_once and not self.bulk:
            raise ValueError("send_once needs rows moved by bulk copies")
        self.send_once = self.bulk if send_once is None else bool(send_once)
        self.peer_copy_of = None
        if self.send_once:
            self.copy_of = symm_mem.empty(max(self.max_rows, 1), dtype=torch.int32, device=dev)
            self.copy_of.fill_(-1)
            self.copy_hdl = symm_mem.rendezvous(self.copy_of, self.group)
            self.peer_copy_of = (ctypes.c_void_p * self.world)(*[int(p) for p in self.copy_hdl.buffer_ptrs])
            torch.cuda.synchronize(dev)
            dist.barrier(group=self.group)   # every rank's marks read -1 before anyone stores one
        self.kept_all = torch.empty((self.world, E), dtype=torch.int32, device=dev)
        self.dest_base = torch.empty(E, dtype=torch.int32, device=dev)
        self.cnt = torch.empty((self.world, self.epr), dtype=torch.int32, device=dev)
        self.local_offsets = torch.empty(self.epr + 1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(8, dtype=torch.int32, device=dev)
        self.token = torch.zeros(1, dtype=torch.int32, device=dev)

    def exchange(self, x: torch.Tensor, result=None) -> EPResult:
        r = result if result is not None else self.sess.result()
        offs = r.offsets
        dev = self.buf.device
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

        def ptr(t):
            return ctypes.c_void_p(t.data_ptr())
        L = _cabi.lib()
        # the count exchange is also a barrier: nobody overwrites a buffer its owner may still be reading
        kept = (offs[1:] - offs[:-1]).contiguous()
        dist.all_gather_into_tensor(self.kept_all, kept, group=self.group)
        _cabi.check(L.moe_rd_ep_plan(ptr(self.kept_all), self.world, self.rank, self.sess.E, self.max_rows,
                                     ptr(self.dest_base), ptr(self.cnt), ptr(self.local_offsets), ptr(self.status),
                                     stream))
        params = self.sess.params
        if self.bulk:
            params = _cabi.Params.from_buffer_copy(self.sess.params)
            params.scatter_impl = _cabi.SCATTER_IMPL["bulk"]
        if self.send_once:
            _cabi.check(L.moe_rd_ep_scatter_once(ctypes.byref(params), ptr(x), ptr(r.expert_ids),
                                                 ptr(r.inverse_perm), ptr(offs), ptr(self.dest_base), self.world,
                                                 self.rank, self.peer_rows, self.peer_scales, self.peer_copy_of,
                                                 ptr(self.status), stream))
        else:
            _cabi.check(L.moe_rd_ep_scatter(ctypes.byref(params), ptr(x), ptr(r.expert_ids),
                                            ptr(r.inverse_perm), ptr(offs), ptr(self.dest_base), self.world,
                                            self.peer_rows, self.peer_scales, ptr(self.status), stream))
        self._barrier()  # every rank's stores are done and visible after this
        if self.send_once:
            # rows that did not cross NVLink: copies of an earlier row of the same token in this buffer
            _cabi.check(L.moe_rd_ep_replicate(
                ctypes.byref(params), ptr(self.buf), None if self.layout == "packed" or not self.fp8
                else ctypes.c_void_p(self.scales.data_ptr()), ptr(self.copy_of),
                ctypes.c_void_p(self.local_offsets.data_ptr() + 4 * self.epr), self.max_rows, ptr(self.status),
                stream))
        return EPResult(self.rows, self.scales, self.local_offsets, self.cnt, -1, -1)

    def _barrier(self) -> None:
        dist.all_reduce(self.token, group=self.group)

    def check(self) -> None:
        """Reads the device status block of this object's kernels (synchronises)
        and raises if one of them recorded a failed check, e.g. id 202: the rows
        bound for a rank exceed ``max_recv_rows``."""
        st = [int(v) for v in self.status.cpu()]
        if st[0] != 0:
            self.status.zero_()
            raise _cabi.MoeRdError(-9, f"device status {st}")

    def expert_output_buffer(self) -> torch.Tensor:
        """[max_recv_rows, H] bf16 in symmetric memory: the experts of this rank
        write their outputs here, row i for received row i, before ``combine``."""
        if getattr(self, "y", None) is None:
            import torch.distributed._symmetric_memory as symm_mem
            H = self.sess.H
            self.y_buf = symm_mem.empty(self.max_rows * H, dtype=torch.bfloat16, device=self.buf.device)
            self.y_hdl = symm_mem.rendezvous(self.y_buf, self.group)
            self.peer_y = (ctypes.c_void_p * self.world)(*[int(p) for p in self.y_hdl.buffer_ptrs])
            self.y = self.y_buf.view(self.max_rows, H)
        return self.y

    def combine(self, result=None, shared: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out[t] = shared[t] + sum_k w[t,k] * y_owner[row of (t,k)]: the return
        exchange and the un-permute in one kernel that pulls each row from the
        rank that owns its expert (``expert_output_buffer`` there) over NVLink.
        Call on every rank (collective): a one-element all-reduce before the
        kernel orders it after every rank's expert outputs, one after it keeps the
        buffers from being overwritten while a peer still reads them."""
        r = result if result is not None else self.sess.result()
        self.expert_output_buffer()
        T, K, H, E = self.sess.T, self.sess.K, self.sess.H, self.sess.E
        dev = self.buf.device
        out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        self._barrier()
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

        def ptr(t):
            return None if t is None else ctypes.c_void_p(t.data_ptr())
        sh = None if shared is None else shared.reshape(T, H).contiguous()
        _cabi.check(_cabi.lib().moe_rd_ep_combine(
            T, H, K, E, self.world, self.peer_y, ptr(r.expert_ids), ptr(r.inverse_perm), ptr(r.combine_weights),
            ptr(r.offsets), ptr(self.dest_base), ptr(sh), ptr(out), stream))
        self._barrier()
        return out

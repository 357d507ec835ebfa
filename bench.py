#!/usr/bin/env python
"""Benchmark of the MoE routing-and-dispatch path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5] [--impl ours|reference]

One "step" is one pass of the whole path (gate logits -> scoring/top-k ->
histogram/scan -> row scatter [-> expert-parallel exchange at N > 1]) over one
batch of seeded synthetic tokens.  Rank 0 prints ONE JSON line.

* ``value``: routed tokens/s, whole job, inputs resident in HBM, device time
  from CUDA events around every step on the launching stream (L2 flushed by a
  256 MiB write between steps), max over ranks.
* ``e2e``: the same metric through the public callable with HOST buffers:
  pinned-host tokens copied in and every output copied back inside the timed
  region.
* ``roofline``: the row-scatter kernel (dominant), algorithmic bytes / its
  device time, against the measured HBM copy bandwidth of this pool.
* ``cpu_baseline`` / ``--impl reference``: the CPU oracle (a port of the
  reference's algorithm; the reference has no CPU implementation of this path)
  on all of the box's host cores.
* ``other_workloads`` (N = 1): a few steps of the other single-GPU workloads, and
  ``gate_vs_cublas``: the gate stage beside ``torch.mm`` (cuBLAS, bf16 x bf16 ->
  fp32) on the same operands - a comparison leg, never on the product path.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path[:0] = [str(ROOT), str(ROOT / "ernie-evolve-results_b200")]

# dram__bytes_read.sum + dram__bytes_write.sum of one scatter_kernel launch at the full workload, read once
# from a stored ncu capture of that kernel (it is not re-measured by this script; the JSON line says so).
# Below the algorithmic bytes: part of x is still in L2 from the gate pass and the last written lines have
# not left L2 when the kernel ends.
NCU_SCATTER_TRAFFIC = {"c2": 346.879e6, "c3": 1019.949e6, "c4": 546.921e6, "c5": 546.921e6, "ref": 1152.398e6}

METRIC = "routed_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def measured_hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def session_kwargs(kw):
    out = {k: v for k, v in kw.items() if k in ("score_fn", "bias_mode", "n_groups", "topk_groups", "group_topk",
                                                  "renorm", "routed_scale", "norm_min", "capacity", "rows_format",
                                                  "w_layout")}
    return out


def cpu_pass(tensors, kw, ranks=1, E=None):
    """One full pass of the path on the CPU oracle (all ranks' tokens; EP exchange simulated for ranks > 1)."""
    from oracle import cpu_oracle
    from moe_rd import workloads
    import numpy as np
    import torch

    def bits(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    per = []
    for r in range(ranks):
        t = tensors[r]
        w = t["w"].numpy() if t["w"].dtype == torch.float32 else bits(t["w"])
        per.append(cpu_oracle.route_dispatch(bits(t["x"]), w, **workloads.oracle_kwargs(kw, t["bias"])))
    if ranks > 1:
        cpu_oracle.ep_exchange(per, E, ranks)
    return per


def time_cpu(name, ranks, budget_s=12.0, max_passes=3, T=None):
    from oracle import cpu_oracle
    from moe_rd import workloads
    cpu_oracle.lib()
    cpu_oracle.set_threads(os.cpu_count() or 1)
    cores = cpu_oracle.max_threads()
    tensors, kw = [], None
    for r in range(ranks):
        t, kw = workloads.make(name, rank=r, T=T)
        tensors.append(t)
    E = workloads.SPECS[name]["E"]
    Tn = tensors[0]["x"].shape[0]
    times = []
    t_start = time.perf_counter()
    while len(times) < max_passes and (not times or time.perf_counter() - t_start < budget_s):
        t0 = time.perf_counter()
        cpu_pass(tensors, kw, ranks, E)
        times.append(time.perf_counter() - t0)
    best = statistics.median(times)
    return {"value": ranks * Tn / best, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{len(times)} full passes of {name} ({ranks} x {Tn} tokens), median",
            "seconds_per_pass": best}


def run_reference(args, rank, world):
    if rank != 0:
        return
    name = args.workload
    from moe_rd import workloads
    spec = workloads.SPECS[name]
    from oracle import cpu_oracle
    cpu_oracle.lib()
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: ask for every host core explicitly
    cpu_oracle.set_threads(os.cpu_count() or 1)
    tensors, kw = [], None
    for r in range(world):
        t, kw = workloads.make(name, rank=r)
        tensors.append(t)
    E, T = spec["E"], spec["T"]
    t0 = time.perf_counter()
    cpu_pass(tensors, kw, world, E)  # warm-up pass, also sizes the sample
    first = time.perf_counter() - t0
    budget = 180.0
    if first * args.steps > budget:  # bounded sample: the leading tokens of every rank
        T = max(128, int(T * budget / (first * args.steps)) // 128 * 128)
        for t in tensors:
            t["x"] = t["x"][:T].contiguous()
        if "capacity" in kw and kw["capacity"]:
            kw = dict(kw, capacity=int(-(-1.25 * T * spec["K"] // E)))
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        cpu_pass(tensors, kw, world, E)
        times.append(time.perf_counter() - t0)
    total = sum(times)
    value = world * T * len(times) / total
    cores = cpu_oracle.max_threads()
    cfg = workload_config(name, spec, world)
    if T != spec["T"]:
        # bounded sample: say what was really processed per rank
        cfg["tokens_per_rank"] = T
        cfg["sample_of_tokens_per_rank"] = spec["T"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{len(times)} full passes of {name} ({world} x {T} tokens) on {cores} threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference project has no CPU implementation of this path; this is the CPU oracle "
                "(a port of the algorithm read from its CUDA source), OpenMP over all host threads",
    }
    print(json.dumps(line), flush=True)


def workload_config(name, spec, world):
    return {"workload": name, "tokens_per_rank": spec["T"], "hidden": spec["H"], "experts": spec["E"],
            "top_k": spec["K"], "experts_per_rank": spec["E"] // world if name == "c5" else spec["E"],
            "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": "flushed by a 256 MiB device write between steps"}


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import moe_rd
    from moe_rd import workloads, _cabi
    from moe_rd.runtime import Session

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the routing/dispatch path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    name = args.workload
    spec = workloads.SPECS[name]
    tensors, kw = workloads.make(name, rank=rank)
    T, H, E, K = spec["T"], spec["H"], spec["E"], spec["K"]
    x = tensors["x"].to(dev)
    w = tensors["w"].to(dev)
    bias = None if tensors["bias"] is None else tensors["bias"].to(dev)
    fused = world > 1 and args.ep == "fused"
    sess = Session(T, H, E, K, device=dev, w_dtype=w.dtype, scatter_impl="none" if fused else args.scatter,
                   **session_kwargs(kw))
    ep = None
    if world > 1:
        from moe_rd.ep import ExpertParallel, ExpertParallelFused
        ep = (ExpertParallelFused(sess, dist.group.WORLD,
                                  bulk={"auto": None, "bulk": True, "simt": False}[args.scatter],
                                  layout=args.ep_layout, send_once=False if args.ep_every_pair else None) if fused
              else ExpertParallel(sess, dist.group.WORLD))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        sess.run(x, w, bias)
        if ep is not None:
            ep.exchange(x) if fused else ep.exchange()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    barrier()
    sess.status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # nvidia-smi needs a moment to start and samples every 100 ms: keep the same
    # load running (untimed, on every rank alike) until it has seen clocks under load.
    t_hold = time.perf_counter()
    while True:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
        more = torch.tensor([1 if time.perf_counter() - t_hold < 1.5 else 0], device=dev)
        if world > 1:
            dist.broadcast(more, src=0)
        if int(more.item()) == 0:
            break
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = _cabi.launch_count()
    barrier()
    for s, e in ev:
        flush.zero_()
        s.record()
        step()
        e.record()
    barrier()
    launches = _cabi.launch_count() - launches0
    times = [s.elapsed_time(e) for s, e in ev]
    total_ms = torch.tensor([sum(times)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    value = world * T * args.steps / (total_ms / 1e3)

    # --- spread of the timed steps on this rank, and the same call with a warm L2 (no flush in between)
    st = sorted(times)
    pct = lambda q: st[min(len(st) - 1, max(0, int(round(q * (len(st) - 1)))))]  # noqa: E731
    evw = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for s, e in evw:
        s.record()
        step()
        e.record()
    barrier()
    warm = [s.elapsed_time(e) for s, e in evw]
    timing = {"cold_l2_ms": {"mean": sum(times) / len(times), "median": statistics.median(times),
                             "p10": pct(0.1), "p90": pct(0.9)},
              "warm_l2_ms": {"mean": sum(warm) / len(warm), "median": statistics.median(warm)},
              "note": "this rank's steps; value and ms_per_step use the cold-L2 mean, max over ranks"}
    if world == 1:
        # the same call recorded once into a CUDA graph and replayed (one submission per step), cold L2
        timing["graph_replay_cold_l2_ms"] = graph_replay_ms(sess, x, w, bias, flush, args.steps)

    # --- per-stage device times for the roofline of the dominant kernel (row scatter)
    stage = []
    for _ in range(min(args.steps, 10)):
        flush.zero_()
        stage.append(sess.run_timed(x, w, bias))
    stage_ms = [statistics.mean(s[i] for s in stage) for i in range(5)]
    kept = int(sess.offsets[-1].item())
    fp8 = kw.get("rows_format", "bf16") == "fp8"
    row_bytes = H * (1 if fp8 else 2) + ((H // 128) * 4 if fp8 else 0)
    scatter_bytes = T * H * 2 + kept * row_bytes + T * K * 4
    op_bytes = workloads.algorithmic_bytes(T, H, E, K, w_bytes=w.element_size(), fp8=fp8, kept_rows=kept)
    peak, peak_kind = measured_hbm_peak()
    op_ms = total_ms / args.steps
    whole = {"algorithmic_bytes": op_bytes, "ms": op_ms, "achieved": op_bytes / (op_ms * 1e-3) / 1e9,
             "frac_of_measured": op_bytes / (op_ms * 1e-3) / 1e9 / peak,
             "frac_of_8000": op_bytes / (op_ms * 1e-3) / 1e9 / 8000.0}
    stages = {"gate": stage_ms[0], "route": stage_ms[1], "scan": stage_ms[2], "positions": stage_ms[3],
              "scatter": stage_ms[4]}
    nvlink = None
    if world > 1:
        # the exchange alone, and the bytes that really left this GPU
        # (median of 9, the ranks aligned before each sample: the first collective of the exchange otherwise
        # also measures how far apart the ranks happen to be)
        evx = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(9)]
        for s_, e_ in evx:
            flush.zero_()
            sess.run(x, w, bias)
            dist.all_reduce(torch.zeros(1, device=dev))
            s_.record()
            ep.exchange(x) if fused else ep.exchange()
            e_.record()
        torch.cuda.synchronize()
        ex_ms = statistics.median(s_.elapsed_time(e_) for s_, e_ in evx)
        offs = sess.offsets.cpu()
        epr = E // world
        send_once = bool(getattr(ep, "send_once", False))
        # bytes this rank sends to every rank d: one row per kept pair, or, with the send-once exchange, one row
        # per (token, rank) that has a kept pair there plus a 4-byte mark for each further pair
        owner = (sess.expert_ids // epr).to(torch.int64)
        valid = sess.inverse_perm >= 0
        sent = torch.zeros(world, dtype=torch.float64, device=dev)
        for d in range(world):
            per_token = ((owner == d) & valid).sum(dim=1)
            if send_once:
                sent[d] = float((per_token > 0).sum()) * row_bytes + float((per_token - 1).clamp_min(0).sum()) * 4
            else:
                sent[d] = float(per_token.sum()) * row_bytes
        sent_all = [torch.empty_like(sent) for _ in range(world)]
        dist.all_gather(sent_all, sent)
        egress = float(sum(float(sent[d]) for d in range(world) if d != rank))
        # bytes this rank RECEIVES from the other ranks (routing can load the owners unevenly)
        ingress = float(sum(float(v[rank]) for r_, v in enumerate(sent_all) if r_ != rank))
        all_pairs_egress = float((int(offs[E]) - int(offs[(rank + 1) * epr] - offs[rank * epr])) * row_bytes)
        red = torch.tensor([ex_ms, egress, op_ms, ingress, all_pairs_egress], dtype=torch.float64, device=dev)
        dist.all_reduce(red, op=dist.ReduceOp.MAX)
        ex_ms, egress, step_ms, ingress_max, all_pairs_egress = (float(v) for v in red)
        mean = torch.tensor([ingress], dtype=torch.float64, device=dev)
        dist.all_reduce(mean, op=dist.ReduceOp.SUM)
        ingress_mean = float(mean.item()) / world
        link_gbs = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool (900 nominal)
        wire = max(egress, ingress_max)  # the busiest direction of the busiest rank bounds the exchange
        roof_ms = max(wire / link_gbs / 1e6, op_bytes / peak / 1e6)
        nvlink = {"egress_bytes_per_rank_max": egress, "ingress_bytes_per_rank_max": ingress_max,
                  "ingress_bytes_per_rank_mean": ingress_mean, "exchange_ms": ex_ms,
                  "exchange_gbs": wire / (ex_ms * 1e-3) / 1e9, "link_peak_gbs": link_gbs,
                  "link_peak_kind": "measured peer copy per direction (900 nominal)",
                  "roofline_ms": roof_ms, "step_ms": step_ms, "frac_of_roofline": roof_ms / step_ms,
                  "frac_of_900": max(wire / 900.0 / 1e6, op_bytes / peak / 1e6) / step_ms, "mode": args.ep,
                  "layout": getattr(ep, "layout", None), "send_once": send_once,
                  "egress_bytes_if_every_pair_crossed": all_pairs_egress}
    clocks = sampler.stop() if rank == 0 else None
    if fused:
        roofline = {"bound": "nvlink",
                    "kernel": "scatter_bulk_fp8_kernel<EP> (cp.async.bulk peer stores)" if ep.bulk
                    else "scatter_kernel<EP> (16-byte peer stores)",
                    "achieved": nvlink["exchange_gbs"], "peak": nvlink["link_peak_gbs"], "unit": "GB/s",
                    "frac": nvlink["exchange_gbs"] / nvlink["link_peak_gbs"],
                    "peak_kind": nvlink["link_peak_kind"], "traffic": None,
                    "bytes_per_launch": max(nvlink["egress_bytes_per_rank_max"], nvlink["ingress_bytes_per_rank_max"]),
                    "kernel_ms": nvlink["exchange_ms"],
                    "stage_ms": stages, "whole_op": whole}
    else:
        scatter_gbs = scatter_bytes / (stage_ms[4] * 1e-3) / 1e9
        roofline = {
            "bound": "hbm", "kernel": "scatter_kernel", "achieved": scatter_gbs, "peak": peak, "unit": "GB/s",
            "frac": scatter_gbs / peak, "peak_kind": f"{peak_kind} HBM copy bandwidth",
            "traffic": NCU_SCATTER_TRAFFIC.get(name),
            "traffic_source": "stored ncu capture of scatter_kernel at this workload, not measured in this run",
            "bytes_per_launch": scatter_bytes,
            "kernel_ms": stage_ms[4], "stage_ms": stages, "whole_op": whole,
        }

    # --- end to end through the public callable with host buffers
    x_host = tensors["x"].pin_memory()
    res0 = moe_rd.route_dispatch(x, w, bias, **kw)
    outs = [t for t in (res0.permuted, res0.scales, res0.offsets, res0.inverse_perm, res0.combine_weights) if t is not None]
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs]
    h2d = x_host.numel() * x_host.element_size()
    d2h = sum(t.numel() * t.element_size() for t in outs)
    del res0
    e2e_steps = max(3, min(args.steps, 10))
    ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(e2e_steps)]
    x_in = torch.empty_like(x)

    def e2e_step():
        x_in.copy_(x_host, non_blocking=True)
        if fused:
            r = moe_rd.route_dispatch(x_in, w, bias, scatter_impl="none", **kw)
            o = ep.exchange(x_in, r)
            src = [t for t in (o.rows, o.scales, r.offsets, r.inverse_perm, r.combine_weights) if t is not None]
            src = [t[:h.shape[0]] if t.dim() == 2 and t.shape[0] > h.shape[0] else t for t, h in zip(src, host_out)]
        else:
            r = moe_rd.route_dispatch(x_in, w, bias, **kw)
            if ep is not None:
                ep.exchange(r)
            src = [t for t in (r.permuted, r.scales, r.offsets, r.inverse_perm, r.combine_weights) if t is not None]
        for h, d in zip(host_out, src):
            h.copy_(d, non_blocking=True)

    for _ in range(2):
        e2e_step()
    barrier()
    for s, e in ev2:
        flush.zero_()
        s.record()
        e2e_step()
        e.record()
    barrier()
    e2e_ms = torch.tensor([sum(s.elapsed_time(e) for s, e in ev2)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = world * T * e2e_steps / (float(e2e_ms.item()) / 1e3)
    e2e_extra = {}
    if world == 1:
        # The same loop as a serving process would run it: copies on streams of their own and two sets of
        # buffers, so that step i's read-back, step i+1's pass and step i+2's upload overlap (PCIe carries
        # both directions at once).  Every step still uploads its inputs from pinned memory, runs the call
        # through the public Session with a cold L2, and reads every output back; only the waiting is gone.
        e2e_extra = {"serial_value": e2e_value,
                     "note": "value: uploads, calls and read-backs of consecutive steps overlapped on three "
                             "streams with two sets of buffers; serial_value: one step at a time on one stream"}
        e2e_value = T * e2e_steps / (pipelined_e2e_ms(sess, Session(T, H, E, K, device=dev, w_dtype=w.dtype,
                                                                    scatter_impl=args.scatter,
                                                                    **session_kwargs(kw)),
                                                      x_host, w, bias, flush, e2e_steps) / 1e3)

    sweep = None
    if world == 1 and not args.no_sweep:
        del sess, x, x_in, x_host, host_out, outs
        torch.cuda.empty_cache()
        sweep = run_sweep(dev, flush, [n for n in ("c1", "c2", "c3", "ref") if n != name], peak)
    line = None
    if rank == 0:
        cpu = time_cpu(name, 1) if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": op_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": workload_config(name, spec, world),
            "roofline": roofline,
            "e2e": dict({"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                         "steps": e2e_steps}, **e2e_extra),
            "gpu_launches": int(launches),
            "nvlink": nvlink,
            "clocks": clocks,
            "kept_rows": kept,
            "timing": timing,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if sweep is not None:
            line["other_workloads"] = sweep["other_workloads"]
            line["gate_vs_cublas"] = sweep["gate_vs_cublas"]
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def pipelined_e2e_ms(sess_a, sess_b, x_host, w, bias, flush, steps):
    """Device time of `steps` end-to-end steps (after two untimed ones): upload of x from pinned memory ->
    Session.run -> read-back of every output into pinned memory, with the three phases of consecutive steps
    on three streams and two sets of device and host buffers."""
    import torch
    dev = sess_a.device
    sessions = (sess_a, sess_b)
    x_in = [torch.empty(x_host.shape, dtype=x_host.dtype, device=dev) for _ in range(2)]

    def outputs(sess):
        return [t for t in (sess.permuted, sess.scales, sess.offsets, sess.inverse_perm, sess.combine_weights)
                if t is not None]

    host = [[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outputs(sv)] for sv in sessions]
    up, run, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    uploaded = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    read_back = [torch.cuda.Event() for _ in range(2)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)

    def one(i):
        k = i & 1
        with torch.cuda.stream(up):
            if i >= 2:
                up.wait_event(computed[k])        # the pass two steps ago has read this input buffer
            x_in[k].copy_(x_host, non_blocking=True)
            uploaded[k].record(up)
        with torch.cuda.stream(run):
            run.wait_event(uploaded[k])
            if i >= 2:
                run.wait_event(read_back[k])      # its outputs have been read back
            flush.zero_()
            sessions[k].run(x_in[k], w, bias)
            computed[k].record(run)
        with torch.cuda.stream(down):
            down.wait_event(computed[k])
            for h, d in zip(host[k], outputs(sessions[k])):
                h.copy_(d, non_blocking=True)
            read_back[k].record(down)

    for i in range(2):
        one(i)
    torch.cuda.synchronize(dev)
    t0.record(up)
    for i in range(2, 2 + steps):
        one(i)
    with torch.cuda.stream(down):
        t1.record(down)
    torch.cuda.synchronize(dev)
    for sv in sessions:
        sv.status()
    return t0.elapsed_time(t1)


def graph_replay_ms(sess, x, w, bias, flush, steps):
    import torch
    graph = sess.capture(x, w, bias)
    for _ in range(3):
        graph.replay()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    torch.cuda.synchronize()
    for s_, e_ in ev:
        flush.zero_()
        s_.record()
        graph.replay()
        e_.record()
    torch.cuda.synchronize()
    sess.status()
    return statistics.mean(s_.elapsed_time(e_) for s_, e_ in ev)


def run_sweep(dev, flush, names, peak, steps=10):
    """A few steps of other single-GPU workloads (device-timed, L2 flushed between steps), and for the
    workloads whose gate runs on the tensor cores the gate stage beside cuBLAS on the same operands:
    torch.mm of x [T,H] bf16 with the bf16 operand the gate kernel consumes ([H,E], or [H,2E] hi|lo columns
    for an fp32 weight, the reference's own GEMM shape, kernel.cu:4327-4339), fp32 output."""
    import torch
    from moe_rd import workloads, _cabi
    from moe_rd.runtime import Session
    other, cmp_ = {}, {}
    for name in names + ["c4"]:
        spec = workloads.SPECS[name]
        T, H, E, K = spec["T"], spec["H"], spec["E"], spec["K"]
        tensors, kw = workloads.make(name)
        x, w = tensors["x"].to(dev), tensors["w"].to(dev)
        bias = None if tensors["bias"] is None else tensors["bias"].to(dev)
        sess = Session(T, H, E, K, device=dev, w_dtype=w.dtype, **session_kwargs(kw))
        for _ in range(3):
            flush.zero_()
            sess.run(x, w, bias)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        torch.cuda.synchronize()
        for s_, e_ in ev:
            flush.zero_()
            s_.record()
            sess.run(x, w, bias)
            e_.record()
        torch.cuda.synchronize()
        sess.status()
        ms = statistics.mean(s_.elapsed_time(e_) for s_, e_ in ev)
        stage = []
        for _ in range(5):
            flush.zero_()
            stage.append(sess.run_timed(x, w, bias))
        st = [statistics.mean(v[i] for v in stage) for i in range(5)]
        kept = int(sess.offsets[-1].item())
        fp8 = kw.get("rows_format", "bf16") == "fp8"
        nbytes = workloads.algorithmic_bytes(T, H, E, K, w_bytes=w.element_size(), fp8=fp8, kept_rows=kept)
        gbs = nbytes / (ms * 1e-3) / 1e9
        if name != "c4":  # c4 is the headline workload itself; it is here for the cuBLAS leg only
            other[name] = {"ms_per_step": ms, "value": T / (ms * 1e-3), "unit": UNIT, "kept_rows": kept,
                           "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "frac_of_measured": gbs / peak,
                           "frac_of_8000": gbs / 8000.0,
                           "stage_ms": {"gate": st[0], "route": st[1], "positions": st[3], "scatter": st[4]},
                           "stage_note": "where gate and routing are one kernel its time is under gate",
                           "graph_replay_ms": graph_replay_ms(sess, x, w, bias, flush, steps),
                           "steps": steps}
        if E >= 64:
            # the gate product alone: gate and routing kept in two kernels for this leg
            sep = Session(T, H, E, K, device=dev, w_dtype=w.dtype, flags=_cabi.FLAG_SEPARATE_GATE_AND_ROUTING,
                          **session_kwargs(kw))
            for _ in range(3):
                sep.run(x, w, bias)
            gate_ms = []
            for _ in range(5):
                flush.zero_()
                gate_ms.append(sep.run_timed(x, w, bias)[0])
            gate_us = statistics.mean(gate_ms) * 1e3
            del sep
            if w.dtype == torch.float32:
                wf = w if kw.get("w_layout", "HE") == "HE" else w.t()
                hi = wf.to(torch.bfloat16)
                lo = (wf - hi.to(torch.float32)).to(torch.bfloat16)
                wb = torch.cat([hi, lo], dim=1).contiguous()
            else:
                wb = (w if kw.get("w_layout", "HE") == "HE" else w.t()).contiguous()
            try:
                mm = lambda: torch.mm(x, wb, out_dtype=torch.float32)  # noqa: E731
                mm()
                out_kind = "fp32"
            except (TypeError, RuntimeError):
                mm = lambda: torch.mm(x, wb)  # noqa: E731
                out_kind = "bf16"
            for _ in range(3):
                mm()
            evc = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            torch.cuda.synchronize()
            for s_, e_ in evc:
                flush.zero_()
                s_.record()
                mm()
                e_.record()
            torch.cuda.synchronize()
            cub = statistics.mean(s_.elapsed_time(e_) for s_, e_ in evc) * 1e3
            cmp_[name] = {"shape": f"[{T},{H}]x[{H},{wb.shape[1]}]", "ours_us": gate_us, "cublas_us": cub,
                          "cublas_out": out_kind,
                          "note": "both are CUDA-event pairs around the launch(es) with a cold L2; ours includes the "
                                  "per-call weight split for fp32 weights and writes split-K partials"}
            del wb
        del sess, x, w
        torch.cuda.empty_cache()
    return {"other_workloads": other, "gate_vs_cublas": cmp_}


def run_combine(args):
    """`--op combine`: the weighted combine on the workload's shapes (one GPU), same timing rules."""
    import torch
    import moe_rd
    from moe_rd import workloads
    spec = workloads.SPECS[args.workload]
    T, H, K = spec["T"], spec["H"], spec["K"]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(7)
    R = T * K
    y = torch.randn(R, H, generator=g, dtype=torch.float32).to(torch.bfloat16).to(dev)
    sh = torch.randn(T, H, generator=g, dtype=torch.float32).to(torch.bfloat16).to(dev)
    inv = torch.randperm(R, generator=g).to(torch.int32).view(T, K).to(dev)
    w = torch.rand(T, K, generator=g).to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        moe_rd.combine(y, inv, w, sh)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    for s_, e_ in ev:
        flush.zero_()
        s_.record()
        moe_rd.combine(y, inv, w, sh)
        e_.record()
    torch.cuda.synchronize()
    ms = sum(s_.elapsed_time(e_) for s_, e_ in ev) / args.steps
    nbytes = R * H * 2 + 2 * T * H * 2 + T * K * 8
    peak, kind = measured_hbm_peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "combined_tokens_per_s", "value": T / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": args.workload + " combine", "tokens": T, "hidden": H, "top_k": K,
                   "l2": "flushed by a 256 MiB device write between steps"},
        "roofline": {"bound": "hbm", "kernel": "combine_kernel", "achieved": gbs, "peak": peak, "unit": "GB/s",
                     "frac": gbs / peak, "peak_kind": f"{kind} HBM copy bandwidth", "traffic": None,
                     "bytes_per_launch": nbytes, "kernel_ms": ms},
        "gpu_launches": args.steps}), flush=True)


def run_combine_add(args):
    """`--op combine_add`: the residual (accumulating) combine on the workload's shapes (one GPU) with every
    row live, i.e. its worst case; same timing rules.  Bytes: every row of y once, row metadata, and the rows
    of `out` the reductions land on, once each way (they are resolved in L2 while the K rows of a token
    arrive)."""
    import torch
    import moe_rd
    from moe_rd import workloads
    spec = workloads.SPECS[args.workload]
    T, H, K = spec["T"], spec["H"], spec["K"]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(7)
    R = T * K
    y = torch.randn(R, H, generator=g, dtype=torch.float32).to(torch.bfloat16).to(dev)
    out = torch.randn(T, H, generator=g, dtype=torch.float32).to(torch.bfloat16).to(dev)
    tok = (torch.randperm(R, generator=g) % T).to(torch.int32).to(dev)
    w = torch.rand(R, generator=g).to(dev)
    n = torch.tensor([R], dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        moe_rd.combine_add_rows(y, tok, w, n, out)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    for s_, e_ in ev:
        flush.zero_()
        s_.record()
        moe_rd.combine_add_rows(y, tok, w, n, out)
        e_.record()
    torch.cuda.synchronize()
    ms = sum(s_.elapsed_time(e_) for s_, e_ in ev) / args.steps
    nbytes = R * H * 2 + 2 * T * H * 2 + R * 8
    peak, kind = measured_hbm_peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "combined_tokens_per_s", "value": T / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload + " residual combine, all rows live", "tokens": T, "hidden": H,
                   "top_k": K, "l2": "flushed by a 256 MiB device write between steps"},
        "roofline": {"bound": "hbm", "kernel": "combine_add_rows_kernel", "achieved": gbs, "peak": peak,
                     "unit": "GB/s", "frac": gbs / peak, "peak_kind": f"{kind} HBM copy bandwidth", "traffic": None,
                     "bytes_per_launch": nbytes, "kernel_ms": ms},
        "gpu_launches": args.steps}), flush=True)


def run_ep_kernels(args):
    """`--op ep_kernels --ranks W`: the expert-parallel kernels of ONE rank at full size with every rank's
    buffers on this GPU (the kernels take plain device pointers and none waits on another, so W ranks can be
    played in one process).  What crosses NVLink in a real run is HBM traffic here, so the figures bound the
    kernels' own cost; it is also the one way to look at them with a profiler, which cannot attach to a
    multi-rank run.  Times rank 0's peer-store scatter (every pair, and send-once) and the owner-side copy
    kernel with event pairs after an L2 flush."""
    import ctypes
    import torch
    from moe_rd import workloads, _cabi
    from moe_rd.runtime import Session
    world = args.ranks
    spec = workloads.SPECS["c5"]
    T, H, E, K = spec["T"], spec["H"], spec["E"], spec["K"]
    dev = torch.device("cuda", 0)
    L = _cabi.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())            # noqa: E731
    ptrs = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])      # noqa: E731
    epr = E // world
    sessions, xs = [], []
    for r in range(world):
        t, kw = workloads.make("c5", rank=r)
        s = Session(T, H, E, K, device=dev, w_dtype=t["w"].dtype, scatter_impl="none", **session_kwargs(kw))
        x = t["x"].to(dev)
        s.run(x, t["w"].to(dev), t["bias"].to(dev))
        sessions.append(s)
        xs.append(x)
    max_rows = 2 * T * K
    pitch = H + H // 32
    rows = [torch.zeros(max_rows * pitch, dtype=torch.uint8, device=dev) for _ in range(world)]
    copy_of = [torch.full((max_rows,), -1, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    plans = [dict(dest_base=torch.empty(E, dtype=torch.int32, device=dev),
                  cnt=torch.empty((world, epr), dtype=torch.int32, device=dev),
                  local_offsets=torch.empty(epr + 1, dtype=torch.int32, device=dev)) for _ in range(world)]
    kept_all = torch.stack([(s.offsets[1:] - s.offsets[:-1]) for s in sessions]).contiguous()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    times = {"scatter_every_pair": [], "scatter_send_once": [], "owner_copies": []}
    steps = max(args.steps, 3)
    for _ in range(steps + 1):
        for r in range(world):
            p = plans[r]
            _cabi.check(L.moe_rd_ep_plan(ptr(kept_all), world, r, E, max_rows, ptr(p["dest_base"]), ptr(p["cnt"]),
                                         ptr(p["local_offsets"]), ptr(status), stream))
        for key in ("scatter_every_pair", "scatter_send_once"):
            for r in range(world):
                s = sessions[r]
                params = _cabi.Params.from_buffer_copy(s.params)
                params.scatter_impl = _cabi.SCATTER_IMPL["bulk"]
                a = (ctypes.byref(params), ptr(xs[r]), ptr(s.expert_ids), ptr(s.inverse_perm), ptr(s.offsets),
                     ptr(plans[r]["dest_base"]), world)
                if r == 0:
                    flush.zero_()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                if key == "scatter_send_once":
                    _cabi.check(L.moe_rd_ep_scatter_once(*a, r, ptrs(rows), None, ptrs(copy_of), ptr(status), stream))
                else:
                    _cabi.check(L.moe_rd_ep_scatter(*a, ptrs(rows), None, ptr(status), stream))
                if r == 0:
                    e1.record()
                    torch.cuda.synchronize()
                    times[key].append(e0.elapsed_time(e1))
        for r in range(world):
            params = _cabi.Params.from_buffer_copy(sessions[r].params)
            n_rows = ctypes.c_void_p(plans[r]["local_offsets"].data_ptr() + 4 * epr)
            if r == 0:
                marks = int((copy_of[0] >= 0).sum())
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            _cabi.check(L.moe_rd_ep_replicate(ctypes.byref(params), ptr(rows[r]), None, ptr(copy_of[r]), n_rows,
                                              max_rows, ptr(status), stream))
            if r == 0:
                e1.record()
                torch.cuda.synchronize()
                times["owner_copies"].append(e0.elapsed_time(e1))
    assert int(status[0]) == 0, status.tolist()
    ms = {k: statistics.median(v[1:]) for k, v in times.items()}
    received = int(plans[0]["local_offsets"][-1])
    copy_bytes = 2 * marks * pitch
    peak, kind = measured_hbm_peak()
    print(json.dumps({
        "metric": "ep_kernel_ms", "value": ms["scatter_send_once"] + ms["owner_copies"], "unit": "ms", "n_gpus": 1,
        "steps": steps, "warmup": 1, "ms_per_step": ms["scatter_send_once"] + ms["owner_copies"],
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": f"c5, expert-parallel kernels of rank 0 of {world}, all buffers on one GPU",
                   "tokens_per_rank": T, "hidden": H, "experts": E, "top_k": K,
                   "l2": "flushed by a 256 MiB device write before each timed kernel"},
        "kernel_ms": ms, "rows_received_by_rank0": received, "rows_copied_by_rank0": marks,
        "roofline": {"bound": "hbm", "kernel": "ep_replicate_kernel", "achieved": copy_bytes / (ms["owner_copies"] * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s", "frac": copy_bytes / (ms["owner_copies"] * 1e-3) / 1e9 / peak,
                     "peak_kind": f"{kind} HBM copy bandwidth", "traffic": None, "bytes_per_launch": copy_bytes,
                     "kernel_ms": ms["owner_copies"]},
        "gpu_launches": (steps + 1) * 4 * world}), flush=True)


def run_combine_ep(args, rank, world, local_rank):
    """`--op combine` at N > 1: the expert-parallel combine (every rank pulls its pairs' expert outputs from
    the owning ranks over NVLink inside the combine kernel).  Routing and the dispatch run once, untimed, to
    fix the mapping; a step is one collective `combine` (barrier, kernel, barrier)."""
    import torch
    import torch.distributed as dist
    from moe_rd import workloads
    from moe_rd.runtime import Session
    from moe_rd.ep import ExpertParallelFused
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    name = "c5"
    spec = workloads.SPECS[name]
    T, H, E, K = spec["T"], spec["H"], spec["E"], spec["K"]
    t, kw = workloads.make(name, rank=rank)
    keys = ("score_fn", "bias_mode", "n_groups", "topk_groups", "group_topk", "renorm", "routed_scale", "capacity",
            "rows_format")
    sess = Session(T, H, E, K, device=dev, w_dtype=t["w"].dtype, scatter_impl="none",
                   **{k: v for k, v in kw.items() if k in keys})
    ep = ExpertParallelFused(sess)
    x, w, b = t["x"].to(dev), t["w"].to(dev), t["bias"].to(dev)
    sess.run(x, w, b)
    out = ep.exchange(x)
    y = ep.expert_output_buffer()
    n = int(out.offsets[-1].item())
    y[:n].normal_()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        ep.combine()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    dist.barrier()
    for s_, e_ in ev:
        flush.zero_()
        s_.record()
        ep.combine()
        e_.record()
    torch.cuda.synchronize()
    ms = sum(s_.elapsed_time(e_) for s_, e_ in ev) / args.steps
    offs = sess.offsets.cpu()
    epr = E // world
    remote_rows = int(offs[E]) - int(offs[(rank + 1) * epr] - offs[rank * epr])
    red = torch.tensor([ms, float(remote_rows) * H * 2], dtype=torch.float64, device=dev)
    dist.all_reduce(red, op=dist.ReduceOp.MAX)
    ms, ingress = float(red[0]), float(red[1])
    if rank == 0:
        link = 770.0
        gbs = ingress / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "combined_tokens_per_s", "value": world * T / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": "c5 combine, expert parallel", "tokens_per_rank": T, "hidden": H, "top_k": K,
                       "experts": E, "l2": "flushed by a 256 MiB device write between steps"},
            "roofline": {"bound": "nvlink", "kernel": "combine_kernel<EP> (16-byte peer loads)", "achieved": gbs,
                         "peak": link, "unit": "GB/s", "frac": gbs / link,
                         "peak_kind": "measured peer copy per direction (900 nominal)", "traffic": None,
                         "bytes_per_launch": ingress, "kernel_ms": ms},
            "gpu_launches": args.steps}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    # NCCL prints its version banner on stdout at this level; stdout carries the one JSON line
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c1", "c2", "c3", "c4", "c5", "ref"])
    ap.add_argument("--no-sweep", action="store_true",
                    help="skip the other_workloads / gate_vs_cublas legs of the N = 1 line")
    ap.add_argument("--scatter", default="auto", choices=["auto", "simt", "bulk"])
    ap.add_argument("--op", default="route_dispatch", choices=["route_dispatch", "combine", "combine_add", "ep_kernels"])
    ap.add_argument("--ranks", type=int, default=2, choices=[2, 4, 8], help="--op ep_kernels: ranks played on one GPU")
    ap.add_argument("--ep-layout", default=None, choices=["packed", "separate"],
                    help="fused exchange, fp8 rows: scales after each row (one copy per pair) or in a buffer of their own")
    ap.add_argument("--ep-every-pair", action="store_true",
                    help="fused exchange: every pair carries its row over NVLink (no send-once / owner-side copies)")
    ap.add_argument("--ep", default="fused", choices=["fused", "nccl"],
                    help="expert-parallel exchange at N > 1: one peer-store kernel, or NCCL all-to-all + reorder")
    args = ap.parse_args()
    rank, world, local_rank = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch with torchrun for --gpus > 1 (one process per GPU)")
    if args.op == "ep_kernels":
        if rank == 0:
            run_ep_kernels(args)
        return
    if args.op == "combine_add":
        if rank == 0:
            run_combine_add(args)
        return
    if args.op == "combine":
        if world > 1:
            run_combine_ep(args, rank, world, local_rank)
        elif rank == 0:
            run_combine(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()

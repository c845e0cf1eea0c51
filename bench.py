#!/usr/bin/env python
"""Benchmark of the alias-method walk path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5|c2|c1|dw26] [--impl ours|reference]

One "step" is one pass of the walk kernel over the whole batch of walkers of the workload.
Default workload: BASELINE config 5 -- biased offline PPR (tp 0.15, max length 100) on a seeded
R-MAT scale-26 graph (~1.8 G directed edges), 8 M walkers sharded evenly over the N GPUs, graph
and tables replicated per GPU.  Rank 0 prints ONE JSON line.

--impl reference times the CPU implementation of the same path (the OpenMP oracle; the
reference project itself is CUDA-only) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: scale, raw edge factor, walkers, walk length, app, tp
    "c1": dict(scale=16, edge_factor=16, walkers=4096, length=80, app="deepwalk", tp=0.0,
               desc="BASELINE config 1: biased offline DeepWalk, R-MAT scale 16, 4,096 walkers x 80"),
    "c2": dict(scale=22, edge_factor=16, walkers=40000, length=80, app="deepwalk", tp=0.0,
               desc="BASELINE config 2: biased offline DeepWalk, R-MAT scale 22, 40,000 walkers x 80"),
    "c5": dict(scale=26, edge_factor=28, walkers=8000000, length=100, app="ppr", tp=0.15,
               desc="BASELINE config 5: biased offline PPR tp=0.15 max length 100, R-MAT scale 26 "
                    "(~1.8G directed edges), 8M walkers sharded over the GPUs"),
    "dw26": dict(scale=26, edge_factor=28, walkers=8000000, length=80, app="deepwalk", tp=0.0,
                 desc="biased offline DeepWalk, R-MAT scale 26 (~1.8G directed edges), 8M walkers x 80"),
    "c5s": dict(scale=22, edge_factor=28, walkers=1000000, length=100, app="ppr", tp=0.15,
                desc="reduced config 5 for profiling: PPR on R-MAT scale 22, 1M walkers"),
}
GRAPH_SEED, WEIGHT_SEED, START_SEED, WALK_SEED = 1, 7, 42, 42
ALG_BYTES_PER_EDGE = 24   # 8 offsets + 8 slot + 4 neighbour + 4 path store
ALG_BYTES_PER_BUILD_EDGE = 12  # 4 weight + 8 slot


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def shard(n_total, world, rank):
    lo = n_total * rank // world
    hi = n_total * (rank + 1) // world
    return lo, hi - lo


def combine_over_ranks(dist, values, device=None):
    """(max over ranks, sum over ranks) of a list of floats; identity without a process group."""
    import torch
    t = torch.tensor(values, dtype=torch.float64, device=device)
    if dist is None:
        return t.tolist(), t.tolist()
    mx, sm = t.clone(), t.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    return mx.tolist(), sm.tolist()


def make_graph(ctx, wl):
    raw = wl["edge_factor"] << wl["scale"]
    ctx.generate_rmat(wl["scale"], raw, 0.57, 0.19, 0.19, False, GRAPH_SEED, WEIGHT_SEED)
    return ctx.graph_info()


def cpu_leg(ctx, wl, app_id, threads, want_seconds=12.0):
    """Time the CPU oracle on a bounded sample of the workload: alias build over a vertex range and
    walks over a walker range, same inputs (downloaded from the GPU), same Philox streams."""
    from oracle import oracle as O
    V, E, _ = ctx.graph_info()
    xadj, adjncy, wgt = ctx.download()
    threads = threads or O.num_threads()
    # alias build: a vertex prefix holding ~1/16 of the edges (bounded)
    target = min(E, max(1 << 20, E // 16))
    v_end = int(np.searchsorted(xadj, target, side="left"))
    v_end = max(1, min(V, v_end))
    t0 = time.perf_counter()
    O.alias_build(xadj, wgt, 0, v_end, threads)
    t_build = time.perf_counter() - t0
    build_eps = float(xadj[v_end]) / t_build
    del wgt
    prob, alias, valid = ctx.alias_export()
    # walks: calibrate on a small range, then size the sample for ~want_seconds
    hop = wl["length"] + 1
    n_total = wl["walkers"]
    probe = min(n_total, 100000)
    starts = O.gen_starts(n_total if n_total <= 2000000 else 2000000, V, START_SEED)
    t0 = time.perf_counter()
    _, l0 = O.walk(xadj, adjncy, np.zeros(1, np.float32), (prob, alias, valid), starts[:probe], hop, app=app_id,
                   tp=wl["tp"], seed=WALK_SEED, threads=threads)
    t_probe = time.perf_counter() - t0
    n_s = int(min(len(starts), max(probe, probe * want_seconds / max(t_probe, 1e-6))))
    t0 = time.perf_counter()
    _, l1 = O.walk(xadj, adjncy, np.zeros(1, np.float32), (prob, alias, valid), starts[:n_s], hop, app=app_id,
                   tp=wl["tp"], seed=WALK_SEED, threads=threads)
    t_walk = time.perf_counter() - t0
    eps = float(l1.sum()) / t_walk
    return {"value": eps, "unit": "sampled edges/s", "cores": threads, "kind": "port",
            "sample": "first %d of %d walkers (%.2f s); alias build of the first %d vertices / %d edges: %.3g edges/s"
                      % (n_s, n_total, t_walk, v_end, int(xadj[v_end]), build_eps),
            "alias_build_edges_per_s": build_eps, "seconds": t_walk, "edges": int(l1.sum())}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-records", action="store_true", help="walk over the 8-byte slot table only")
    ap.add_argument("--cpu-threads", type=int, default=0)
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from skywalker_b200 import APP_DEEPWALK, APP_PPR
    app_id = APP_PPR if wl["app"] == "ppr" else APP_DEEPWALK
    hop = wl["length"] + 1
    config = {"workload": args.workload + ": " + wl["desc"], "graph": "R-MAT a/b/c/d=0.57/0.19/0.19/0.05",
              "scale": wl["scale"], "raw_edge_factor": wl["edge_factor"], "walkers_total": wl["walkers"],
              "hop_num": hop, "tp": wl["tp"], "seeds": {"graph": GRAPH_SEED, "weight": WEIGHT_SEED,
                                                        "start": START_SEED, "walk": WALK_SEED},
              "cache": "inputs larger than L2 (table and CSR are GBs; no flush needed)",
              "parallelism": "walkers sharded, graph+tables replicated"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        if not torch.cuda.is_available():
            print(json.dumps({"impl": "reference", "unavailable": "no GPU to generate the workload's inputs on"}))
            return 0
        from skywalker_b200.api import Context
        torch.cuda.set_device(local_rank)
        ctx = Context(local_rank)
        V, E, md = make_graph(ctx, wl)
        ctx.alias_build_offline()
        vals = []
        for _ in range(max(1, min(args.steps, 3))):
            leg = cpu_leg(ctx, wl, app_id, args.cpu_threads, want_seconds=10.0)
            vals.append(leg)
        best = max(vals, key=lambda d: d["value"])
        ms = best["seconds"] * 1e3
        out = {"impl": "reference", "metric": "sampled edges/s", "value": best["value"], "unit": "sampled edges/s",
               "n_gpus": args.gpus, "steps": len(vals), "warmup": 0, "ms_per_step": ms, "higher_is_better": True,
               "scaling": "strong", "vs_baseline": None, "dtype": "u32 ids / f32 prob", "data": "synthetic",
               "config": dict(config, V=V, E=E, inputs="generated on the GPU by the library's seeded R-MAT generator, "
                              "then copied to the host; only the CPU walk is timed"),
               "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
               "e2e": {"value": best["value"], "unit": "sampled edges/s", "h2d_bytes_per_step": 0,
                       "d2h_bytes_per_step": 0}}
        print(json.dumps(out))
        return 0

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: skywalker_b200 has no CPU path"}))
        return 1
    from skywalker_b200.api import Context
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    ctx = Context(local_rank)
    stream = torch.cuda.current_stream()
    ctx.set_stream(stream.cuda_stream)

    t0 = time.perf_counter()
    V, E, max_deg = make_graph(ctx, wl)
    t_gen = time.perf_counter() - t0
    build_ms = [ctx.alias_build_offline() for _ in range(3)]
    build_best = min(build_ms)
    peak, peak_kind = measured_peak()

    n_total = wl["walkers"]
    lo, n_local = shard(n_total, world, rank)
    starts = torch.empty(max(n_local, 1), dtype=torch.int32, device=dev)
    paths = torch.empty(max(n_local, 1) * hop, dtype=torch.int32, device=dev)
    lengths = torch.empty(max(n_local, 1), dtype=torch.int32, device=dev)
    ctx.generate_starts(n_local, START_SEED, starts, id_base=lo)
    torch.cuda.synchronize()

    def step(i):
        return ctx.walk(starts, hop, app=app_id, tp=wl["tp"], seed=WALK_SEED + i, walker_base=lo, paths=paths,
                        lengths=lengths, n=n_local)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # the same walks over the plain 8-byte slot table first (3 accesses per step), for comparison
    slots_ms, slots_edges = [], 0
    for i in range(args.warmup + 2):
        _, _, ms, edges = step(100 + i)
        if i >= args.warmup:
            slots_ms.append(ms)
            slots_edges += edges
    records_build_ms = None
    if not args.no_records:
        records_build_ms = ctx.walk_records_build()
    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = ctx.kernel_launches
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kernel_ms, edges_local = 0.0, 0
    ev0.record(stream)
    for i in range(args.steps):
        _, _, ms, edges = step(100 + i)
        kernel_ms += ms
        edges_local += edges
    ev1.record(stream)
    barrier()
    clocks = sampler.stop()
    launches = ctx.kernel_launches - launches0
    span_ms = ev0.elapsed_time(ev1)

    mx, sm = combine_over_ranks(dist, [span_ms, kernel_ms, float(edges_local), float(launches)], dev)
    span_ms, kernel_ms = mx[0], mx[1]
    edges_all, launches = sm[2], int(sm[3])
    value = edges_all / (span_ms * 1e-3)

    # end to end through the host-buffer entry point: pinned starts in, paths + lengths out
    e2e = None
    if not args.no_e2e:
        h_starts = torch.empty(max(n_local, 1), dtype=torch.int32).pin_memory()
        h_paths = torch.empty(max(n_local, 1) * hop, dtype=torch.int32).pin_memory()
        h_len = torch.empty(max(n_local, 1), dtype=torch.int32).pin_memory()
        h_starts.copy_(starts.cpu())
        np_starts = h_starts.numpy().view(np.uint32)
        np_paths = h_paths.numpy().view(np.uint32)
        np_len = h_len.numpy().view(np.uint32)

        def estep(i):
            return ctx.walk(np_starts, hop, app=app_id, tp=wl["tp"], seed=WALK_SEED + i, walker_base=lo,
                            paths=np_paths, lengths=np_len, n=n_local)
        estep(0)
        barrier()
        e_steps = max(1, min(args.steps, 5))
        t0 = time.perf_counter()
        e_edges = 0
        for i in range(e_steps):
            e_edges += estep(100 + i)[3]
        barrier()
        e_ms = (time.perf_counter() - t0) * 1e3
        m2, s2 = combine_over_ranks(dist, [e_ms, float(e_edges)], dev)
        e_ms, e_edges = m2[0], s2[1]
        e2e = {"value": e_edges / (e_ms * 1e-3), "unit": "sampled edges/s", "steps": e_steps,
               "ms_per_step": e_ms / e_steps, "h2d_bytes_per_step": 4 * n_local,
               "d2h_bytes_per_step": 4 * n_local * hop + 4 * n_local,
               "note": "skw_walk with pinned host buffers: starts H2D, kernel, full path matrix + lengths D2H"}

    # NCCL gather of the per-walker lengths to rank 0 (results gather; outside the timed region)
    gather_ms = None
    if dist is not None:
        bufs = [torch.empty_like(lengths) for _ in range(world)] if rank == 0 else None
        dist.gather(lengths, bufs, dst=0)       # first collective sets NCCL up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        dist.gather(lengths, bufs, dst=0)
        torch.cuda.synchronize()
        gather_ms = (time.perf_counter() - t0) * 1e3

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_leg(ctx, wl, app_id, args.cpu_threads)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample", "alias_build_edges_per_s")}

    if rank == 0:
        per_launch_ms = kernel_ms / args.steps
        edges_per_launch = edges_all / args.steps / world
        achieved = edges_per_launch * ALG_BYTES_PER_EDGE / (per_launch_ms * 1e-3) / 1e9
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath):
            try:
                tj = json.load(open(tpath)).get(args.workload)
                if tj:
                    traffic = tj["dram_bytes_per_sampled_edge"] * edges_per_launch
            except Exception:
                traffic = None
        out = {
            "metric": "sampled edges/s", "value": value, "unit": "sampled edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": span_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u32 ids / f32 prob", "data": "synthetic",
            "config": dict(config, V=V, E=E, max_degree=max_deg, walkers_per_gpu=n_local, graph_gen_s=t_gen),
            "kernel_ms_per_step": per_launch_ms,
            "sampled_edges_per_step": edges_all / args.steps,
            "alias_build": {"value": E / (build_best * 1e-3), "unit": "edges/s", "ms": build_best,
                            "roofline": {"bound": "hbm", "achieved": E * ALG_BYTES_PER_BUILD_EDGE / (build_best * 1e-3) / 1e9,
                                         "peak": peak, "unit": "GB/s",
                                         "frac": E * ALG_BYTES_PER_BUILD_EDGE / (build_best * 1e-3) / 1e9 / peak,
                                         "peak_kind": peak_kind}},
            "layout": "8-byte slots" if args.no_records else "fused 32-byte walk records",
            "walk_records_build_ms": records_build_ms,
            "slots_layout": {"kernel_ms_per_step": float(np.mean(slots_ms)),
                             "value": slots_edges / (sum(slots_ms) * 1e-3) if slots_ms else None,
                             "unit": "sampled edges/s (this rank, kernel time)"},
            "roofline": {"bound": "hbm", "kernel": "walk_offline_kernel" if args.no_records else "walk_records_walk_kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_sampled_edge": ALG_BYTES_PER_EDGE},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "result_gather_ms": gather_ms,
        }
        print(json.dumps(out))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    ctx.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())

#!/usr/bin/env python
"""Benchmark of the alias-method sampling / random-walk path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5|c2|c1|c3|c4|c4off|dw26|dw22|c5s]
                    [--impl ours|reference]

One "step" is one pass of the hot path over one batch: all walkers of the workload (walks) or one
batch of seed vertices (k-hop).  Default workload: benchmark configuration 5 -- biased offline PPR
(tp 0.15, max length 100) on a seeded R-MAT scale-26 graph (~1.8 G directed edges), 8 M walkers
sharded evenly over the N GPUs, graph and tables replicated per GPU.  Rank 0 prints ONE JSON line.

--impl reference times the CPU implementation of the same path (the OpenMP oracle; the reference
project itself is CUDA-only) on a bounded sample of the same workload.
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
    "c1": dict(graph="rmat", scale=16, edge_factor=16, kind="walk", mode="offline", units=4096, length=80,
               app="deepwalk", tp=0.0,
               desc="benchmark configuration 1: biased offline DeepWalk, R-MAT scale 16, 4,096 walkers x 80"),
    "c2": dict(graph="rmat", scale=22, edge_factor=16, kind="walk", mode="offline", units=40000, length=80,
               app="deepwalk", tp=0.0,
               desc="benchmark configuration 2: biased offline DeepWalk, R-MAT scale 22, 40,000 walkers x 80"),
    "c3": dict(graph="plaw", V=3070000, raw_edges=117000000, exponent=2.1, dmin=12.0, cap=33000, kind="walk",
               mode="online", units=40000, length=80, app="node2vec", tp=0.0, p=2.0, q=0.5,
               desc="benchmark configuration 3: online biased node2vec p=2 q=0.5 (rejection), undirected power-law graph "
                    "3.07M vertices / 117M undirected edges, degree ~ Zipf 2.1 capped at 33k, 40,000 walkers x 80"),
    "c4": dict(graph="rmat", scale=23, V=4850000, raw_edges=72000000, kind="khop", mode="online", units=65536,
               fanout=[25, 10],
               desc="benchmark configuration 4: online biased 2-hop sampling, fan-out 25 then 10 with replacement, "
                    "R-MAT-like directed graph 4.85M vertices / ~69M edges, batches of 65,536 random seeds"),
    "c4off": dict(graph="rmat", scale=23, V=4850000, raw_edges=72000000, kind="khop", mode="offline", units=65536,
                  fanout=[25, 10], khop_flags=1,
                  desc="offline biased 2-hop sampling by the rule of the reference's offline sampler (fan-out 25 then "
                       "10 with replacement, every neighbour once where a vertex has no more than the fan-out), graph "
                       "and seeds of benchmark configuration 4; the reference's own kernel runs beside it"),
    "c5": dict(graph="rmat", scale=26, edge_factor=28, kind="walk", mode="offline", units=8000000, length=100,
               app="ppr", tp=0.15,
               desc="benchmark configuration 5: biased offline PPR tp=0.15 max length 100, R-MAT scale 26 "
                    "(~1.8G directed edges), 8M walkers sharded over the GPUs"),
    "dw26": dict(graph="rmat", scale=26, edge_factor=28, kind="walk", mode="offline", units=8000000, length=80,
                 app="deepwalk", tp=0.0,
                 desc="biased offline DeepWalk, R-MAT scale 26 (~1.8G directed edges), 8M walkers x 80"),
    "dw22": dict(graph="rmat", scale=22, edge_factor=16, kind="walk", mode="offline", units=1000000, length=80,
                 app="deepwalk", tp=0.0,
                 desc="biased offline DeepWalk on the graph of configuration 2 (R-MAT scale 22), 1M walkers x 80: the "
                      "reduced DeepWalk case for profiling and for the reference's own kernel"),
    "c5s": dict(graph="rmat", scale=22, edge_factor=28, kind="walk", mode="offline", units=1000000, length=100,
                app="ppr", tp=0.15, desc="reduced config 5 for profiling: PPR on R-MAT scale 22, 1M walkers"),
}
GRAPH_SEED, WEIGHT_SEED, START_SEED, WALK_SEED = 1, 7, 42, 42
ALG_BYTES_PER_EDGE = 24        # offline step: 8 offsets + 8 slot + 4 neighbour + 4 path store
ALG_BYTES_PER_BUILD_EDGE = 12  # offline build: 4 weight + 8 slot
# DRAM bytes per sampled edge, (dram__bytes_read.sum + dram__bytes_write.sum) / sampled edges of one
# launch, from an ncu capture of the reduced PPR workload "c5s" (same kernels, scale 22, 1 M walkers).
# Traffic grows in proportion to walkers and steps, so roofline.traffic = this figure x the sampled
# edges of a full launch.  The figures belong to the kernels as they were when captured: a change to a
# step kernel needs a new capture.
DRAM_BYTES_PER_SAMPLED_EDGE = {"walk_records_ppr_kernel": 101.5, "walk_records_walk_kernel": 105.2,
                               "walk_offline_kernel": 162.9}


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
    if wl["graph"] == "plaw":
        ctx.generate_powerlaw(wl["V"], wl["raw_edges"], wl["exponent"], wl["dmin"], wl["cap"], GRAPH_SEED, WEIGHT_SEED)
    else:
        raw = wl.get("raw_edges") or (wl["edge_factor"] << wl["scale"])
        ctx.generate_rmat(wl["scale"], raw, 0.57, 0.19, 0.19, False, GRAPH_SEED, WEIGHT_SEED,
                          num_vertices=wl.get("V", 0))
    return ctx.graph_info()


def app_id(wl):
    from skywalker_b200 import APP_DEEPWALK, APP_NODE2VEC, APP_PPR
    return {"deepwalk": APP_DEEPWALK, "ppr": APP_PPR, "node2vec": APP_NODE2VEC}[wl.get("app", "deepwalk")]


def host_memory_available():
    """Bytes this process may still allocate on the host: the smaller of MemAvailable and what the
    cgroup limit leaves (a rank that outgrows it takes the whole box down)."""
    avail = None
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemAvailable:"):
                avail = int(line.split()[1]) * 1024
    except Exception:
        pass
    for lim_path, cur_path in (("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory.current"),
                               ("/sys/fs/cgroup/memory/memory.limit_in_bytes",
                                "/sys/fs/cgroup/memory/memory.usage_in_bytes")):
        try:
            lim = open(lim_path).read().strip()
            cur = int(open(cur_path).read().strip())
            if lim != "max" and int(lim) < (1 << 60):
                left = int(lim) - cur
                avail = left if avail is None else min(avail, left)
        except Exception:
            pass
    return avail


def host_copy_bytes(V, E, online):
    """Host bytes of the CPU checker's inputs: offsets, neighbours, and weights (online) or the
    exported table (offline), plus staging."""
    return 4 * (V + 1) + 4 * E + (4 * E if online else 8 * E + V) + (1 << 30)


def host_copy(ctx, online, with_weights=False):
    """The resident graph (and, for offline modes, the GPU-built table) copied to the host."""
    xadj, adjncy, wgt = ctx.download(weights=online or with_weights)
    table = None if online else ctx.alias_export()
    return {"xadj": xadj, "adjncy": adjncy, "wgt": wgt if online else np.zeros(1, np.float32), "table": table,
            "build_weights": wgt if (with_weights and not online) else None}


def cpu_leg(host, wl, threads, want_seconds=12.0, steps=1, warmup=0, build_weights=None):
    """Time the CPU oracle on a bounded sample of the workload, same inputs (downloaded from the GPU)
    and same Philox streams: alias build over a vertex prefix, then the workload's own step."""
    from oracle import oracle as O
    xadj, adjncy, wgt, table = host["xadj"], host["adjncy"], host["wgt"], host["table"]
    V, E = len(xadj) - 1, int(xadj[-1])
    # all host cores this process may use (torchrun exports OMP_NUM_THREADS=1, which must not shrink the
    # CPU arm to one thread)
    threads = threads or len(os.sched_getaffinity(0)) or O.num_threads()
    online = wl["mode"] == "online"
    target = min(E, max(1 << 20, E // 16))
    v_end = max(1, min(V, int(np.searchsorted(xadj, target, side="left"))))
    bw = wgt if online else build_weights
    build_eps = None
    if bw is not None:
        t0 = time.perf_counter()
        O.alias_build(xadj, bw, 0, v_end, threads)
        build_eps = float(xadj[v_end]) / (time.perf_counter() - t0)
    n_total = wl["units"]
    cap = min(n_total, 2000000)
    starts = O.gen_starts(cap, V, START_SEED)

    def run(n):
        if wl["kind"] == "khop":
            _, sl = O.khop(xadj, adjncy, wgt, table, starts[:n], wl["fanout"], online=online,
                           flags=wl.get("khop_flags", 0), seed=WALK_SEED,
                           threads=threads)
            return int(sl.sum())
        _, l = O.walk(xadj, adjncy, wgt, table, starts[:n], wl["length"] + 1, app=app_id(wl), online=online,
                      tp=wl.get("tp", 0.0), p=wl.get("p", 2.0), q=wl.get("q", 0.5), seed=WALK_SEED, threads=threads)
        return int(l.sum())

    probe = max(1, min(cap, 100000 if not online else 256))
    t0 = time.perf_counter()
    run(probe)
    t_probe = time.perf_counter() - t0
    n_s = int(min(cap, max(probe, probe * want_seconds / max(t_probe, 1e-6))))
    for _ in range(warmup):
        run(n_s)
    edges, t_run = 0, 0.0
    for _ in range(max(1, steps)):      # every step is one pass over the same bounded sample
        t0 = time.perf_counter()
        edges += run(n_s)
        t_run += time.perf_counter() - t0
    edges //= max(1, steps)
    t_run /= max(1, steps)
    sample = "first %d of %d %s (%.2f s)" % (n_s, n_total, "seeds" if wl["kind"] == "khop" else "walkers", t_run)
    if build_eps is not None:
        sample += "; alias build of the first %d vertices / %d edges: %.3g edges/s" % (v_end, int(xadj[v_end]), build_eps)
    return {"value": edges / t_run, "unit": "sampled edges/s", "cores": threads, "kind": "port", "sample": sample,
            "alias_build_edges_per_s": build_eps, "seconds": t_run, "edges": edges}


def reference_cuda_leg(host, wl, hop, device, ctx=None, d_buffers=None, records=False):
    """The reference's OWN offline walk kernel (sample_kernel_static through OfflineWalk) on this
    workload's graph, start vertices and GPU-built table: throughput by the reference's own timer.  For
    offline DeepWalk (graph and table are handed over through host arrays; its walks come from another
    random stream, so only the rate is comparable); PPR and offline 2-hop workloads run the reference's
    unbiased walk and offline sampler instead."""
    from oracle import oracle as O
    from oracle import reference_kernel as R
    if not R.available():
        return {"unavailable": "oracle/_ref/libskw_ref.so was not built (no reference tree on the build machine)"}
    V, E = len(host["xadj"]) - 1, int(host["xadj"][-1])
    if (wl["kind"] == "khop" and wl["mode"] == "offline" and len(wl["fanout"]) == 2 and wl.get("khop_flags", 0) == 1
            and E <= (1 << 28)):
        # the reference's own offline 2-hop sampler (sample_kernel through OfflineSample) on the same seeds
        n, (f1, f2) = wl["units"], wl["fanout"]
        seeds = O.gen_starts(n, V, START_SEED)
        data, sl, sec, edges = R.offline_sample(host["xadj"], host["adjncy"], host["table"], seeds, f1, f2,
                                                device=device, repeats=3)
        deg = np.diff(host["xadj"].astype(np.int64))
        have = np.arange(f1)[None, :] < sl[:, :1]
        parents = data[:, 1:1 + f1][have].astype(np.int64)
        due = deg[parents] > 0
        dropped = int((due & (sl[:, 1:][have] == 0)).sum())
        return {"kernel": "sample_kernel via OfflineSample (src/offline_sample.cu:72-141, 443-513)",
                "value": edges / sec, "unit": "sampled edges/s", "seconds": sec, "sampled_edges": int(edges),
                "seeds": n, "hop2_jobs_dropped": dropped, "hop2_jobs_due": int(due.sum()),
                "note": "best of 3 runs, the reference's own wall-clock timer around its launch and its own count of "
                        "sampled edges; table built by this library.  The reference's kernel publishes a slot of its "
                        "hop-2 job queue before writing it and drops jobs it reads too early (hop2_jobs_dropped of "
                        "hop2_jobs_due), so it samples somewhat fewer edges than the rule asks for"}
    if wl["kind"] == "walk" and wl["mode"] == "offline" and wl.get("app") == "ppr" and ctx is not None:
        # The reference's offline biased kernel has no stop rule, its unbiased walk has: the same graph, start
        # vertices and termination probability through UnbiasedWalkKernelStatic (uniform neighbour, no table),
        # and this library's walk of the same kind (SKW_WALK_UNBIASED) beside it, like for like.
        from skywalker_b200 import APP_PPR, WALK_UNBIASED
        n = wl["units"]
        starts = O.gen_starts(n, V, START_SEED)
        _, lens, sec = R.unbiased_walk(host["xadj"], host["adjncy"], starts, hop, tp=wl["tp"], device=device,
                                       repeats=3, want_paths=False)
        edges = int(lens.sum())
        d_starts, d_result, d_lengths = d_buffers
        ctx.generate_starts(n, START_SEED, d_starts)
        best, our_edges = None, 0
        for r in range(3):
            _, _, ms, our_edges = ctx.walk(d_starts, hop, app=APP_PPR, tp=wl["tp"], flags=WALK_UNBIASED,
                                           seed=WALK_SEED + r, paths=d_result, lengths=d_lengths, n=n)
            best = ms if best is None else min(best, ms)
        return {"kernel": "UnbiasedWalkKernelStatic via UnbiasedWalk (src/unbiased_walk.cu:104-130, 194-278)",
                "value": edges / sec, "unit": "sampled edges/s", "seconds": sec, "sampled_edges": edges, "walkers": n,
                "ours_same_kind": {"kernel": "SKW_WALK_UNBIASED over the walk records (walk_records_ppr_kernel)"
                                             if records else "SKW_WALK_UNBIASED (walk_offline_kernel)",
                                   "value": our_edges / (best * 1e-3),
                                   "unit": "sampled edges/s", "ms": best, "sampled_edges": int(our_edges)},
                "note": "UNBIASED walks with the workload's stop rule (the reference's biased offline kernel has none): "
                        "uniform neighbour, no alias table.  Best of 3 runs, the reference's own wall-clock timer "
                        "around its launch (cuRAND XORWOW set-up per thread included); ours by CUDA events"}
    if wl["kind"] != "walk" or wl["mode"] != "offline" or wl.get("app") != "deepwalk" or E > 0xFFFFFF00:
        return {"unavailable": "the reference's bounded kernels cover offline DeepWalk (biased), unbiased walks with "
                               "a stop rule and offline 2-hop sampling; run --workload c1, c2, dw22, c5, c5s or c4off"}
    n = wl["units"]
    starts = O.gen_starts(n, V, START_SEED)
    paths, lens, sec = R.offline_walk(host["xadj"], host["adjncy"], host["table"], starts, hop, device=device, repeats=3)
    edges = int(lens.sum())
    return {"kernel": "sample_kernel_static via OfflineWalk (src/offline_walk.cu:75-124, 181-230)", "value": edges / sec,
            "unit": "sampled edges/s", "seconds": sec, "sampled_edges": edges, "walkers": n,
            "note": "best of 3 runs, the reference's own wall-clock timer around its launch (cuRAND XORWOW set-up "
                    "per thread included, as in the reference); table built by this library"}


PARITY_WALKERS, PARITY_SEEDS = 10000, 2048


def parity_sample(ctx, wl, host, lo, n_local, d_starts, d_result, d_lengths, mode, hop, threads):
    """Bit-compare the product path with the CPU oracle on the first K units of this rank's shard, at
    the workload's own size: one extra untimed pass over the WHOLE shard through the same entry point
    and path selection the timed steps use (seed WALK_SEED, start seed START_SEED), then the first K
    result rows against oracle.walk / oracle.khop on the same global unit ids; walks also through the
    packed host entry point.  Returns (units compared, equal)."""
    import torch
    from oracle import oracle as O
    khop = wl["kind"] == "khop"
    online = wl["mode"] == "online"
    V = len(host["xadj"]) - 1
    threads = threads or len(os.sched_getaffinity(0)) or O.num_threads()
    K = min(n_local, PARITY_SEEDS if khop else PARITY_WALKERS)
    if K == 0:
        return 0, True
    ctx.generate_starts(n_local, START_SEED, d_starts, id_base=lo)
    h_starts = O.gen_starts(K, V, START_SEED, id_base=lo)
    ok = bool(np.array_equal(d_starts[:K].cpu().numpy().view(np.uint32), h_starts))
    if khop:
        ctx.sample_khop(d_starts, wl["fanout"], mode=mode, flags=wl.get("khop_flags", 0), seed=WALK_SEED,
                        instance_base=lo, data=d_result,
                        sample_lengths=d_lengths, n=n_local)
        cells, lens_per = ctx.khop_layout(wl["fanout"])
        got_d = d_result[:K * cells].cpu().numpy().view(np.uint32).reshape(K, cells)
        got_l = d_lengths[:K * lens_per].cpu().numpy().view(np.uint32).reshape(K, lens_per)
        want_d, want_l = O.khop(host["xadj"], host["adjncy"], host["wgt"], host["table"], h_starts, wl["fanout"],
                                online=online, flags=wl.get("khop_flags", 0), seed=WALK_SEED, instance_base=lo,
                                threads=threads)
        ok = ok and bool(np.array_equal(got_d, want_d)) and bool(np.array_equal(got_l, want_l))
        # the packed host entry point on the same seeds
        packed, pl, pcells, _, _ = ctx.sample_khop_packed(h_starts, wl["fanout"], mode=mode,
                                                          flags=wl.get("khop_flags", 0), seed=WALK_SEED,
                                                          instance_base=lo)
        want_p = want_d[want_d != 0xFFFFFFFF]
        ok = ok and pcells == len(want_p) and bool(np.array_equal(packed[:pcells], want_p))
        return K, ok and bool(np.array_equal(pl, want_l))
    kw = dict(app=app_id(wl), tp=wl.get("tp", 0.0), p=wl.get("p", 2.0), q=wl.get("q", 0.5), seed=WALK_SEED,
              walker_base=lo)
    ctx.walk(d_starts, hop, mode=mode, paths=d_result, lengths=d_lengths, n=n_local, **kw)
    got_p = d_result[:K * hop].cpu().numpy().view(np.uint32).reshape(K, hop)
    got_l = d_lengths[:K].cpu().numpy().view(np.uint32)
    want_p, want_l = O.walk(host["xadj"], host["adjncy"], host["wgt"], host["table"], h_starts, hop, online=online,
                            threads=threads, **kw)
    live = np.arange(hop)[None, :] <= want_l[:, None]
    ok = ok and bool(np.array_equal(got_l, want_l)) and bool(np.array_equal(got_p[live], want_p[live]))
    # the packed host entry point on the same walkers
    for u8 in ((False, True) if hop <= 256 else (False,)):
        packed, pl, cells, _, _ = ctx.walk_packed(h_starts, hop, mode=mode, lengths_u8=u8, **kw)
        ok = ok and bool(np.array_equal(pl, want_l)) and cells == int(want_l.sum()) + K
        ok = ok and bool(np.array_equal(packed[:cells], want_p[live]))
    return K, ok


def online_algorithmic_bytes(ctx, wl, result, lengths):
    """Algorithmic bytes of one online step from the realised frontier: 16 + 4*deg(v) per walk step,
    8 + 4*deg(v) per DISTINCT frontier vertex of each hop (a vertex met several times in one hop is
    built once) plus 8 per sample for k-hop."""
    xadj = ctx.download(weights=False)[0].astype(np.int64)
    deg = np.diff(xadj)
    if wl["kind"] == "khop":
        data, sl = result, lengths
        f1 = wl["fanout"][0]
        total = 8.0 * int(sl.sum())
        for parents in (data[:, 0], data[:, 1:1 + f1].reshape(-1)):
            parents = np.unique(parents[parents != 0xFFFFFFFF])
            total += float((8 + 4 * deg[parents]).sum())
        return total
    paths, lens = result, lengths
    hop = paths.shape[1]
    live = np.arange(hop)[None, :] < lens[:, None]
    return float((16 + 4 * deg[paths[live]]).sum())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the bit-comparison with the CPU oracle")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip the reference's own CUDA walk kernel")
    ap.add_argument("--no-records", action="store_true", help="walk over the 8-byte slot table only")
    ap.add_argument("--cpu-threads", type=int, default=0)
    ap.add_argument("--units", type=int, default=0,
                    help="walkers / seeds in the whole job instead of the workload's own count, e.g. one "
                         "GPU's share of an N-GPU run; the line's config says so")
    args = ap.parse_args()
    wl = dict(WORKLOADS[args.workload])
    if args.units > 0:
        wl["units"] = args.units
        wl["desc"] = wl["desc"] + " [--units %d instead of the configuration's own count]" % args.units
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    args.warmup = max(args.warmup, 3)

    import torch
    from skywalker_b200 import MODE_OFFLINE, MODE_ONLINE
    online = wl["mode"] == "online"
    mode = MODE_ONLINE if online else MODE_OFFLINE
    khop = wl["kind"] == "khop"
    hop = wl.get("length", 0) + 1
    config = {"workload": args.workload + ": " + wl["desc"], "units_total": wl["units"], "mode": wl["mode"],
              "seeds": {"graph": GRAPH_SEED, "weight": WEIGHT_SEED, "start": START_SEED, "walk": WALK_SEED},
              "cache": "inputs larger than L2 (table and CSR are GBs; no flush needed)",
              "parallelism": "units sharded by global id, graph+tables replicated"}
    for k in ("scale", "edge_factor", "raw_edges", "length", "tp", "p", "q", "fanout"):
        if k in wl:
            config[k] = wl[k]

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
        if not online:
            ctx.alias_build_offline()
        host = host_copy(ctx, online, with_weights=True)
        # every step = one pass of the CPU path over the same bounded sample (at most ~10 s, and ~2 minutes
        # for the W + K passes together); value = edges of the K steps / their time
        ref_warm = args.warmup
        best = cpu_leg(host, wl, args.cpu_threads, want_seconds=min(10.0, 120.0 / max(1, args.steps + ref_warm)),
                       steps=args.steps, warmup=ref_warm, build_weights=host["build_weights"])
        out = {"impl": "reference", "metric": "sampled edges/s", "value": best["value"], "unit": "sampled edges/s",
               "n_gpus": args.gpus, "steps": args.steps, "warmup": ref_warm, "ms_per_step": best["seconds"] * 1e3,
               "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u32 ids / f32 prob",
               "data": "synthetic",
               "config": dict(config, V=V, E=E),
               "inputs": "generated on the GPU by the library's seeded generator, then copied to the host; only the "
                         "CPU path is timed",
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
    # a dedicated stream shared by torch and the library, so that torch's events see the kernels
    # (handle 0, torch's default stream, means "the context's own stream" to skw_ctx_set_stream)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    assert stream.cuda_stream != 0
    ctx.set_stream(stream.cuda_stream)

    t0 = time.perf_counter()
    V, E, max_deg = make_graph(ctx, wl)
    t_gen = time.perf_counter() - t0
    peak, peak_kind = measured_peak()
    build_best = min(ctx.alias_build_offline() for _ in range(3))   # reported for every workload

    # multi-GPU: the slot array is cut into N * P equal chunks, rank r builds chunks r, N + r, 2N + r ...
    # (every vertex that overlaps them) and piece k -- the N neighbouring chunks k*N .. k*N + N - 1 -- is
    # all-gathered in place over NCCL while the ranks already build their chunk of piece k + 1; checked
    # against the replicated build
    sliced = None
    if dist is not None and not online:
        from skywalker_b200.api import edge_chunk_ranges
        PIECES = 4
        xadj_h = ctx.download_xadj()
        S, ranges = edge_chunk_ranges(xadj_h, world * PIECES)
        d_slots, d_valid = ctx.alias_device_arrays(padded=True)
        t_slots = torch.as_tensor(d_slots, device=dev)
        t_valid = torch.as_tensor(d_valid, device=dev)
        want = (int(t_slots[:E].sum().item()), int(t_valid.sum().item()))     # checksum of the replicated table
        best = None
        for rep in range(3):
            t_slots.zero_()
            t_valid.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            slice_ms, works = 0.0, []
            for k in range(PIECES):
                c = k * world + rank
                slice_ms += ctx.alias_build_offline(*ranges[c])
                # in place: chunk c of this rank into the piece's N neighbouring chunks on every rank; the
                # collective runs on NCCL's stream behind the build it waits for, beside the next build
                works.append(dist.all_gather_into_tensor(t_slots[k * world * S:(k + 1) * world * S],
                                                         t_slots[c * S:(c + 1) * S], async_op=True))
            # a vertex's flag is set by the ranks that built it and zero elsewhere
            works.append(dist.all_reduce(t_valid, op=dist.ReduceOp.MAX, async_op=True))
            for w in works:
                w.wait()
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            mxs, _ = combine_over_ranks(dist, [(t2 - t0) * 1e3, slice_ms], dev)
            if best is None or mxs[0] < best[0]:
                best = mxs
        got = (int(t_slots[:E].sum().item()), int(t_valid.sum().item()))
        sliced = {"ms": best[0], "slice_build_ms": best[1], "pieces": PIECES,
                  "value": E / (best[0] * 1e-3), "unit": "edges/s",
                  "equals_replicated_build": got == want,
                  "note": "the slot array in N * pieces equal chunks; every rank builds the vertices overlapping "
                          "its chunk of a piece, the piece is all-gathered in place over NCCL while the next one is "
                          "built; then one all-reduce of the per-vertex flags.  slice_build_ms = kernel time of this "
                          "rank's builds (max over ranks)"}
        del xadj_h

    n_total = wl["units"]
    lo, n_local = shard(n_total, world, rank)
    nl = max(n_local, 1)
    starts = torch.empty(nl, dtype=torch.int32, device=dev)
    if khop:
        cells, lens_per = Context.khop_layout(wl["fanout"])
        result = torch.empty(nl * cells, dtype=torch.int32, device=dev)
        lengths = torch.empty(nl * lens_per, dtype=torch.int32, device=dev)
    else:
        result = torch.empty(nl * hop, dtype=torch.int32, device=dev)
        lengths = torch.empty(nl, dtype=torch.int32, device=dev)
    ctx.generate_starts(n_local, START_SEED, starts, id_base=lo)
    torch.cuda.synchronize()

    def step(i, s=starts, r=result, l=lengths, enqueue_only=False, flags=0):
        """One pass over the batch; a new seed (and for k-hop a new batch of seed vertices) every step."""
        if khop:
            if s is starts:
                ctx.generate_starts(n_local, START_SEED + i, starts, id_base=lo)
            return ctx.sample_khop(s, wl["fanout"], mode=mode, flags=wl.get("khop_flags", 0), seed=WALK_SEED + i,
                                   instance_base=lo, data=r,
                                   sample_lengths=l, n=n_local)
        return ctx.walk(s, hop, app=app_id(wl), mode=mode, tp=wl.get("tp", 0.0), p=wl.get("p", 2.0),
                        q=wl.get("q", 0.5), seed=WALK_SEED + i, walker_base=lo, paths=r, lengths=l, n=n_local,
                        enqueue_only=enqueue_only, flags=flags)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    slots_info, records_build_ms = None, None
    use_records = (not online) and (not khop) and wl.get("app") != "node2vec" and not args.no_records
    if use_records:
        # the same walks over the plain 8-byte slot table first (3 accesses per step), for comparison
        ms_list, e_sum = [], 0
        for i in range(args.warmup + 2):
            _, _, ms, edges = step(100 + i)
            if i >= args.warmup:
                ms_list.append(ms)
                e_sum += edges
        slots_info = {"kernel_ms_per_step": float(np.mean(ms_list)), "value": e_sum / (sum(ms_list) * 1e-3),
                      "unit": "sampled edges/s (this rank, kernel time)"}
        records_build_ms = ctx.walk_records_build()
    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = ctx.kernel_launches
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kernel_ms, edges_local = 0.0, 0
    # offline walks are queued back to back (no host round trip between steps); the online paths
    # and k-hop return their counters per call
    queued = (not online) and (not khop)
    ev0.record(stream)
    for i in range(args.steps):
        _, _, ms, edges = step(100 + i, enqueue_only=queued)
        if not queued:
            kernel_ms += ms
            edges_local += edges
    ev1.record(stream)
    barrier()
    launches = ctx.kernel_launches - launches0
    span_ms = ev0.elapsed_time(ev1)
    if queued:
        edges_local = ctx.take_sampled_edges()
        kernel_ms = span_ms     # one kernel per step and nothing else on the stream
    # the timed region can be shorter than one nvidia-smi sampling period: keep the same load running
    # for a moment so that the clock samples are taken under it
    t_hold = time.perf_counter()
    while time.perf_counter() - t_hold < 0.7:
        step(0, enqueue_only=queued)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["note"] = "sampled over the timed region and 0.7 s of the same steps repeated after it"
    if queued:
        ctx.take_sampled_edges()    # drop the count of the extra steps
    mx, sm = combine_over_ranks(dist, [span_ms, kernel_ms, float(edges_local), float(launches)], dev)
    span_ms, kernel_ms = mx[0], mx[1]
    edges_all, launches = sm[2], int(sm[3])
    value = edges_all / (span_ms * 1e-3)

    # online walks again with the tables kept for the rest of the call (the reference's --cache idea):
    # same walks, each distinct vertex built once per call instead of once per step
    cached_info = None
    if online and not khop:
        from skywalker_b200 import WALK_CACHE_TABLES
        ms_c, e_c = 0.0, 0
        for i in range(2):
            _, _, ms, edges = step(100 + i, flags=WALK_CACHE_TABLES)
            ms_c += ms
            e_c += edges
        cached_info = {"kernel_ms_per_step": ms_c / 2, "value": e_c / (ms_c * 1e-3),
                       "unit": "sampled edges/s (this rank, kernel time)",
                       "note": "SKW_WALK_CACHE_TABLES: every distinct vertex built once per call"}

    # algorithmic bytes of an online step need the realised frontier of the last step
    online_bytes, last_edges = None, 1.0
    if online and rank == 0:
        res_h = result.cpu().numpy().view(np.uint32).reshape(nl, -1)
        len_h = lengths.cpu().numpy().view(np.uint32)
        online_bytes = online_algorithmic_bytes(ctx, wl, res_h, len_h.reshape(nl, -1) if khop else len_h)
        last_edges = float(len_h.sum())

    # end to end through the host-buffer entry point: pinned inputs in, full result arrays out
    e2e = None
    if not args.no_e2e:
        h_starts = torch.empty(nl, dtype=torch.int32).pin_memory()
        h_res = torch.empty(result.numel(), dtype=torch.int32).pin_memory()
        h_len = torch.empty(lengths.numel(), dtype=torch.int32).pin_memory()
        h_starts.copy_(starts.cpu())
        np_s, np_r, np_l = (t.numpy().view(np.uint32) for t in (h_starts, h_res, h_len))
        if khop:
            np_r, np_l = np_r.reshape(nl, -1), np_l.reshape(nl, -1)
        e_steps = max(1, min(args.steps, 20))

        def timed_host_calls(call):
            for i in range(3):      # warm calls: staging buffers reach their steady size
                call(50 + i)
            barrier()
            t0 = time.perf_counter()
            edges, per_call = 0, []
            for i in range(e_steps):
                t1 = time.perf_counter()
                edges += call(100 + i)
                per_call.append(round((time.perf_counter() - t1) * 1e3, 3))
            barrier()
            ms_ = (time.perf_counter() - t0) * 1e3
            m2, s2 = combine_over_ranks(dist, [ms_, float(edges)], dev)
            return m2[0], s2[1], per_call

        e_ms, e_edges, e_calls = timed_host_calls(lambda i: step(i, np_s, np_r, np_l)[3])
        rows = {"ms_per_call_this_rank": e_calls, "ms_per_call_median": float(np.median(e_calls)), "value": e_edges / (e_ms * 1e-3), "unit": "sampled edges/s", "steps": e_steps,
                "ms_per_step": e_ms / e_steps, "h2d_bytes_per_step": 4 * n_local,
                # walks into pinned memory transfer the written cells of each row (length + 1) and the lengths;
                # k-hop trees are dense and are copied whole
                "d2h_bytes_per_step": (4 * (result.numel() + lengths.numel()) if khop else
                                       int(4 * (e_edges / e_steps / world + 2 * n_local))),
                "note": "host-buffer entry point with pinned memory: start vertices H2D, kernels, then "
                        + ("the whole result tree D2H" if khop else
                           "cells 0..length of every path row written into the pinned n x hop_num matrix by a "
                           "kernel, plus the lengths D2H")}
        e2e = rows
        if khop:
            # the same trees returned packed: only cells that hold a sample cross the bus
            flat_r = np_r.reshape(-1)

            def packed_tree_call(i):
                out = ctx.sample_khop_packed(np_s, wl["fanout"], mode=mode, flags=wl.get("khop_flags", 0),
                                             seed=WALK_SEED + i, instance_base=lo, packed=flat_r,
                                             sample_lengths=np_l, n=n_local)
                packed_tree_call.cells = out[2]
                return out[4]
            p_ms, p_edges, p_calls = timed_host_calls(packed_tree_call)
            e2e = {"ms_per_call_this_rank": p_calls, "ms_per_call_median": float(np.median(p_calls)),
                   "value": p_edges / (p_ms * 1e-3), "unit": "sampled edges/s", "steps": e_steps,
                   "ms_per_step": p_ms / e_steps, "h2d_bytes_per_step": 4 * n_local,
                   "d2h_bytes_per_step": int(4 * (packed_tree_call.cells + lengths.numel())),
                   "note": "host-buffer entry point skw_sample_khop_packed with pinned memory: seed vertices H2D, "
                           "per-hop kernels, then the cells of the result tree that hold a sample packed back to "
                           "back on the device and copied slice by slice, plus the per-vertex sample counts",
                   "dense_tree": rows}
        if not khop:
            # the same walks returned packed (lengths + the walks back to back): only result cells cross
            # the bus, as one contiguous stream instead of one small write per row
            def packed_call(i, u8=False):
                return ctx.walk_packed(np_s, hop, app=app_id(wl), mode=mode, tp=wl.get("tp", 0.0), p=wl.get("p", 2.0),
                                       q=wl.get("q", 0.5), seed=WALK_SEED + i, walker_base=lo, packed=np_r,
                                       lengths=np_l.view(np.uint8)[:n_local] if u8 else np_l, n=n_local,
                                       lengths_u8=u8)[4]
            p_ms, p_edges, p_calls = timed_host_calls(packed_call)
            packed32 = {"ms_per_call_this_rank": p_calls, "ms_per_call_median": float(np.median(p_calls)),
                        "value": p_edges / (p_ms * 1e-3), "unit": "sampled edges/s", "steps": e_steps,
                        "ms_per_step": p_ms / e_steps, "h2d_bytes_per_step": 4 * n_local,
                        "d2h_bytes_per_step": int(4 * (p_edges / e_steps / world + 2 * n_local)),
                        "note": "skw_walk_packed: the same with 32-bit lengths"}
            e2e = packed32
            if hop <= 256:
                # lengths of at most 255 travel as bytes: the result is bound by the bus
                p_ms, p_edges, p_calls = timed_host_calls(lambda i: packed_call(i, True))
                e2e = {"ms_per_call_this_rank": p_calls, "ms_per_call_median": float(np.median(p_calls)),
                       "value": p_edges / (p_ms * 1e-3), "unit": "sampled edges/s", "steps": e_steps,
                       "ms_per_step": p_ms / e_steps, "h2d_bytes_per_step": 4 * n_local,
                       "d2h_bytes_per_step": int(4 * (p_edges / e_steps / world + n_local) + n_local),
                       "packed_u32_lengths": packed32}
            e2e["note"] = ("host-buffer entry point skw_walk_packed_u8 with pinned memory: start vertices H2D, walk "
                           "kernel, prefix sum of the lengths, pack kernel writing lengths[w] + 1 vertices per walk "
                           "back to back, one contiguous copy per slice into the pinned result buffer, lengths "
                           "D2H as bytes")
            e2e["row_layout"] = rows

    # NCCL gather of the results to rank 0 (outside the timed region): the per-unit lengths, and the
    # result arrays themselves when the shards are equal and fit beside the graph on rank 0
    gather_ms, gather_note = None, None
    if dist is not None:
        bufs = [torch.empty_like(lengths) for _ in range(world)] if rank == 0 else None
        dist.gather(lengths, bufs, dst=0)       # first collective sets NCCL up
        torch.cuda.synchronize()
        whole = wl["units"] % world == 0 and result.numel() * 4 * world <= (16 << 30)
        rbufs = [torch.empty_like(result) for _ in range(world)] if (rank == 0 and whole) else None
        t0 = time.perf_counter()
        dist.gather(lengths, bufs, dst=0)
        if whole:
            dist.gather(result, rbufs, dst=0)
        torch.cuda.synchronize()
        gather_ms = (time.perf_counter() - t0) * 1e3
        gather_note = ("lengths and result arrays (%d MB per rank)" % (result.numel() * 4 >> 20)) if whole else "lengths"
        del rbufs

    # the ceiling the step kernels run against: dependent random 32-byte accesses per second, probed
    # live on this GPU (footprint 16 GiB, far beyond L2)
    probe_gacc = None
    if rank == 0:
        try:
            probe_gacc = ctx.probe_random_gather(16 << 30, 128)
        except Exception:
            probe_gacc = None

    # Parity at the workload's own size, on every rank: the first K units of the rank's shard against the
    # CPU oracle (bit for bit), results AND-reduced.  The oracle needs the graph (and table) on the host;
    # ranks take turns in waves sized by the host memory that is free.
    cpu, parity, ref_cuda = None, None, None
    need = host_copy_bytes(V, E, online) + (4 * E if world == 1 and not online else 0)
    avail = host_memory_available()
    at_once = world if avail is None else int(min(world, (0.6 * avail) // need))
    if dist is not None:
        t = torch.tensor([at_once], dtype=torch.int64, device=dev)
        dist.broadcast(t, src=0)       # rank 0's reading decides for all (one host)
        at_once = int(t.item())
    if args.no_parity:
        parity = {"units": 0, "equal": None, "ranks": world, "skipped": "--no-parity"}
    elif at_once < 1:
        parity = {"units": 0, "equal": None, "ranks": world,
                  "skipped": "host memory: %.1f GB free, the checker's inputs need %.1f GB" % ((avail or 0) / 1e9, need / 1e9)}
    else:
        units, equal = 0, True
        for wave in range(0, world, at_once):
            if wave <= rank < wave + at_once:
                host = host_copy(ctx, online, with_weights=(world == 1))
                units, equal = parity_sample(ctx, wl, host, lo, n_local, starts, result, lengths, mode, hop,
                                             args.cpu_threads)
                if rank == 0 and world == 1 and not args.no_cpu_baseline:
                    cpu = cpu_leg(host, wl, args.cpu_threads, build_weights=host["build_weights"])
                    cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample", "alias_build_edges_per_s")}
                if rank == 0 and world == 1 and not args.no_reference_cuda:
                    try:
                        ref_cuda = reference_cuda_leg(host, wl, hop, local_rank, ctx, (starts, result, lengths),
                                                      records=use_records)
                    except Exception as e:      # never lose the bench line to the comparison arm
                        ref_cuda = {"unavailable": "failed: %s" % e}
                del host
            if dist is not None:
                dist.barrier()
        t = torch.tensor([1 if equal else 0, units], dtype=torch.int64, device=dev)
        if dist is not None:
            mn = t.clone()
            dist.all_reduce(mn, op=dist.ReduceOp.MIN)
            t = mn
        parity = {"units": int(t[1].item()), "equal": bool(t[0].item()), "ranks": world,
                  "what": "first K %s of every rank's shard, row layout%s, against the CPU oracle bit for bit"
                          % ("seeds" if khop else "walkers",
                             " and packed tree" if khop else " and packed layout (32-bit and byte lengths)")}
    config["parity_sample"] = parity
    if sliced is not None:
        config["alias_build_sliced_equals_replicated"] = sliced["equals_replicated_build"]

    if rank == 0:
        per_step_ms = kernel_ms / args.steps
        edges_per_step_rank = edges_all / args.steps / world
        if online:
            bytes_note = ("16 + 4*deg(v) bytes per walk step" if not khop else
                          "8 + 4*deg(v) per distinct frontier vertex of a hop + 8 per sample") + ", summed over the last step's frontier"
            achieved = online_bytes / (per_step_ms * 1e-3) / 1e9 * (edges_per_step_rank / max(last_edges, 1.0))
            direct = not khop      # online walks compute drawn slots directly unless a flag asks for tables
            kernel_name = ("walk_online_direct_kernel" if direct else
                           "frontier_collect + degree-class builders + " + ("khop_hop_kernel" if khop else
                                                                            "walk_online_step_kernel"))
        else:
            bytes_note = "24 bytes per sampled edge"
            achieved = edges_per_step_rank * ALG_BYTES_PER_EDGE / (per_step_ms * 1e-3) / 1e9
            kernel_name = (("walk_records_ppr_kernel" if wl.get("app") == "ppr" else "walk_records_walk_kernel")
                           if use_records else "walk_offline_kernel")
        per_edge = DRAM_BYTES_PER_SAMPLED_EDGE.get(kernel_name)
        traffic = per_edge * edges_per_step_rank if per_edge else None
        build_gbs = E * ALG_BYTES_PER_BUILD_EDGE / (build_best * 1e-3) / 1e9
        out = {
            "metric": "sampled edges/s", "value": value, "unit": "sampled edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": span_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u32 ids / f32 prob", "data": "synthetic",
            "config": dict(config, V=V, E=E),
            "max_degree": max_deg, "units_per_gpu": n_local, "graph_gen_s": t_gen,
            "kernel_ms_per_step": per_step_ms,
            "sampled_edges_per_step": edges_all / args.steps,
            "alias_build": {"value": E / (build_best * 1e-3), "unit": "edges/s", "ms": build_best,
                            "roofline": {"bound": "hbm", "achieved": build_gbs, "peak": peak, "unit": "GB/s",
                                         "frac": build_gbs / peak, "peak_kind": peak_kind}},
            "alias_build_sliced": sliced,
            "layout": "fused 32-byte walk records" if use_records else "8-byte slots",
            "walk_records_build_ms": records_build_ms, "slots_layout": slots_info,
            "online_cached_tables": cached_info,
            "roofline": {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_kind": peak_kind,
                         "algorithmic_bytes": bytes_note,
                         "random_access_probe_gaccess_per_s": probe_gacc,
                         "sampled_edges_per_probe_access": (edges_per_step_rank / (per_step_ms * 1e-3) / 1e9 / probe_gacc
                                                            if probe_gacc else None),
                         "note": "a step is a chain of dependent random accesses; the probe is the rate of such "
                                 "accesses this GPU sustains whatever their size (8-128 B), so sampled edges per "
                                 "probe access, not the byte fraction, says how close the step kernel is to the "
                                 "hardware"},
            "cpu_baseline": cpu, "reference_cuda": ref_cuda, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "result_gather_ms": gather_ms, "result_gather": gather_note,
        }
        print(json.dumps(out))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    ctx.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())

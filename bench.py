#!/usr/bin/env python
"""Benchmark of the sampled mini-batch GCN training path (ALGORITHM:GCNNEIGHBORGPU) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload reddit|arxiv|products|papers] [--impl reference]

A "step" is one mini-batch through the whole hot path: fan-out sampling -> block construction ->
feature/label gather -> per-layer aggregation + dense layer -> loss -> backward -> gradient sum over
ranks -> Adam.  Rank 0 prints ONE JSON line.

  value      aggregated edges per second over all ranks, seeds already resident in HBM.
             Aggregated edges of a step = sum of e_size over the blocks (forward, the reference's
             Sampler::get_compute_cnt, core/ntsSampler.hpp:629-635) + sum over blocks l >= 1 (backward;
             the input-side block is never back-propagated, core/ntsContext.hpp:292).
  e2e        the same metric through the public API (the trainer's batch loop) with the batch's seeds
             copied from pinned host memory and the loss read back to the host every step.
  timing     a region is EXACTLY --steps K steps between a barrier + device synchronize on both sides, timed
             with CUDA events, max over ranks.  K steps of this workload last a few milliseconds, so the
             region is repeated until about --min-region-s of device time has been measured and the MEDIAN
             region is reported (`regions` says how many); the clock sampler runs across all of them.
  roofline   the dominant kernel, the layer-0 forward aggregation (spmm_ring_kernel with the feature gather
             fused; every launch of the timed regions, timed by the library's own CUDA event pairs on the
             launching stream): algorithmic bytes / that time against the measured HBM copy bandwidth.
  all_aggregation  the same ratio over all aggregation launches (forward and backward) of the timed regions.
  cpu_baseline  the reference's own CPU training path (oracle/_ref/ref_harness, kind "reference") timed on
             this box's host cores on a few batches of the same workload, at the reference's default thread
             count and with all cores; when that binary is absent, the C oracle port of it (kind "port").
  secondary  the Products-shaped workload (3 layers, 20 % of the rows cached, the others read from pinned host
             memory) measured the same way at this N, so that its scaling can be read from the lines of a
             1/2/4/8 run; --no-secondary switches it off.

The datasets the reference uses are not available; graphs, features and labels are seeded synthetic
data with the published shapes (see neutronbench_b200/synth.py).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0   # earlier measurement on this pool; used only when MEASURED_PEAKS.json is absent
NVLINK_PEER_GBS = 770.0     # measured peer copy bandwidth per direction per GPU on this pool (900 nominal)


def ncu_traffic_bytes(workload, fuse_gather, all_cached):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the layer-0 forward aggregation, from the
    committed ncu capture of this workload (profiles/ncu_traffic.json holds the figure and names the capture)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    if not os.path.exists(path):
        return None
    try:
        table = json.load(open(path))
    except Exception:
        return None
    key = f"{workload}|fuse_gather={int(bool(fuse_gather))}|all_cached={int(bool(all_cached))}"
    entry = table.get(key)
    return None if entry is None else entry.get("dram_bytes_per_launch")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="timed steps per region and rank (0 = one epoch of this rank's shard)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="reddit", choices=["arxiv", "reddit", "products", "papers", "cora"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cache-rate", type=float, default=None, help="override the workload's GPU cache rate")
    ap.add_argument("--cpu-batches", type=int, default=3, help="batches timed for the CPU baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fuse-gather", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the Products-shaped secondary measurement")
    ap.add_argument("--secondary-steps", type=int, default=100)
    ap.add_argument("--min-region-s", type=float, default=0.3, help="repeat the K-step region until this much time is measured")
    ap.add_argument("--max-regions", type=int, default=100)
    ap.add_argument("--python-step", action="store_true", help="issue a step kernel by kernel from Python instead of nb_gcn_step")
    ap.add_argument("--pipelines", type=int, default=0,
                    help="PIPELINES of the reference cfg: P batches in flight (one training, P-1 being sampled), 1 = plain "
                         "loop; 0 = 4 when the host has at least 4 cores per rank (every batch in flight is a library "
                         "thread that waits on its stream), else 3")
    ap.add_argument("--pdl", type=int, default=None, help="1 / 0: programmatic dependent launch for the training half's kernels")
    ap.add_argument("--stage-misses", type=int, default=None,
                    help="1 / 0: uncached rows staged once per distinct source by the sampling half (default: only for a "
                         "feature table sharded over GPUs)")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="nb_gcn_set_option on the trainer's handle (tuning switches; results never depend on them)")
    ap.add_argument("--cache-row-pitch", type=int, default=0, help="floats between rows of the GPU feature cache (0: default)")
    ap.add_argument("--value-readback", type=int, default=1,
                    help="1: the device-resident region also reads every step's loss back (one step late), as a "
                         "training loop that logs its loss does; 0: nothing is read inside that region (3 %% faster on "
                         "one GPU, but with several ranks the unthrottled host threads cost more than that)")
    ap.add_argument("--settle-s", type=float, default=0.5,
                    help="seconds of untimed regions (after the W warm-up steps) before the first timed region")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload's node and edge counts (functional checks)")
    ap.add_argument("--seed", type=int, default=2000)
    return ap.parse_args()


def workload_config(name, args):
    from neutronbench_b200 import GCNConfig, synth
    import dataclasses
    sh = synth.SHAPES[name]
    if args.scale != 1.0:
        sh = dataclasses.replace(sh, vertices=max(1000, int(sh.vertices * args.scale)),
                                 edges=max(10000, int(sh.edges * args.scale)))
    hidden = [sh.hidden] * (len(sh.fanout) - 1)
    cache_rate = {"arxiv": 1.0, "reddit": 1.0, "products": 0.2, "papers": 0.0}[name]
    if args.cache_rate is not None:
        cache_rate = args.cache_rate
    cfg = GCNConfig(layers=[sh.feature] + hidden + [sh.classes], fanout=sh.fanout, batch_size=sh.batch,
                    learn_rate=0.01, weight_decay=0.0001, drop_rate=0.5,
                    cache_type="rate" if cache_rate > 0 else "none", cache_rate=cache_rate, seed=args.seed,
                    fuse_gather=not args.no_fuse_gather,
                    stage_misses=None if args.stage_misses is None else bool(args.stage_misses),
                    cache_row_pitch=getattr(args, "cache_row_pitch", 0))
    return sh, cfg


def build_workload(name, args, device, rank=0, world=1):
    """Graph topology, features, labels and the train split, all seeded.  Data preparation is not timed."""
    import torch
    from neutronbench_b200 import FullyRepGraph, GNNDatum, Workspace, synth
    sh, cfg = workload_config(name, args)
    edges = synth.rmat_torch(sh.vertices, sh.edges, sh.rmat, args.seed, device=device)
    big = Workspace(int(edges.size(0)) * 9 + sh.vertices * 16 + (64 << 20), device)
    graph = FullyRepGraph.from_edges(edges, sh.vertices, big)
    torch.cuda.synchronize()
    del edges
    big.close()
    del big
    torch.cuda.empty_cache()
    gen = torch.Generator(device=device).manual_seed(args.seed + 1)
    mask = synth.split_mask(sh.vertices, args.seed)
    train_ids = np.nonzero(mask == 0)[0].astype(np.uint32)
    if name == "papers":
        # the table does not fit one GPU at the full shape: every rank generates and keeps the rows of its own id range
        from neutronbench_b200.peer import ShardedFeatureTable, shard_rows_for
        rows_per = shard_rows_for(sh.vertices, world)
        lo, hi = rank * rows_per, min(sh.vertices, (rank + 1) * rows_per)
        g2 = torch.Generator(device=device).manual_seed(args.seed + 7 + rank)
        local = torch.randn((max(hi - lo, 0), sh.feature), generator=g2, device=device, dtype=torch.float32)
        label = torch.randint(0, sh.classes, (sh.vertices,), generator=gen, device=device, dtype=torch.int64)
        if world > 1:
            shards = ShardedFeatureTable.from_rank_shard(local, sh.vertices, rank, world, device)
            del local
        else:
            shards = ShardedFeatureTable.from_local_parts([local], rows_per)
        datum = GNNDatum(None, label, mask, shards=shards)
        return sh, cfg, graph, datum, train_ids, None
    feat_dev = torch.randn((sh.vertices, sh.feature), generator=gen, device=device, dtype=torch.float32)
    label = torch.randint(0, sh.classes, (sh.vertices,), generator=gen, device=device, dtype=torch.int64)
    if cfg.cache_type == "rate" and cfg.cache_rate >= 1.0:
        feature = feat_dev                       # every row is a cache hit; the table only seeds the cache
    else:
        feature = feat_dev.cpu().pin_memory()    # misses are reads of mapped pinned host memory
    datum = GNNDatum(feature, label, mask)
    return sh, cfg, graph, datum, train_ids, feat_dev


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = f"/tmp/nb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", os.environ.get("NB_CLOCK_LMS", "200"), "-i", str(self.index)],
                                         stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.remove(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def aggregated_edges(blocks):
    fwd = sum(b.e_size for b in blocks)
    bwd = sum(b.e_size for b in blocks[1:])
    return fwd, bwd


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_arm(sh, cfg, graph, feat_dev, label, train_ids, batches, warmup, seed):
    """The reference's CPU path as restated by the oracle (sample_one + MiniBatchFuseOp GCN step,
    toolkits/GCN_CPU_NEIGHBOR.hpp:225-427) on the host cores: OpenMP aggregation, BLAS dense layers
    (numpy stands in for libtorch's CPU mm).  Returns (edges/s, ms per batch, threads, per-batch ms)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    co = graph.column_offset.cpu().numpy().astype(np.uint64)
    ri = graph.row_indices.cpu().numpy().view(np.uint32)
    feat = feat_dev.cpu().numpy()
    lab = label.cpu().numpy()
    rng = np.random.RandomState(seed)
    W0 = np.concatenate([rng.uniform(-1, 1, cfg.layers[i] * cfg.layers[i + 1]).astype(np.float32)
                         * np.float32(np.sqrt(6.0 / (cfg.layers[i] + cfg.layers[i + 1])))
                         for i in range(len(cfg.layers) - 1)])
    net = oracle.GCN(cfg.layers, W0, cfg.learn_rate, cfg.weight_decay, cfg.drop_rate, cfg.seed, blas=True)
    threads = oracle.lib().orc_num_threads()
    times, edges = [], 0
    for b in range(warmup + batches):
        seeds = train_ids[b * cfg.batch_size: (b + 1) * cfg.batch_size]
        t0 = time.perf_counter()
        blocks, _ = oracle.sample_batch(co, ri, sh.vertices, seeds, list(cfg.fanout), cfg.seed, b)
        net.train_step(blocks, feat, lab)
        dt = time.perf_counter() - t0
        if b >= warmup:
            times.append(dt)
            f, bw = aggregated_edges(blocks)
            edges += f + bw
    total = sum(times)
    return edges / total, 1e3 * total / len(times), threads, [1e3 * t for t in times]


def cpu_arm_reference(sh, cfg, graph, feat_dev, label, train_ids, batches, warmup):
    """The reference's OWN CPU training path (oracle/_ref/ref_harness bench: its Sampler::sample_one,
    get_feature, MiniBatchFuseOp, libtorch mm/loss/autograd and CPU Adam, compiled from the reference
    tree with single-rank shims) on the same graph, features and seed list, once with the reference's default
    thread count (ncpus/2 - 1, core/ntsSampler.hpp:221-228) and once with THREADS = all cores.  Returns a list of
    (edges/s, ms per batch, threads), or None when the harness binary is not there (it is built only where the
    reference tree exists)."""
    import re
    import shutil
    import tempfile
    import torch
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    if not os.path.exists(harness):
        return None
    tmp = tempfile.mkdtemp(prefix="nb_ref_")
    try:
        V = sh.vertices
        co, ri = graph.column_offset, graph.row_indices
        deg = co[1:] - co[:-1]
        dst = torch.repeat_interleave(torch.arange(V, device=co.device, dtype=torch.int32), deg)
        pairs = torch.stack([ri, dst], dim=1).cpu().numpy()      # CSC order: rebuilding gives the same CSC
        del dst
        pairs.tofile(os.path.join(tmp, "g.edge"))
        del pairs
        feat_dev.cpu().numpy().astype("<f4").tofile(os.path.join(tmp, "feat.f32"))
        label.cpu().numpy().astype("<i8").tofile(os.path.join(tmp, "label.i64"))
        need = (warmup + batches) * cfg.batch_size
        train_ids[:need].astype("<u4").tofile(os.path.join(tmp, "seeds.u32"))
        runs = []
        for threads_arg in (0, os.cpu_count() or 0):
            cmd = [harness, "bench", os.path.join(tmp, "g.edge"), str(V), os.path.join(tmp, "feat.f32"),
                   os.path.join(tmp, "label.i64"), os.path.join(tmp, "seeds.u32"), ",".join(map(str, cfg.fanout)),
                   "-".join(map(str, cfg.layers)), str(cfg.batch_size), str(warmup), str(batches), str(cfg.drop_rate),
                   str(cfg.learn_rate), str(cfg.weight_decay), str(threads_arg)]
            out = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
            m = re.search(r"REFBENCH ms_per_batch=([0-9.]+) agg_edges_per_batch=([0-9.]+) omp_threads=(\d+) batches=(\d+)",
                          out.stdout)
            if not m or int(m.group(4)) == 0:
                continue
            ms, edges, threads = float(m.group(1)), float(m.group(2)), int(m.group(3))
            runs.append((edges / (ms * 1e-3), ms, threads))
        return runs or None
    except Exception:
        return None
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def host_baseline(sh, cfg, graph, feat, label, train_ids, batches, warmup, seed):
    """Reference binary when available (kind "reference"), otherwise the oracle port (kind "port")."""
    runs = cpu_arm_reference(sh, cfg, graph, feat, label, train_ids, batches, warmup)
    if runs:
        eps, ms, threads = max(runs, key=lambda r: r[0])     # the faster of the two thread counts is the baseline
        return {"value": eps, "unit": "edges/s", "cores": threads, "kind": "reference", "ms_per_step": ms,
                "host_cpus": os.cpu_count(),
                "by_threads": [{"threads": t, "value": e, "ms_per_step": m} for (e, m, t) in runs],
                "sample": f"{batches} mini-batches of the same workload after {warmup} warm-up: the reference's own "
                          f"CPU path (Sampler::sample_one + MiniBatchFuseOp + libtorch, built -O3 -march=native) with "
                          f"THREADS at its default ({runs[0][2]}) and at all {os.cpu_count()} cores; the faster run "
                          f"({threads} threads) is reported; libtorch uses its default intra-op threads for the dense "
                          f"layers"}
    eps, ms, threads, _ = cpu_arm(sh, cfg, graph, feat, label, train_ids, batches, warmup, seed)
    return {"value": eps, "unit": "edges/s", "cores": threads, "kind": "port", "ms_per_step": ms,
            "sample": f"{batches} mini-batches of the same workload after {warmup} warm-up, C oracle port of the "
                      f"reference's CPU path, OpenMP + BLAS on all host threads"}


# ------------------------------------------------------------------------------------------ GPU arm
def measure(tk, graph, cfg, train_ids, args, K, W, rank, world, local_rank, device, want_events=True):
    """Times the trainer's own batch loop on this rank's share of the shuffled train list.  Returns a dict with
    the device-timed and end-to-end figures (max over ranks per region, median over regions)."""
    import torch
    import torch.distributed as dist
    from neutronbench_b200 import Sampler, _lib
    from neutronbench_b200.toolkit import shard_for_rank

    rng = np.random.RandomState(args.seed)
    ids = train_ids.copy()
    rng.shuffle(ids)
    shard = shard_for_rank(ids, rank, world)
    if K <= 0:
        K = (len(shard) + cfg.batch_size - 1) // cfg.batch_size      # one epoch of this rank's shard

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_vec(values, op):
        if world == 1:
            return list(values)
        t = torch.tensor(list(values), dtype=torch.float64, device=device)
        dist.all_reduce(t, op=op)
        return t.tolist()

    def steps(smp, n, staged):
        read = (not staged) or bool(args.value_readback)
        if cfg.pipelines > 1:
            done = tk.run_pipelined(smp, max_batches=n, train=True, read_back=read, pad_to_steps=n)[3]
            assert done == n
            return
        for _ in range(n):
            tk.train_step(smp)
            if read:
                tk.read_stats()

    def run(staged, record_events, settle=False):
        regions_cap = max(1, args.max_regions)
        settle_cap = max(1, 4000 // max(K, 1)) if (settle and args.settle_s > 0) else 0
        # + the fully timed region after the timed ones, + the untimed settling regions before them
        need = (W + K * (regions_cap + 1 + settle_cap)) * cfg.batch_size
        reps = (need + len(shard) - 1) // len(shard)
        seeds_all = np.tile(shard, reps)[:need]
        smp = Sampler(graph, seeds_all, cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed, with_edge_weights=False)
        if staged:
            smp.stage_seeds_on_device()
        clocks = ClockSampler(local_rank)
        if rank == 0 and record_events:
            clocks.start()           # nvidia-smi needs ~0.1 s to produce its first sample: start before warm-up
        steps(smp, W, staged)
        barrier()
        if settle and args.settle_s > 0:
            # Untimed regions of K steps until the job has run for settle_s seconds: with eight ranks on a host of 32
            # cores the first few tenths of a second after start-up run up to 10 % slower than the steady state
            # (whichever pass comes first shows it, the other one does not), and W warm-up steps are over in a millisecond.
            s0 = torch.cuda.Event(enable_timing=True)
            s1 = torch.cuda.Event(enable_timing=True)
            s0.record()
            steps(smp, K, staged)
            s1.record()
            barrier()
            one = reduce_vec([s0.elapsed_time(s1)], dist.ReduceOp.MAX if world > 1 else None)[0]
            more = min(settle_cap, max(1, math.ceil(args.settle_s * 1e3 / max(one, 1e-3)))) - 1
            for _ in range(more):
                steps(smp, K, staged)
            barrier()
        tk.events = [] if (record_events and not tk.use_engine) else None
        if record_events and tk.use_engine:
            # inside the timed regions only the dominant kernel is bracketed by events (two records per step); the
            # other aggregation launches and the per-phase times are taken in one more region after them, which does
            # not count towards `value`: an event record between two kernels keeps the second from starting under
            # the first one's tail, and eight of them per step cost 13 us of a 0.23 ms step (more with several ranks)
            _lib.call("nb_gcn_set_timing", tk._ensure_engine(), 2)
        launches0 = _lib.load().nb_launch_count()
        phase = None
        region_ms, region_edges = [], []
        regions = 1
        r = 0
        while r < regions:
            tk.agg_edges_fwd = tk.agg_edges_bwd = 0
            t0 = torch.cuda.Event(enable_timing=True)
            t1 = torch.cuda.Event(enable_timing=True)
            t0.record()
            steps(smp, K, staged)
            t1.record()
            barrier()
            region_ms.append(t0.elapsed_time(t1))
            region_edges.append(tk.agg_edges_fwd + tk.agg_edges_bwd)
            if r == 0:   # how many regions make up the minimum measured time: decided once, the same on every rank
                first = reduce_vec([region_ms[0]], dist.ReduceOp.MAX if world > 1 else None)[0]
                regions = min(regions_cap, max(1, math.ceil(args.min_region_s * 1e3 / max(first, 1e-3))))
            r += 1
        clk = clocks.stop() if (rank == 0 and record_events) else None
        launches = _lib.load().nb_launch_count() - launches0
        ev = tk.events
        tk.events = None
        if record_events and tk.use_engine:
            import ctypes
            eng = tk._ensure_engine()
            a_ms, a_b, a_n = (ctypes.c_double * 2)(), (ctypes.c_uint64 * 2)(), (ctypes.c_uint64 * 2)()
            _lib.call("nb_gcn_read_timing_by_class", eng, a_ms, a_b, a_n)
            dominant = (a_ms[0], int(a_b[0]), int(a_n[0]))          # layer-0 aggregation over the timed regions
            _lib.call("nb_gcn_set_timing", eng, 1)                   # one more region of K steps, every class timed
            steps(smp, K, staged)
            barrier()
            f_ms, f_b, f_n = (ctypes.c_double * 2)(), (ctypes.c_uint64 * 2)(), (ctypes.c_uint64 * 2)()
            _lib.call("nb_gcn_read_timing_by_class", eng, f_ms, f_b, f_n)
            ph = (ctypes.c_double * 4)()
            _lib.call("nb_gcn_read_phase_times", eng, ph)
            _lib.call("nb_gcn_set_timing", eng, 0)
            ev = ("engine", dominant, list(f_ms), [int(x) for x in f_b], [int(x) for x in f_n])
            phase = {"sample_host": ph[0] / K, "trans": ph[1] / K, "graph": ph[2] / K, "nn": ph[3] / K,
                     "region": "one region of K steps with every launch class timed, after the regions that make up `value`"}
        tk.check_device_errors()     # a bounded wait that gave up, or an id outside its table, voids the numbers
        ms_max = reduce_vec(region_ms, dist.ReduceOp.MAX if world > 1 else None)
        edges_sum = reduce_vec(region_edges, dist.ReduceOp.SUM if world > 1 else None)
        order = sorted(range(len(ms_max)), key=lambda i: ms_max[i])
        mid = order[len(order) // 2] if len(order) % 2 else order[len(order) // 2 - 1]   # a measured region, not a mean
        return {"ms": ms_max[mid], "edges": edges_sum[mid], "regions": len(ms_max), "ms_min": min(ms_max),
                "ms_max": max(ms_max), "launches_per_region": launches / len(ms_max), "clocks": clk, "events": ev,
                "total_steps": K * len(ms_max), "phase_ms_per_step": phase}

    a = run(staged=True, record_events=want_events, settle=True)
    b = run(staged=False, record_events=False)
    return K, a, b


def roofline_of(events, peak, peak_src, traffic, cfg):
    def gbps(nbytes, ms):
        return nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0

    if isinstance(events, tuple):      # native step: totals measured by the library's own CUDA events
        _, (dom_ms, dom_bytes, dom_n), cls_ms, cls_bytes, cls_n = events
        all_ms, all_bytes, all_n = sum(cls_ms), sum(cls_bytes), sum(cls_n)
        per_call = {"layer0_forward": {"GBps": gbps(dom_bytes, dom_ms), "ms_avg": dom_ms / max(dom_n, 1),
                                       "bytes_avg": dom_bytes / max(dom_n, 1)},
                    "other_aggregation": {"GBps": gbps(cls_bytes[1], cls_ms[1]), "ms_avg": cls_ms[1] / max(cls_n[1], 1),
                                          "bytes_avg": cls_bytes[1] / max(cls_n[1], 1)}}
    else:                              # Python step: one event pair per aggregation call
        per_kernel = {}
        for (name, b, s_, e_) in events or []:
            d = per_kernel.setdefault(name, [0, 0.0, 0])
            d[0] += b
            d[1] += s_.elapsed_time(e_)
            d[2] += 1
        first = next((k for k in ("fwd0_gather_fused", "fwd0") if k in per_kernel), None)
        dom_bytes, dom_ms, dom_n = per_kernel[first] if first else (0, 0.0, 0)
        all_ms = sum(v[1] for v in per_kernel.values())
        all_bytes = sum(v[0] for v in per_kernel.values())
        all_n = sum(v[2] for v in per_kernel.values())
        per_call = {k: {"GBps": gbps(v[0], v[1]), "ms_avg": v[1] / v[2], "bytes_avg": v[0] / v[2]}
                    for k, v in per_kernel.items()}
    achieved = gbps(dom_bytes, dom_ms)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "peak_source": peak_src,
                "kernel": "layer-0 forward aggregation (gather fused)" if cfg.fuse_gather else "layer-0 forward aggregation",
                "launches": dom_n, "avg_launch_ms": dom_ms / max(dom_n, 1),
                "algorithmic_bytes_per_launch": dom_bytes / max(dom_n, 1), "per_call": per_call}
    all_agg = {"bound": "hbm", "achieved": gbps(all_bytes, all_ms), "peak": peak, "unit": "GB/s",
               "frac": gbps(all_bytes, all_ms) / peak, "launches": all_n,
               "what": "every aggregation launch (forward and backward) of one region of K steps that follows the timed regions, "
                       "with every launch bracketed by events"}
    return roofline, all_agg


def sharded_gather_report(tk, graph, cfg, primary, rank, world):
    """Rows of one sampled batch that the staging gather of this rank reads from other GPUs, against the NVLink
    ingress of one GPU.  One batch drawn here (outside the timed regions) stands for the step: the input block of a
    Papers-shaped batch has several hundred thousand distinct sources."""
    import torch
    from neutronbench_b200 import Sampler
    shards = tk.datum.shards
    if shards is None:
        return None
    ids = np.arange(cfg.batch_size, dtype=np.uint32) * max(1, graph.global_vertices // cfg.batch_size) + rank
    smp = Sampler(graph, ids, cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed + 1, with_edge_weights=False)
    blk = smp.sample_one().sampled_sgs[0]
    src = blk.src().to(torch.int64)
    owner = src // int(shards.shard_rows)
    rows = int(src.numel())
    remote = int((owner != rank).sum().item())
    row_bytes = int(cfg.layers[0]) * 4
    ph = primary["phase_ms_per_step"] or {}
    gather_ms = ph.get("trans") or 0.0          # device time of one batch's staging gather (its own stream)
    step_ms = primary["ms_per_step"]
    out = {"rows_per_batch": rows, "remote_rows_per_batch": remote, "remote_fraction": remote / max(rows, 1),
           "remote_bytes_per_batch": remote * row_bytes, "gather_ms_per_batch": gather_ms,
           "batches_in_flight": int(cfg.pipelines),
           "remote_GBps_sustained": remote * row_bytes / (step_ms * 1e-3) / 1e9 if step_ms > 0 else 0.0,
           "remote_GBps_inside_one_gather": remote * row_bytes / (gather_ms * 1e-3) / 1e9 if gather_ms > 0 else 0.0,
           "nvlink_ingress_GBps": {"measured_peer_copy": 770.0, "nominal": 900.0},
           "what": "rank 0's figures; sustained = remote bytes of a batch / step time (what the link has to carry), "
                   "inside one gather = the same bytes / that gather's own device time while up to batches_in_flight "
                   "gathers and the training kernels share the GPU"}
    return out


# ------------------------------------------------------------------------------------------ full-graph workload
def bench_cora(args, device):
    """--workload cora: the full-graph GCN (configuration of the reference's CPU-runnable case: 2,708 vertices, 13,264
    edges with self loops, 1433-16-7, 200 epochs) through GCN_GPU_impl / ForwardSingleGPUfuseOp.  A step is one epoch
    (forward, masked loss, backward, Adam over the whole graph); aggregated edges per step = 2 forward + 1 backward
    aggregation over all edges.  The CPU baseline is the C oracle port of the same epoch (kind "port": the reference's
    GCN_CPU toolkit loads its graph through the distributed engine and is not built here)."""
    import torch
    from neutronbench_b200 import (FullyRepGraph, GCN_GPU_impl, GCNConfig, GNNDatum, PartitionedGraph, Workspace, _lib,
                                   synth)
    V, F, C, hidden = 2708, 1433, 7, 16
    edges = synth.uniform_undirected_numpy(V, 5278, args.seed)
    rng = np.random.RandomState(args.seed + 1)
    feat = (rng.random_sample((V, F)) < 0.013).astype(np.float32)
    label = rng.randint(0, C, size=V).astype(np.int64)
    mask = synth.split_mask(V, args.seed)
    cfg = GCNConfig(layers=[F, hidden, C], fanout=(-1, -1), batch_size=V, drop_rate=0.5, learn_rate=0.01,
                    weight_decay=0.0005, seed=args.seed)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(device), V, Workspace(64 << 20))
    pg = PartitionedGraph(g, Workspace(64 << 20))
    tk = GCN_GPU_impl(pg, GNNDatum(torch.from_numpy(feat).to(device), torch.from_numpy(label).to(device), mask), cfg)
    K = args.steps if args.steps > 0 else 200
    W = max(args.warmup, 3)
    for _ in range(W):
        tk.epoch(train=True)
    torch.cuda.synchronize()
    clocks = ClockSampler(0)
    clocks.start()

    def region(read_back):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        for _ in range(K):
            tk.epoch(train=True)
            if read_back:
                tk.read_stats()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1)

    def median_region(read_back):
        first = region(read_back)
        n = min(args.max_regions, max(1, math.ceil(args.min_region_s * 1e3 / max(first, 1e-3))))
        ms = sorted([first] + [region(read_back) for _ in range(n - 1)])
        return ms[(len(ms) - 1) // 2], len(ms)

    launches0 = _lib.load().nb_launch_count()
    ms_a, regions = median_region(False)
    launches = (_lib.load().nb_launch_count() - launches0) / regions
    ms_b, regions_b = median_region(True)
    clk = clocks.stop()
    edges_per_step = 3 * pg.edges
    # the layer-0 aggregation alone, for the roofline figure
    y = torch.empty((V, F), device=device)
    x = tk.datum.local_feature
    stream = torch.cuda.current_stream().cuda_stream
    from neutronbench_b200.cuda_stream import ptr
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 200
    e0.record()
    for _ in range(reps):
        _lib.call("nb_spmm_csc_fwd_fused", ptr(x), ptr(y), ptr(pg.row_indices), ptr(pg.column_offset), ptr(pg.src_norm),
                  ptr(pg.dst_norm), V, F, stream)
    e1.record()
    torch.cuda.synchronize()
    agg_ms = e0.elapsed_time(e1) / reps
    agg_bytes = 4 * F * (V + V) + 4 * pg.edges + 4 * (V + 1) + 4 * (V + V)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else FALLBACK_HBM_GBS
    achieved = agg_bytes / (agg_ms * 1e-3) / 1e9
    line = {"metric": "aggregated_edges_per_s", "value": edges_per_step * K / (ms_a * 1e-3), "unit": "edges/s", "n_gpus": 1,
            "steps": K, "warmup": W, "ms_per_step": ms_a / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"cora-shaped full graph: {V} nodes, {pg.edges} edges (incl. self loops), layers "
                                   f"{F}-{hidden}-{C}, one step = one full-graph epoch",
                       "l2_policy": "none: the whole working set of this workload (about 31 MB) is smaller than L2, on every "
                                    "implementation", "parallelism": "dp1"},
            "epoch_time_s": ms_a / K / 1e3, "regions": regions,
            "e2e": {"value": edges_per_step * K / (ms_b * 1e-3), "unit": "edges/s", "ms_per_step": ms_b / K,
                    "regions": regions_b, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 16},
            "gpu_launches": int(round(launches)),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "kernel": "layer-0 aggregation of the full graph (F = 1433), L2-resident",
                         "avg_launch_ms": agg_ms, "algorithmic_bytes_per_launch": agg_bytes},
            "clocks": clk}
    if not args.no_cpu_baseline:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle
        co64, ri = oracle.build_csc(edges, V)
        co = co64.astype(np.uint32)
        ro, ci = oracle.csr_from_csc(co, ri, V)
        out_d, in_d = oracle.degrees(edges, V, clamp=True)
        s_out, s_in = np.sqrt(out_d.astype(np.float64)).astype(np.float32), np.sqrt(in_d.astype(np.float64)).astype(np.float32)
        wf = np.float32(1) / (s_out[ri] * s_in[np.repeat(np.arange(V), np.diff(co.astype(np.int64)))])
        wb = np.float32(1) / (s_out[np.repeat(np.arange(V), np.diff(ro.astype(np.int64)))] * s_in[ci])
        Wt = tk.P.W.cpu().numpy().copy()
        M, Vv, grad = np.zeros_like(Wt), np.zeros_like(Wt), np.zeros_like(Wt)
        o = tk.P.offsets
        train = np.nonzero(mask == 0)[0]
        times = []
        for ep in range(1 + max(1, args.cpu_batches)):
            t0 = time.perf_counter()
            w0, w1 = Wt[o[0]:o[1]].reshape(F, hidden), Wt[o[1]:o[2]].reshape(hidden, C)
            y0 = oracle.spmm_fwd(feat, wf, ri, co)
            x1 = oracle.relu_dropout(y0 @ w0, 0.5, args.seed, 0, ep)
            y1 = oracle.spmm_fwd(x1, wf, ri, co)
            z = y1 @ w1
            _, dzt, _ = oracle.softmax_nll(z[train], label[train])
            dz = np.zeros_like(z)
            dz[train] = dzt
            grad[o[1]:o[2]] = (y1.T @ dz).reshape(-1)
            dx1 = oracle.spmm_bwd(dz @ w1.T, wb, ro, ci, act=x1, scale=2.0)
            grad[o[0]:o[1]] = (y0.T @ dx1).reshape(-1)
            oracle.adam(Wt, grad, M, Vv, 0.01, 0.9, 0.999, 1e-9, 0.0005, 0.9, 0.999)
            if ep > 0:
                times.append(time.perf_counter() - t0)
        ms = 1e3 * sum(times) / len(times)
        line["cpu_baseline"] = {"value": edges_per_step / (ms * 1e-3), "unit": "edges/s", "cores": oracle.lib().orc_num_threads(),
                                "kind": "port", "ms_per_step": ms,
                                "sample": f"{len(times)} full-graph epochs after 1 warm-up: C oracle port (OpenMP aggregation, "
                                          f"numpy BLAS dense layers) on the host cores"}
    print(json.dumps(line))
    return 0


def main():
    args = parse_args()
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return 0
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1 and args.impl != "reference":
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"   # keep NCCL's version banner off stdout: one JSON line only
        # The only collective is a 329 KB gradient sum per step: a few channels carry it, and every channel is a CTA
        # that holds an SM beside the one-CTA-per-SM aggregation kernel (which leaves that many SMs free).
        os.environ.setdefault("NCCL_MAX_CTAS", "4")
        # NCCL launches its CTAs as one thread-block cluster by default, and a cluster needs free SMs that sit
        # together.  The SMs the aggregation kernel leaves free are wherever the scheduler put its CTAs, so the
        # gradient sum of step i would wait for the layer-0 aggregation of step i+1 to end instead of running beside
        # it (measured on 4 GPUs: 0.241 against 0.213 ms per step).  Independent CTAs fit the free SMs.
        os.environ.setdefault("NCCL_CGA_CLUSTER_SIZE", "1")
        dist.init_process_group("nccl", device_id=device)

    from neutronbench_b200 import GCN_GPU_NEIGHBOR_impl, _lib
    if args.pdl is not None:
        _lib.load().nb_set_pdl(int(args.pdl))
    if args.workload == "cora":
        if rank != 0:
            return 0
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference's full-graph CPU toolkit (GCN_CPU) loads its "
                              "graph through the distributed engine, which is not built here; --workload cora reports the C "
                              "oracle port as cpu_baseline"}))
            return 0
        return bench_cora(args, device)
    if args.workload == "papers" and args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the Papers-shaped feature table (57 GB) is a multi-GPU "
                          "scale test; the reference's CPU path is timed on the other workloads"}))
        return 0
    sh, cfg, graph, datum, train_ids, feat_dev = build_workload(args.workload, args, device, rank, world)
    batches_per_epoch = (len(train_ids) + cfg.batch_size - 1) // cfg.batch_size

    def describe(sh, cfg, graph, pipelines, train_ids):
        return {
            "workload": f"{sh.name}-shaped synthetic R-MAT: {sh.vertices} nodes, {graph.global_edges} edges (incl. self "
                        f"loops), feature {sh.feature}, layers {'-'.join(map(str, cfg.layers))}, fanout "
                        f"{list(cfg.fanout)} (hop order), batch {cfg.batch_size}, cache_rate {cfg.cache_rate}",
            "batches_per_epoch": (len(train_ids) + cfg.batch_size - 1) // cfg.batch_size,
            "l2_policy": "inputs larger than L2 (feature store >> 126 MB, each step touches a new random subset)",
            "parallelism": f"dp{world}",
            "fuse_gather": cfg.fuse_gather,
            "step": "python (one call per kernel family)" if args.python_step else
                    ("native (nb_gcn_sample on library threads overlapping nb_gcn_compute)" if pipelines > 1
                     else "native (nb_gcn_step)"),
            "pipelines": pipelines,
            "settle_s": args.settle_s,
            "timed_region": ("seeds resident on the device; every step's loss is read back one step late"
                             if args.value_readback else "seeds resident on the device; nothing is read back"),
            "gradient_sum": "none (one rank)" if world == 1 else
                            ("libnb_b200_comm (NCCL) on the update stream"
                             if os.environ.get("NB_NATIVE_ALLREDUCE", "1") == "1" else "torch.distributed (NCCL)"),
        }

    if args.pipelines <= 0:
        args.pipelines = 4 if (os.cpu_count() or 1) >= 4 * world else 3
    pipelines = 1 if args.python_step else max(1, args.pipelines)
    workload_desc = describe(sh, cfg, graph, pipelines, train_ids)

    if args.impl == "reference":
        K = args.steps if args.steps > 0 else 3
        W = max(args.warmup, 0)
        base = host_baseline(sh, cfg, graph, feat_dev, datum.local_label, train_ids, K, W, args.seed)
        eps, ms = base["value"], base["ms_per_step"]
        line = {"impl": "reference", "metric": "aggregated_edges_per_s", "value": eps, "unit": "edges/s",
                "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_desc,
                "epoch_time_s": ms * batches_per_epoch / 1e3, "cpu_baseline": base,
                "e2e": {"value": eps, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    def make_trainer(graph, datum, cfg):
        cfg.pipelines = pipelines
        tk = GCN_GPU_NEIGHBOR_impl(graph, datum, cfg, rank=rank, world_size=world, use_engine=not args.python_step)
        tk.init_cache()
        # fewer cores than threads that would spin (a main thread, an NCCL proxy and the sampler threads per rank): the
        # sampling half then waits for the GPU on blocking events
        if not args.python_step and os.environ.get("NB_BLOCKING_SYNC_AUTO", "0") == "1" and \
                (os.cpu_count() or 1) < world * (pipelines + 2):
            _lib.call("nb_gcn_set_option", tk._ensure_engine(), b"blocking_sync", 1)
        for opt in args.option:
            name, value = opt.split("=", 1)
            _lib.call("nb_gcn_set_option", tk._ensure_engine(), name.encode(), int(value))
        return tk

    tk = make_trainer(graph, datum, cfg)
    del feat_dev
    W = max(args.warmup, 3)
    K, a, b = measure(tk, graph, cfg, train_ids, args, args.steps, W, rank, world, local_rank, device)

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak = float(json.load(open(peaks_path))["hbm_gbs"])
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    traffic = ncu_traffic_bytes(args.workload, cfg.fuse_gather, cfg.cache_rate >= 1.0)
    roofline, all_agg = roofline_of(a["events"], peak, peak_src, traffic, cfg)

    def summary(K, a, b, cfg, bpe):
        hops = len(cfg.fanout)
        steps_per_epoch = (bpe + world - 1) // world
        return {
            "value": a["edges"] / (a["ms"] * 1e-3), "ms_per_step": a["ms"] / K,
            "epoch_time_s": (a["ms"] / K) * steps_per_epoch / 1e3,
            "regions": a["regions"], "region_ms": {"median": a["ms"], "min": a["ms_min"], "max": a["ms_max"]},
            "e2e": {"value": b["edges"] / (b["ms"] * 1e-3), "unit": "edges/s", "ms_per_step": b["ms"] / K,
                    "epoch_time_s": (b["ms"] / K) * steps_per_epoch / 1e3, "regions": b["regions"],
                    "h2d_bytes_per_step": cfg.batch_size * 4, "d2h_bytes_per_step": 8 + hops * 12},
            "gpu_launches": int(round(a["launches_per_region"])),
            "phase_ms_per_step": a["phase_ms_per_step"],
            "aggregated_edges_per_step": a["edges"] / (K * world),
        }

    primary = summary(K, a, b, cfg, batches_per_epoch)
    stage_primary = bool(tk.stage_misses)

    # ---- the reference's CPU path on the same workload, on this box's host cores (rank 0 of a 1-GPU run only)
    base = None
    if rank == 0 and not args.no_cpu_baseline and world == 1 and args.workload != "papers":
        base = host_baseline(sh, cfg, graph, datum.local_feature, datum.local_label, train_ids, args.cpu_batches, 1,
                             args.seed)
        base["epoch_time_s"] = base["ms_per_step"] * batches_per_epoch / 1e3

    # ---- secondary: the Products-shaped workload at this N (its scaling is a target of its own)
    secondary = None
    if not args.no_secondary and args.workload == "reddit" and args.scale == 1.0:
        del tk, datum, graph
        torch.cuda.empty_cache()
        sh2, cfg2, graph2, datum2, train2, feat2 = build_workload("products", args, device, rank, world)
        del feat2
        tk2 = make_trainer(graph2, datum2, cfg2)
        K2, a2, b2 = measure(tk2, graph2, cfg2, train2, args, args.secondary_steps, W, rank, world, local_rank, device)
        bpe2 = (len(train2) + cfg2.batch_size - 1) // cfg2.batch_size
        secondary = summary(K2, a2, b2, cfg2, bpe2)
        r2, all2 = roofline_of(a2["events"], peak, peak_src, None, cfg2)
        secondary.update({"metric": "aggregated_edges_per_s", "unit": "edges/s", "n_gpus": world, "steps": K2, "warmup": W,
                          "config": describe(sh2, cfg2, graph2, pipelines, train2), "stage_misses": bool(tk2.stage_misses),
                          "layer0_aggregation": {k: r2[k] for k in ("achieved", "frac", "avg_launch_ms",
                                                                    "algorithmic_bytes_per_launch")},
                          "all_aggregation": {k: all2[k] for k in ("achieved", "frac", "launches")}})

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    line = {
        "metric": "aggregated_edges_per_s", "value": primary["value"], "unit": "edges/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": primary["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_desc,
        "epoch_time_s": primary["epoch_time_s"], "regions": primary["regions"], "region_ms": primary["region_ms"],
        "e2e": primary["e2e"], "gpu_launches": primary["gpu_launches"], "roofline": roofline,
        "all_aggregation": all_agg, "clocks": a["clocks"],
        "aggregated_edges_per_step": primary["aggregated_edges_per_step"], "device_error": 0,
        "phase_ms_per_step": primary["phase_ms_per_step"],
        "stage_misses": stage_primary,
    }
    if args.workload == "papers":
        line["config"]["feature_table"] = f"sharded by node-id range over {world} GPUs, peers read with plain loads"
        try:
            line["sharded_gather"] = sharded_gather_report(tk, graph, cfg, primary, rank, world)
        except Exception as exc:   # a reporting aid: never loses the measured line
            line["sharded_gather"] = {"unavailable": repr(exc)}
    if secondary is not None:
        line["secondary"] = secondary
    if base is not None:
        line["cpu_baseline"] = base
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

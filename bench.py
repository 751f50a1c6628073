#!/usr/bin/env python
"""Benchmark of the MGG hot path on B200: 2-layer GCN forward on the Reddit-shaped synthetic graph.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config cfg2|cfg1|cfg3|cfg4]

One "step" is one forward pass (dense 602->16, two neighbor aggregations at width 16, dense 16->41,
softmax) over the whole graph, sharded by node range over N GPUs (one process per GPU; torchrun for
N > 1).  The metric is aggregated edges per second: (aggregations per pass x stored edges) / pass time.
Prints ONE JSON line on rank 0.

--impl reference times the reference's own CPU implementation of the aggregation (SAG_ref compiled
from the reference's sources when that binary is present, else the plain-C port), with the dense /
softmax steps done by the CPU oracle, on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes (read + write) of one aggregation launch from the ncu capture summarised in
# profiles/cfg2_gcn2_1gpu_aggregation_and_dense.txt; only that case has been captured.
NCU_TRAFFIC_BYTES = {("cfg2", 1, 1.0): 494.4e6}
NVLINK_GBS = 900.0          # per direction per GPU (nominal); 770 GB/s measured peer copy on this pool
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"])
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the graph (quick checks only; not a bench value)")
    ap.add_argument("--ps", type=int, default=None)
    ap.add_argument("--wpb", type=int, default=None)
    ap.add_argument("--dist", type=int, default=None)
    ap.add_argument("--fetch", default="auto", choices=["auto", "peer", "replica"],
                    help="how peers see a layer's output: 'peer' = rows pulled from the owner inside the aggregation "
                         "kernel; 'replica' = rows pushed into every PE's copy by the producing kernel; 'auto' = replica "
                         "when there are peers and the copy fits")
    ap.add_argument("--cpu-threads", type=int, default=0,
                    help="host threads of the CPU arm (--impl reference and cpu_baseline); 0 = all the cores this process may use, "
                         "1 = the reference's host aggregation exactly as written (one thread)")
    ap.add_argument("--overlap-blocks", type=int, default=-1,
                    help="row blocks per pushed aggregation (block b is pushed to the peers while block b+1 is gathered); "
                         "1 = no overlap, default = the driver's choice")
    ap.add_argument("--keep-logits", action="store_true",
                    help="also store the last dense layer's output (the fused dense+softmax kernel writes only the probabilities by default)")
    ap.add_argument("--row-order", default="auto", choices=["auto", "degree", "natural"],
                    help="block schedule of the aggregation: rows by decreasing degree, or in id order (auto: the driver's default)")
    ap.add_argument("--group-per-node", action="store_true", help="aggregate with 4 lanes per node (MGGB_AGG_GROUP_PER_NODE); default for cfg4 and cfg5")
    ap.add_argument("--no-group-per-node", action="store_true")
    ap.add_argument("--dense", default="auto", choices=["auto", "simt"],
                    help="'simt' forces the CUDA-core dense kernel (A/B against the tensor-core one)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


CONFIGS = {
    # name: (model, in_dim, hidden, out_dim, default knobs (ps, wpb, dist), description)
    "cfg1": ("agg", 16, 16, 16, (32, 4, 1), "R-MAT 16,384 nodes, one sym-normalised aggregation, dim 16"),
    "cfg2": ("gcn2", 602, 16, 41, (32, 4, 2), "Reddit-shaped power-law graph 232,965 nodes ~114.6M edges, GCN-2 602-16-41"),
    "cfg3": ("gin5", 100, 64, 47, (16, 1, 2), "products-shaped power-law graph 2,449,029 nodes ~123.7M edges, GIN-5 hidden 64"),
    "cfg4": ("agg", 16, 16, 16, (32, 1, 1), "skewed directed R-MAT 4,206,785 nodes ~101.3M edges, one aggregation dim 16"),
    "cfg5": ("gcn2", 128, 16, 172, (32, 1, 1), "symmetric R-MAT 111M nodes ~3.2B edges built shard-locally (64-bit row pointers), GCN-2 128-16-172"),
}


def make_graph(cfg: str, device, scale: float):
    from mgg_osdi23_b200 import graphgen as gg
    if cfg == "cfg1":
        return gg.config1_graph(device=device)
    if cfg == "cfg2":
        return gg.config2_graph(device=device, scale=scale)
    if cfg == "cfg3":
        return gg.config3_graph(device=device, scale=scale)
    shift = 0
    while scale < 1.0 and (1 << shift) * scale < 1.0:
        shift += 1
    return gg.config4_graph(device=device, scale_shift=shift)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons WHILE the timed region runs.

    NVML is polled from a thread every few milliseconds (a timed region lasts tens of milliseconds,
    too short for nvidia-smi's own loop); where the NVML binding is missing it falls back to an
    ``nvidia-smi -lms`` child process.  Read-only: no clock or power setting is touched."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, cuda_index: int):
        self.cuda_index, self.proc, self.lines = cuda_index, None, []
        self.sm, self.mask, self.max_mhz, self.handle, self.nvml = [], 0, None, None, None
        self._stop = threading.Event()
        self.thread = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        self.nvml = pynvml
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(self.cuda_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(visible.split(",")[self.cuda_index]) if visible and visible.split(",")[self.cuda_index].isdigit() else self.cuda_index
            return pynvml.nvmlDeviceGetHandleByIndex(idx)

    def _poll(self):
        n = self.nvml
        while not self._stop.is_set():
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                try:
                    self.mask |= int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    self.mask |= int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
            except Exception:
                break
            time.sleep(0.004)

    def start(self):
        try:
            self.handle = self._nvml_handle()
            self.max_mhz = float(self.nvml.nvmlDeviceGetMaxClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.handle = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.cuda_index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.handle is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            if not self.sm:
                return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"], "source": "nvml"}
            sm = sorted(self.sm)
            reasons = sorted(name for bit, name in self.REASONS.items() if self.mask & bit)
            return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                    "samples": len(sm), "source": "nvml, 4 ms period, during the timed region"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["neither NVML nor nvidia-smi available"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "source": "nvidia-smi"}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvidia-smi -lms 200"}


# -------------------------------------------------------------------------------------------------
# CPU arm: the reference's host aggregation (or the port) + oracle dense/softmax
# -------------------------------------------------------------------------------------------------

def cpu_forward_factory(cfg_name, g_cpu, x_np, weights_np, norm, threads=0):
    """Returns (step_fn, description dict).  step_fn() runs one forward pass on the host with
    ``threads`` host threads (0 = every core this process may use)."""
    import numpy as np
    from oracle.oracle import Oracle, Ref
    orc = Oracle()
    use_ref = Ref.available()
    ref = Ref() if use_ref else None
    if threads <= 0:
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        if g_cpu.num_edges < (1 << 21):     # a few milliseconds of work: handing out ranges costs more than it saves
            threads = 1
    rp = g_cpu.row_ptr.numpy().astype(np.int32)
    col = g_cpu.col_idx.numpy()
    model = CONFIGS[cfg_name][0]
    dinv = orc.inv_sqrt_degree(rp) if norm == "sym" else None

    def sag(t):
        if use_ref:
            return ref.sag_ref(t, rp, col, threads=threads)
        return orc.sag_omp(t, rp, col)[0] if threads > 1 else orc.sag_f32(t, rp, col)

    def agg(t):
        if dinv is None:
            return sag(t)
        return orc.row_scale(sag(orc.row_scale(t, dinv)), dinv)

    def step():
        if model == "agg":
            return agg(x_np)
        if model == "gcn2":
            h = orc.dense(x_np, weights_np[0])
            z = agg(agg(h))
            return orc.softmax(orc.dense(z, weights_np[1]))
        h = orc.dense(x_np, weights_np[0])
        for k in range(5):
            h = orc.dense(sag(h) + h, weights_np[k + 1])
        return orc.softmax(h)

    desc = {"kind": "reference" if use_ref else "port", "cores": threads,
            "sample": ("whole workload, full forward pass per step: aggregations by "
                       + (f"SAG_ref compiled from the reference's include/utils.cuh, called from {threads} threads on disjoint node ranges "
                          "(the function itself is one loop over the nodes; row sums are the same bits)" if use_ref
                          else f"the plain-C port of SAG_ref ({'OpenMP over rows' if threads > 1 else 'single thread'})")
                       + "; dense/softmax by the CPU oracle (OpenMP, not reference code)")}
    return step, desc


def run_reference(args, rank, world):
    import numpy as np
    import torch
    if rank != 0:
        return
    # torch.distributed.run hands every rank OMP_NUM_THREADS=1; rank 0 runs this arm alone
    if world > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    if args.config == "cfg5":
        print(json.dumps({"impl": "reference", "unavailable": "config 5 is never materialised as one graph (built shard by shard); the host reference needs the whole CSR"}), flush=True)
        return
    from mgg_osdi23_b200 import graphgen as gg
    model, din, hid, dout, _, desc = CONFIGS[args.config]
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = make_graph(args.config, dev, args.scale).cpu()
    x = gg.features(g.num_nodes, din, seed=1).numpy()
    weights = build_weights(args.config, "cpu")
    norm = "sym" if model in ("gcn2",) or args.config == "cfg1" else "none"
    step, d = cpu_forward_factory(args.config, g, x, [w.numpy() for w in weights], norm, args.cpu_threads)
    naggs = {"agg": 1, "gcn2": 2, "gin5": 5}[model]
    # bound the run: the driver's K and W are honoured up to ~150 s of CPU work
    t0 = time.perf_counter(); step(); one = time.perf_counter() - t0
    steps = max(1, min(args.steps, int(120.0 / max(one, 1e-3))))
    warm = max(0, min(args.warmup, int(30.0 / max(one, 1e-3))) - 1)
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    value = naggs * g.num_edges / dt
    d["value"] = value
    d["unit"] = "edges/s"
    line = {
        "impl": "reference", "metric": metric_name(model), "value": value, "unit": "edges/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm + 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, g, model, din, hid, dout, None, 1),
        "cpu_baseline": d,
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(model):
    return {"gcn2": "gcn2_fwd_aggregated_edges_per_s", "gin5": "gin5_fwd_aggregated_edges_per_s",
            "agg": "aggregation_edges_per_s"}[model]


def workload_config(args, g, model, din, hid, dout, knobs, world):
    c = {"workload": f"{args.config}: {CONFIGS[args.config][5]}", "nodes": g.num_nodes, "edges": g.num_edges,
         "in_dim": din, "aggregated_width": hid, "classes": dout, "graph": g.meta,
         "partition": f"node-range x{world}", "l2_policy": "inputs larger than L2 (features 561 MB, neighbor ids 458 MB per aggregation)"
         if args.config == "cfg2" else "inputs larger than L2 where the graph is (see edges x 4 B of neighbor ids per aggregation)"}
    if knobs is not None:
        c.update({"ps": knobs.partSize, "wpb": knobs.warpPerBlock, "dist": knobs.interleaved_dist, "group_per_node": bool(knobs.flags & 4)})
    if args.scale != 1.0:
        c["scale"] = args.scale
    return c


def build_weights(cfg, device):
    from mgg_osdi23_b200 import graphgen as gg
    model, din, hid, dout, _, _ = CONFIGS[cfg]
    if model == "gcn2":
        return [gg.glorot_uniform(din, hid, 1, device), gg.glorot_uniform(hid, dout, 2, device)]
    if model == "gin5":
        # scaled down so that five unnormalised sum-aggregations stay finite in fp32
        return ([gg.glorot_uniform(din, hid, 10, device) * 0.05] + [gg.glorot_uniform(hid, hid, 11 + k, device) * 0.05 for k in range(4)]
                + [gg.glorot_uniform(hid, dout, 20, device) * 0.05])
    return []


# -------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------

def run_ours(args, rank, world, local_rank):
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # only a one-element all-reduce goes through NCCL
    # torch.distributed.run gives every rank OMP_NUM_THREADS=1 unless the user chose a value; the host
    # partitioner (split_CSR) is OpenMP code, so share the host cores among the ranks instead.  Must be
    # set before the library is loaded.
    if world > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
        os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // world))
    import numpy as np
    import torch
    import torch.distributed as dist
    from mgg_osdi23_b200 import api, drivers, graphgen as gg
    from mgg_osdi23_b200.symmem import SymmetricBuffer, ReplicaBuffer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl ours needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model_kind, din, hid, dout, dknobs, desc = CONFIGS[args.config]
    group_kernel = (args.group_per_node or args.config in ("cfg4", "cfg5")) and not args.no_group_per_node
    knobs = drivers.Knobs(args.ps or dknobs[0], args.wpb or dknobs[1], args.dist or dknobs[2], flags=4 if group_kernel else 0)

    shard_local = args.config == "cfg5"          # too large to replicate: every rank builds only its rows
    if shard_local:
        shift = 0
        while args.scale < 1.0 and (1 << shift) * args.scale < 1.0:
            shift += 1
        g = gg.config5_shard(rank, world, device=dev, scale_shift=shift)
    else:
        g = make_graph(args.config, dev, args.scale)
    n = g.num_nodes
    rp_host, col_host = g.row_ptr.cpu().numpy(), g.col_idx.cpu().numpy()
    t0 = time.perf_counter()
    shard = drivers.Shard(rp_host, col_host, rank, world, device=dev, num_nodes=n, shard_local=shard_local,
                          order_rows={"auto": None, "degree": True, "natural": False}[args.row_order])
    preproc_ms = (time.perf_counter() - t0) * 1e3
    g_meta, g_edges = g.meta, g.num_edges
    if shard_local and world > 1:                 # stored edges of the whole graph = sum over the shards
        t = torch.tensor([g_edges], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        g_edges = int(t.item())
    del g
    torch.cuda.empty_cache()

    npp = shard.node_per_pe
    fetch = args.fetch
    if fetch == "auto":
        fetch = "replica" if world > 1 and world * npp * hid * 4 < (8 << 30) else "peer"
    if fetch == "replica":
        sym_a = ReplicaBuffer(npp, hid, group, rank, world)
        sym_b = ReplicaBuffer(npp, hid, group, rank, world)
    else:
        sym_a = SymmetricBuffer(npp * hid, group, rank, world)
        sym_b = SymmetricBuffer(npp * hid, group, rank, world)
    weights = build_weights(args.config, dev)
    norm = "sym" if model_kind == "gcn2" or args.config == "cfg1" else "none"
    if model_kind == "gcn2":
        model = drivers.GCN2Forward(shard, din, hid, dout, sym_a, sym_b, knobs, w1=weights[0], w2=weights[1], norm=norm,
                                    dense_flags=4 if args.dense == "simt" else 0)
    elif model_kind == "gin5":
        model = drivers.GIN5Forward(shard, din, hid, dout, sym_a, sym_b, knobs, eps=0.0, weights=weights,
                                    dense_flags=4 if args.dense == "simt" else 0)
    else:
        model = drivers.SingleAggregation(shard, hid, sym_a, knobs, norm=norm)
    model.keep_logits = args.keep_logits
    if args.overlap_blocks >= 1:
        model.overlap_blocks = args.overlap_blocks
    x_dev = gg.features(shard.rows, din, seed=1, device=dev, first_row=shard.lb)
    if model_kind == "agg" and norm == "sym":
        x_dev = x_dev * shard.inv_sqrt_degree()[:, None]
    x_host = torch.empty(x_dev.shape, dtype=torch.float32, pin_memory=True)
    x_host.copy_(x_dev)
    model.d_in.copy_(x_dev)
    del x_dev
    barrier = drivers.nccl_stream_barrier(group) if world > 1 else None

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- device-resident timing ---------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        model.forward(barrier)
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    agg_events = []
    shard.event_sink = agg_events
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    launches0 = api.kernel_launches[0]
    e0.record()
    for _ in range(args.steps):
        model.forward(barrier)
    e1.record()
    sync_all()
    shard.event_sink = None
    # kernels of all ranks in the timed region (a collective: every rank calls it, here)
    launches = int(sum_over_ranks(api.kernel_launches[0] - launches0))
    step_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    agg_ms_local = sum(a.elapsed_time(b) for a, b in agg_events) / max(1, len(agg_events))
    agg_ms = max_over_ranks(agg_ms_local)
    nsite = model.aggregations_per_forward
    agg_ms_by_site = [max_over_ranks(sum(a.elapsed_time(b) for a, b in agg_events[s::nsite]) / max(1, len(agg_events[s::nsite])))
                      for s in range(nsite)]
    clocks = sampler.stop() if rank == 0 else None

    # ---- where the time of a pass goes (a few extra passes, outside the timed region) ---------------
    marks = []
    for _ in range(5):
        model.forward(barrier, marks)
    sync_all()
    spans = len(marks[0]) - 1
    breakdown = [max_over_ranks(sum(m[i].elapsed_time(m[i + 1]) for m in marks) / len(marks)) for i in range(spans)]

    # ---- end to end through the host-buffer entry point ---------------------------------------
    e2e = None
    if not args.no_e2e:
        for _ in range(2):
            model.forward_host(x_host, barrier)
        sync_all()
        e_steps = max(3, min(args.steps, 10))
        e0.record()
        for _ in range(e_steps):
            model.forward_host(x_host, barrier)
        e1.record()
        sync_all()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e_steps)
    naggs = model.aggregations_per_forward
    total_edges = g_edges
    value = naggs * total_edges / (step_ms * 1e-3)

    # per-rank edge split, gathered for the roofline
    stats = torch.tensor([shard.e_local, shard.e_remote, shard.rows], dtype=torch.int64, device=dev)
    if world > 1:
        allstats = [torch.zeros_like(stats) for _ in range(world)]
        dist.all_gather(allstats, stats)
    else:
        allstats = [stats]
    allstats = [s.tolist() for s in allstats]

    if rank == 0:
        hbm, hbm_src = measured_peaks()
        D = hid
        t_roof = max(max(4.0 * D * el / (hbm * 1e9), 4.0 * D * er / (NVLINK_GBS * 1e9)) for el, er, _ in allstats)
        alg_bytes = max(4.0 * D * (el + er) for el, er, _ in allstats)       # per launch, busiest GPU
        achieved = alg_bytes / (agg_ms * 1e-3) / 1e9
        line = {
            "metric": metric_name(model_kind), "value": value, "unit": "edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, type("G", (), {"num_nodes": n, "num_edges": total_edges, "meta": g_meta})(),
                                      model_kind, din, hid, dout, knobs, world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                         "traffic": NCU_TRAFFIC_BYTES.get((args.config, world, args.scale)), "peak_source": f"of {hbm_src}", "kernel": "sag_np_div_kernel",
                         "algorithmic_bytes_per_launch": alg_bytes, "kernel_ms": agg_ms, "kernel_ms_by_call_site": agg_ms_by_site,
                         "aggregation_roofline_ms": t_roof * 1e3, "aggregation_roofline_frac": t_roof * 1e3 / agg_ms,
                         "nvlink_gbs_assumed": NVLINK_GBS},
            "fetch": fetch, "dense_kernel": "cuda-core" if args.dense == "simt" else "tcgen05 where the shape fits",
            "overlap_blocks": model.overlap_blocks,
            "last_layer": "dense + softmax in one kernel" + (", logits stored too" if args.keep_logits else ", logits not stored"),
            "per_gpu_edges": [{"local": el, "remote": er, "rows": r} for el, er, r in allstats],
            "remote_fraction": sum(er for _, er, _ in allstats) / max(1, total_edges),
            "gpu_launches": launches,
            "pass_breakdown_ms": {"spans": "stage" + (", barrier, stage" * ((spans - 1) // 2) if world > 1 else ", stage" * (spans - 1)),
                                  "ms": breakdown},
            "preproc_ms": preproc_ms, "clocks": clocks,
        }
        if not args.no_e2e:
            h2d = int(n * din * 4)
            d2h = int(n * (dout if model_kind != "agg" else hid) * 4)
            line["e2e"] = {"value": naggs * total_edges / (e2e_ms * 1e-3), "unit": "edges/s", "ms_per_step": e2e_ms,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "note": "pinned host features -> device, forward, probabilities -> pinned host; graph structure resident"}
        if world == 1 and not args.no_cpu_baseline and not shard_local:
            line["cpu_baseline"] = cpu_baseline(args, rp_host, col_host, n, din, weights, norm, naggs, total_edges, g_meta)
        print(json.dumps(line), flush=True)

    sync_all()
    sym_a.close(); sym_b.close()
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(args, rp_host, col_host, n, din, weights, norm, naggs, total_edges, meta):
    """Times the CPU arm on the host cores for a bounded number of passes (about 10-30 s)."""
    import torch
    from mgg_osdi23_b200 import graphgen as gg
    g_cpu = gg.Graph(n, torch.from_numpy(rp_host), torch.from_numpy(col_host), meta)
    x = gg.features(n, din, seed=1).numpy()
    step, d = cpu_forward_factory(args.config, g_cpu, x, [w.cpu().numpy() for w in weights], norm, args.cpu_threads)
    t0 = time.perf_counter(); step(); one = time.perf_counter() - t0
    reps = max(1, min(5, int(15.0 / max(one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        step()
    dt = (time.perf_counter() - t0) / reps
    d["value"] = naggs * total_edges / dt
    d["unit"] = "edges/s"
    d["ms_per_step"] = dt * 1e3
    d["sample"] += f"; {reps} timed passes after 1 warm-up"
    return d


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun: python -m torch.distributed.run --nproc-per-node {args.gpus} bench.py ...")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the quantized embedding-bag lookup on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload 0|1|2] [--streams S] [--group G]

One *step* is one functor call (one batch of bags) of the chosen workload.
Prints ONE JSON line:

* ``value``      gathered-row GB/s with every input resident in HBM: the K
                 steps are K separate kernel launches on distinct pre-generated
                 batches, issued from a CUDA graph over S streams.
* ``e2e``        the same metric through the host-pointer C-ABI call
                 (``fbgemm_b200_spmdm_host_submit/wait``): indices, offsets and
                 weights leave pinned host memory and the pooled rows return to
                 the host inside the timed region; only the table is resident.
* ``roofline``   HBM roofline of the lookup kernel on gathered-row bytes.
* ``cpu_baseline`` the reference's CPU path timed on this box's host cores on
                 a bounded sample of the same batches.

``--impl reference`` times only the CPU path (all host threads) and prints the
same line shape with ``"impl": "reference"``.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
GRAPH_CHUNK = 500       # steps per captured graph
NUM_BATCHES = 32        # distinct pre-generated batches the steps rotate over
# DRAM bytes (read + write) per lookup launch, from ncu captures of the same
# launch shape: key = (workload, batches per call).
TRAFFIC_BYTES_PER_LAUNCH = {
    (1, 1): 13_766_144,             # profiles/spmdm_direct_kernel__workload1_one_batch.md
    (1, 16): 171_163_904 + 7_316_992,   # profiles/spmdm_direct_kernel__workload1_16batches.md
    (0, 16): 438_465_024 + 71_525_888,  # profiles/spmdm_direct_kernel__workload0_16batches.md
    (2, 16): 233_486_336 + 49_955_840,  # profiles/spmdm_direct_compact_kernel__workload2_16batches.md
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--warmup", type=int, default=500)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", type=int, default=1, help="which benchmark configuration (0..4): 8-bit, 4-bit (default), pruned 2-bit, 64 mixed tables, 256 large tables")
    ap.add_argument("--streams", type=int, default=16, help="streams the graph spreads the launches over")
    ap.add_argument("--group", type=int, default=1, help="batches concatenated into one call (1 = the config's batch)")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink table rows (and, for workloads 0-2, the batch)")
    ap.add_argument("--tables-scale", type=float, default=1.0, help="workloads 3/4: fraction of the tables")
    ap.add_argument("--batch-scale", type=float, default=1.0, help="workloads 3/4: fraction of the batch")
    ap.add_argument("--launch", default="streams", choices=["plan", "streams"],
                    help="workloads 3/4: one multi-table plan (a launch per kernel variant) or a launch per table")
    ap.add_argument("--redistribution", default="p2p", choices=["p2p", "nccl"],
                    help="workloads 3/4: peer stores from the lookup kernel, or NCCL all-to-all after it")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-pointer leg")
    ap.add_argument("--e2e-steps", type=int, default=2000)
    ap.add_argument("--cpu-seconds", type=float, default=4.0, help="wall-time bound of the CPU sample")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler:
    """Samples SM clock and throttle reasons with NVML while the timed region
    runs (read-only queries)."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        self.period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None

    def _run(self):
        nv = self._nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def concat_batches(batches):
    """Several batches as one call (bags appended, offsets re-based)."""
    import torch

    from fbgemm_b200.workloads import Batch

    idx = torch.cat([b.indices for b in batches])
    offs, base = [batches[0].offsets.to(torch.int64)], int(batches[0].offsets[-1])
    for b in batches[1:]:
        offs.append(b.offsets[1:].to(torch.int64) + base)
        base += int(b.offsets[-1])
    off = torch.cat(offs).to(batches[0].offsets.dtype)
    w = torch.cat([b.weights for b in batches]) if batches[0].weights is not None else None
    return Batch(idx, off, w, sum(b.output_size for b in batches), int(idx.numel()),
                 sum(b.valid_rows for b in batches))


# ---- CPU leg (the reference arm and cpu_baseline) ----------------------------------

def cpu_runner(workload, host_table, host_cit):
    """Returns (call(batch_np) -> ok, kind, description).  Prefers the
    reference's own JIT kernels (bundled in libtorch_cpu.so), then the
    reference's scalar sources, then the oracle port."""
    from oracle import checker

    jit = checker.ReferenceJit()
    ref = checker.Reference()
    if jit.available:
        impl, kind, desc = jit, "reference", "FBGEMM asmjit AVX2/AVX-512 kernels as bundled in libtorch_cpu.so"
    elif ref.available:
        impl, kind, desc = ref, "reference", "FBGEMM scalar EmbeddingSpMDM*_ref compiled from the reference tree"
    else:
        impl, kind, desc = checker.Oracle(), "port", "plain-C oracle port (oracle/embedding_oracle.c)"
    out_dt = np.float16 if str(workload.out_dtype) == "torch.float16" else np.float32

    def call(hb, lo, hi):
        """Bags [lo, hi) of host batch hb, as one functor call on a slice (how
        the reference's callers parallelise: one thread per bag range)."""
        offs = hb["offsets"][lo:hi + 1]
        i0, i1 = int(offs[0]), int(offs[-1])
        idx = hb["indices"][i0:i1]
        wts = hb["weights"][i0:i1] if hb["weights"] is not None else None
        if host_cit is not None:
            ok, _ = impl.spmdm_rowwise_sparse(workload.bit_rate, workload.dim, workload.rows, host_table, idx,
                                              host_cit, offs, wts, workload.normalize_by_lengths)
        else:
            ok, _ = impl.spmdm(workload.bit_rate, workload.dim, workload.rows, host_table, idx, offs, wts,
                               workload.normalize_by_lengths, out_dt)
        return ok

    return call, kind, desc


def time_cpu(workload, batches, host_table, host_cit, threads, max_steps, max_seconds):
    """Run whole batches, each split over `threads` host threads (contiguous
    bag ranges, one functor call each - how the reference's callers and
    benchmarks parallelise this single-threaded kernel), until max_steps
    batches or max_seconds have passed.  Returns (seconds, steps, gathered
    bytes, kind, desc).  With the reference's JIT kernels the split runs on
    OpenMP threads inside the checker library; otherwise on a Python pool."""
    from concurrent.futures import ThreadPoolExecutor

    from fbgemm_b200.workloads import algorithmic_bytes
    from oracle import checker

    call, kind, desc = cpu_runner(workload, host_table, host_cit)
    jit = checker.ReferenceJit()
    out_dt = np.float16 if (str(workload.out_dtype) == "torch.float16" and host_cit is None) else np.float32
    host_batches = []
    for b in batches:
        host_batches.append({
            "indices": b.indices.cpu().numpy(), "offsets": b.offsets.cpu().numpy(),
            "weights": b.weights.cpu().numpy() if b.weights is not None else None,
            "B": b.output_size, "bytes": algorithmic_bytes(workload, b),
            "out": np.zeros(b.output_size * workload.dim, dtype=out_dt)})
    pool = None if jit.available else ThreadPoolExecutor(max_workers=threads)

    def run_batch(hb):
        if jit.available:
            return jit.batch_parallel(workload.bit_rate, workload.dim, workload.rows, host_table, hb["indices"],
                                      hb["offsets"], hb["weights"], workload.normalize_by_lengths, hb["out"], threads,
                                      host_cit)
        B = hb["B"]
        cuts = [B * t // threads for t in range(threads + 1)]
        futs = [pool.submit(call, hb, cuts[t], cuts[t + 1]) for t in range(threads) if cuts[t + 1] > cuts[t]]
        return all(f.result() for f in futs)

    assert run_batch(host_batches[0]), "CPU reference returned false on a valid batch"  # warm-up, JIT generation
    t0 = time.perf_counter()
    steps, nbytes = 0, 0
    while steps < max_steps and (time.perf_counter() - t0) < max_seconds:
        hb = host_batches[steps % len(host_batches)]
        run_batch(hb)
        steps += 1
        nbytes += hb["bytes"]
    dt = time.perf_counter() - t0
    if pool:
        pool.shutdown()
    return dt, steps, nbytes, kind, desc + ("; OpenMP threads over contiguous bag ranges" if jit.available else "")


# ---- multi-table workloads (configurations 3 and 4) ----------------------------------

def main_multi(args):
    """Table-wise sharded multi-table lookup: every rank pools the global batch
    for the tables it owns and the kernels store the pooled rows batch-wise
    into the owning ranks' buffers.  One step = one global batch over all
    tables."""
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=5))  # a lost rank ends the run
    import fbgemm_b200 as F
    from fbgemm_b200 import workloads as W
    from fbgemm_b200.sharding import ShardedLookup, TableWisePlan, expected_cost

    if args.workload == 3:
        specs = W.config3_tables(max(world, int(round(64 * args.tables_scale))), args.scale)
        B, alpha, idt, weighted, name = int(16384 * args.batch_scale), 1.05, torch.int32, False, "mixed 8/4/2-bit"
        mean_len = 30.0
        plan = TableWisePlan.balanced([expected_cost(s, B, mean_len) for s in specs], [s.dim for s in specs], world)
    else:
        per_gpu = max(1, int(round(32 * args.tables_scale)))
        specs = W.config4_tables(per_gpu * world, args.scale)
        B, alpha, idt, weighted, name = int(65536 * args.batch_scale), 1.1, torch.int64, True, "4-bit x128"
        mean_len = 40.0
        plan = TableWisePlan.balanced([1.0] * len(specs), [s.dim for s in specs], world)
    B -= B % world
    tnp = {torch.int32: np.int32, torch.int64: np.int64}
    sl = ShardedLookup(specs, plan, rank, B, dev, torch.float16, mode=args.redistribution, num_buffers=2,
                       weighted=weighted, index_dtype=tnp[idt], offset_dtype=tnp[idt])
    perms = {t: W.row_permutation(specs[t].rows, dev, specs[t].seed + 5) for t in sl.local}
    nsets = 2
    sets = []
    for sidx in range(nsets):
        d = {}
        for t in sl.local:
            g = torch.Generator(device=dev).manual_seed(specs[t].seed + 77 * sidx)
            if args.workload == 3:
                lengths = torch.poisson(torch.full((B,), mean_len, device=dev), generator=g).to(torch.int64)
            else:
                lengths = torch.full((B,), int(mean_len), device=dev, dtype=torch.int64)
            off = W.offsets_from_lengths(lengths, idt)
            n = int(off[-1])
            idx = W.zipf_indices(n, alpha, specs[t].rows, dev, specs[t].seed + 1000 + sidx, idt, perms[t])
            wts = torch.rand(n, generator=g, device=dev) if weighted else None
            d[t] = W.Batch(idx, off, wts, B, n, n)
        sets.append(d)
    del perms
    bytes_local = float(np.mean([sum(b.index_size * specs[t].row_bytes for t, b in d.items()) for d in sets]))
    streams = [torch.cuda.Stream(device=dev) for _ in range(4)]
    handles = [s.cuda_stream for s in streams]

    plans = None
    if args.launch == "plan":
        # one kernel launch per kernel variant instead of one per table
        plans = [sl.make_plan(sets[j % nsets], buffer=j, slot=400 + j) for j in range(2)]
    launches_per_step = plans[0].num_launches if plans else len(sl.local)

    def step(i):
        if plans:
            plans[i % 2].launch()
        else:
            cur = torch.cuda.current_stream()
            for s in streams:
                s.wait_stream(cur)
            sl.launch(sets[i % nsets], buffer=i % 2, slot_base=(i % 4) * 100, streams=handles)
            for s in streams:
                cur.wait_stream(s)
        if args.redistribution == "nccl":
            sl.exchange(i % 2)

    for i in range(max(args.warmup, 3)):
        step(i)
    sl.barrier()
    ok = all(F.status_read(s, dev.index)[0] for s in range(402))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        sl.barrier()
    ms = e0.elapsed_time(e1)
    ok = ok and all(F.status_read(s, dev.index)[0] for s in range(402))
    tot = torch.tensor([bytes_local, ms, float(ok)], device=dev, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist

        t_ms = tot[1:2].clone()
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
        t_b = tot[0:1].clone()
        dist.all_reduce(t_b, op=dist.ReduceOp.SUM)
        t_ok = tot[2:3].clone()
        dist.all_reduce(t_ok, op=dist.ReduceOp.MIN)
        ms, job_bytes, ok = float(t_ms), float(t_b), bool(t_ok)
    else:
        job_bytes = bytes_local
    sec = ms / 1e3
    peak, peak_src = measured_peak()
    value = job_bytes * args.steps / sec / 1e9
    # cpu_baseline (one GPU only): the reference's CPU kernels on a sample of this rank's tables - the whole set does
    # not fit a host (config 4) or would take minutes (config 3), so a few tables stand for the rest
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import types

        threads = os.cpu_count() or 1
        sample = sl.local[:: max(1, len(sl.local) // 3)][:3]
        tot_b, tot_t, kind, desc = 0, 0.0, "", ""
        for t in sample:
            wl = types.SimpleNamespace(bit_rate=specs[t].bit_rate, dim=specs[t].dim, rows=specs[t].rows,
                                       row_bytes=specs[t].row_bytes, out_dtype=torch.float16,
                                       normalize_by_lengths=False)
            dt, steps, nbytes, kind, desc = time_cpu(wl, [sets[0][t]], sl.tables[t].cpu().numpy(), None, threads, 3,
                                                     args.cpu_seconds)
            tot_b, tot_t = tot_b + nbytes, tot_t + dt
        cpu = {"value": tot_b / tot_t / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
               "sample": f"tables {sample} of {len(specs)} (their whole batches, up to 3 passes each), every batch split "
                         f"over {threads} host threads; {desc}; extrapolates to the whole table set by gathered bytes"}
    if rank == 0:
        print(json.dumps({
            "metric": "gathered_row_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if args.workload == 3 else "weak", "vs_baseline": None,
            "dtype": "u8/u4/u2->f32 accumulate", "data": "synthetic",
            "config": {"workload": f"{len(specs)} tables {name}, table-wise over {world} GPU(s), batch {B} per table",
                       "baseline_config_index": args.workload, "tables": len(specs), "total_dim": plan.total_dim,
                       "rows_scale": args.scale, "tables_scale": args.tables_scale, "batch_scale": args.batch_scale,
                       "table_GB_this_rank": round(sum(t.numel() for t in sl.tables.values()) / 1e9, 2),
                       "redistribution": args.redistribution,
                       "launch": (f"multi-table plan, {launches_per_step} kernel launches per step" if plans else
                                  f"one launch per table ({launches_per_step} per step) over 4 streams"),
                       "l2": "tables are far larger than L2; two alternating input sets"},
            "results_ok": ok, "bags_per_s": len(specs) * B * args.steps / sec,
            "frac_of_hbm_peak": value / world / peak, "clocks": clocks.summary(),
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak, "traffic": None, "peak_source": peak_src},
            "e2e": None, "cpu_baseline": cpu}))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


# ---- main -----------------------------------------------------------------------

def main():
    args = parse_args()
    if args.workload in (3, 4) and args.impl != "reference":
        return main_multi(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference" and rank != 0:
        return 0  # the CPU arm runs on rank 0 alone

    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: fbgemm_b200 has no CPU path"}))
        return 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        if args.impl != "reference":
            dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=5))  # a lost rank ends the run

    import fbgemm_b200 as F
    from fbgemm_b200 import workloads as W

    # Table-wise sharding, weak scaling: every rank owns one table of the
    # workload's shape (its own seed) and pools the same number of bags.
    w = W.CONFIGS[args.workload](dev, scale=args.scale, seed=W.SEED + 1000 * rank)
    base = [w.make_batch(s) for s in range(NUM_BATCHES * args.group)]
    batches = [concat_batches(base[i * args.group:(i + 1) * args.group]) if args.group > 1 else base[i]
               for i in range(NUM_BATCHES)]
    bytes_per_step = float(np.mean([W.algorithmic_bytes(w, b) for b in batches]))
    all_bytes_per_step = float(np.mean([W.all_bytes(w, b) for b in batches]))
    bags_per_step = batches[0].output_size
    config = {
        "workload": w.name, "baseline_config_index": args.workload,
        "table_rows": int(w.table.shape[0]), "row_bytes": w.row_bytes, "table_MB": round(w.table.numel() / 1e6, 1),
        "bags_per_step": bags_per_step, "gathered_rows_per_step": round(bytes_per_step / w.row_bytes, 1),
        "gathered_bytes_per_step": round(bytes_per_step), "batches_per_call": args.group,
        "distinct_batches": NUM_BATCHES, "launch": f"CUDA graph, {args.streams} streams",
        "l2": "table (larger than the 126 MB L2) is the gathered input; steps rotate over distinct batches",
        "sharding": "table-wise, one table per GPU" if world > 1 else "single table",
    }

    if args.impl == "reference":
        threads = os.cpu_count() or 1
        host_table = w.table.cpu().numpy()
        host_cit = w.cit.cpu().numpy() if w.cit is not None else None
        time_cpu(w, batches[:2], host_table, host_cit, threads, args.warmup, 2.0)
        dt, steps, nbytes, kind, desc = time_cpu(w, batches, host_table, host_cit, threads, args.steps, 60.0)
        gbs = nbytes / dt / 1e9
        line = {
            "impl": "reference", "metric": "gathered_row_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": f"u{w.bit_rate}->f32 accumulate", "data": "synthetic",
            "config": config, "bags_per_s": bags_per_step * steps / dt,
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": kind,
                             "sample": f"{steps} whole batches, each split over {threads} host threads; {desc}"},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        print(json.dumps(line))
        return 0

    kern = w.make_kernel()
    sharded = None
    if world > 1:
        # Table-wise sharding: this rank's table pools the whole batch and the
        # kernel stores every pooled row straight into the output buffer of the
        # rank that owns that slice of the batch (peer stores over NVLink):
        # lookup and all-to-all in one kernel.
        from fbgemm_b200.sharding import ShardedLookup, TableWisePlan

        assert w.cit is None, "the sharded path covers dense tables"
        tnp = {torch.int32: np.int32, torch.int64: np.int64}
        specs = [W.TableSpec(w.rows, w.dim, w.bit_rate, W.SEED + 1000 * r) for r in range(world)]
        plan = TableWisePlan(list(range(world)), [w.dim] * world, world)
        sharded = ShardedLookup(specs, plan, rank, bags_per_step, dev, w.out_dtype, mode="p2p",
                                num_buffers=NUM_BATCHES, tables={rank: w.table}, weighted=w.has_weight,
                                index_dtype=tnp[w.index_dtype], offset_dtype=tnp[w.offset_dtype])
        config["redistribution"] = ("pooled rows stored by the lookup kernel into the owning rank's "
                                    f"[{bags_per_step // world}, {plan.total_dim}] buffer (peer stores, symmetric memory)")
    else:
        outs = [torch.zeros(b.output_size * w.dim, dtype=w.out_dtype, device=dev) for b in batches]

    def launch(i, stream=None):
        b = batches[i % NUM_BATCHES]
        if sharded is not None:
            sharded.launch({rank: b}, buffer=i % NUM_BATCHES, slot_base=i % 256, stream=stream)
        else:
            kern.launch(b.output_size, b.index_size, w.rows, w.table, b.indices, b.offsets, b.weights,
                        outs[i % NUM_BATCHES], w.cit, slot=i % 256, stream=stream)

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: device-resident inputs ------------------------------------
    for i in range(max(args.warmup, 3)):
        launch(i)
    torch.cuda.synchronize()
    assert all(F.status_read(s)[0] for s in range(256)), "a warm-up lookup reported an error"

    chunk = min(GRAPH_CHUNK, args.steps)
    streams = [torch.cuda.Stream(device=dev) for _ in range(max(1, args.streams))]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        cur = torch.cuda.current_stream()
        for s in streams:
            s.wait_stream(cur)
        for i in range(chunk):
            with torch.cuda.stream(streams[i % len(streams)]):
                launch(i)
        for s in streams:
            cur.wait_stream(s)
    graph_launches = F.launch_count()  # capture counted `chunk` launches that did not run
    replays, rest = divmod(args.steps, chunk)
    graph.replay()
    torch.cuda.synchronize()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
    barrier()
    with ClockSampler(local_rank) as clocks:
        e0.record()
        marks[0].record()
        for r in range(replays):
            graph.replay()
            marks[r + 1].record()   # between replays: spread of the per-step time over the run
        for i in range(rest):
            launch(i)
        e1.record()
        torch.cuda.synchronize()
    barrier()
    ms = e0.elapsed_time(e1)
    per_step_us = sorted(marks[r].elapsed_time(marks[r + 1]) * 1e3 / chunk for r in range(replays))

    def pct(q):
        return per_step_us[min(len(per_step_us) - 1, int(q * len(per_step_us)))] if per_step_us else None

    # one call alone on an idle GPU (launch to completion), median of 20
    lat = []
    for i in range(20):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        launch(i)
        b.record()
        torch.cuda.synchronize()
        lat.append(a.elapsed_time(b) * 1e3)
    single_call_us = sorted(lat)[len(lat) // 2]
    ok = all(F.status_read(s)[0] for s in range(256))
    timed_launches = replays * chunk + rest
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        tot = torch.tensor([bytes_per_step, float(bags_per_step)], device=dev, dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        job_bytes_per_step, job_bags_per_step = float(tot[0]), float(tot[1])
    else:
        job_bytes_per_step, job_bags_per_step = bytes_per_step, float(bags_per_step)
    sec = ms / 1e3
    value = job_bytes_per_step * args.steps / sec / 1e9
    per_launch_us = ms * 1e3 / timed_launches
    peak, peak_src = measured_peak()
    achieved = bytes_per_step / (per_launch_us * 1e-6) / 1e9

    # ---- e2e: host buffers through the C ABI -------------------------------------
    e2e = None
    if not args.no_e2e:
        lanes = 8
        hb = []
        for b in batches:
            pin = lambda t: t.cpu().pin_memory().numpy() if t is not None else None  # noqa: E731
            hb.append((pin(b.indices), pin(b.offsets), pin(b.weights),
                       torch.zeros(b.output_size * w.dim, dtype=w.out_dtype).pin_memory().numpy(), b))
        ctx = F.get_context(local_rank)
        import ctypes as C

        from fbgemm_b200 import _capi
        steps_e2e = min(args.e2e_steps, args.steps)

        def submit(i):
            idx, off, wts, out, b = hb[i % NUM_BATCHES]
            rc = _capi.lib().fbgemm_b200_spmdm_host_submit(
                ctx.handle, i % lanes, C.byref(kern.cfg), b.output_size, b.index_size, w.rows,
                host_key, idx.ctypes.data, off.ctypes.data, wts.ctypes.data if wts is not None else None,
                out.ctypes.data, cit_key)
            _capi.check(rc, "host_submit")

        # The caller's table lives in host memory; it is registered once (one
        # upload) and stays resident in HBM under its host address.
        host_tbl = w.table.cpu().numpy()
        ctx.register_table(host_tbl)
        host_key = host_tbl.ctypes.data
        cit_key = None
        if w.cit is not None:
            host_cit = w.cit.cpu().numpy()
            ctx.register_table(host_cit)
            cit_key = host_cit.ctypes.data
        for i in range(lanes):
            submit(i)
        for i in range(lanes):
            assert kern.host_wait(i % lanes)
        barrier()
        t0 = time.perf_counter()
        for i in range(steps_e2e):
            if i >= lanes:
                kern.host_wait(i % lanes)
            submit(i)
        for i in range(min(lanes, steps_e2e)):
            kern.host_wait((steps_e2e + i) % lanes)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        barrier()
        if world > 1:
            import torch.distributed as dist

            t = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        h2d = float(np.mean([x[0].nbytes + x[1].nbytes + (x[2].nbytes if x[2] is not None else 0) for x in hb]))
        d2h = float(np.mean([x[3].nbytes for x in hb])) + 16
        e2e = {"value": job_bytes_per_step * steps_e2e / dt / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": round(h2d), "d2h_bytes_per_step": round(d2h), "steps": steps_e2e,
               "ms_per_step": dt / steps_e2e * 1e3, "bags_per_s": job_bags_per_step * steps_e2e / dt,
               "path": "fbgemm_b200_spmdm_host_submit/wait, 8 pipelined lanes, pinned host buffers, table resident"
                       + ("; every rank calls it on its own table and gets its rows back in its own host buffer "
                          "(the host-pointer interface has no redistribution step)" if world > 1 else ""),
               "timer": "host perf_counter bracketed by device synchronisation"}
        ctx.unregister_table(host_tbl)
        if w.cit is not None:
            ctx.unregister_table(host_cit)

    # ---- the practical ceiling: the same rows fetched with no arithmetic ----------
    ceiling = None
    if rank == 0:
        import ctypes as C

        from fbgemm_b200 import _capi
        rows_all = torch.cat([(w.cit[b.indices.long()] if w.cit is not None else b.indices).to(torch.int32)
                              for b in batches])
        rows_all = rows_all[rows_all >= 0].contiguous()
        mean_len = max(1, int(round(sum(b.index_size for b in batches) / sum(b.output_size for b in batches))))
        sink = torch.zeros(1, dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream

        def probe():
            _capi.check(_capi.lib().fbgemm_b200_probe_row_gather(
                w.table.data_ptr(), w.row_bytes, w.row_bytes, rows_all.data_ptr(), rows_all.numel(), mean_len,
                sink.data_ptr(), stream), "probe")
        for _ in range(3):
            probe()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(10):
            probe()
        p1.record()
        torch.cuda.synchronize()
        probe_ms = p0.elapsed_time(p1) / 10
        ceiling = rows_all.numel() * w.row_bytes / (probe_ms * 1e-3) / 1e9

    # ---- cpu_baseline (rank 0, one GPU only) ------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        host_table = w.table.cpu().numpy()
        host_cit = w.cit.cpu().numpy() if w.cit is not None else None
        dt, steps, nbytes, kind, desc = time_cpu(w, batches, host_table, host_cit, threads, 10 ** 9, args.cpu_seconds)
        dt1, steps1, nbytes1, _, _ = time_cpu(w, batches, host_table, host_cit, 1, 10 ** 9, min(3.0, args.cpu_seconds))
        cpu = {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
               "sample": f"{steps} whole batches in {dt:.1f} s, each split over {threads} host threads; {desc}",
               "bags_per_s": bags_per_step * steps / dt,
               "one_thread": {"value": nbytes1 / dt1 / 1e9, "unit": "GB/s",
                              "sample": f"{steps1} whole batches in {dt1:.1f} s on one thread"}}

    if rank == 0:
        line = {
            "metric": "gathered_row_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": f"u{w.bit_rate}->f32 accumulate", "data": "synthetic",
            "config": config, "results_ok": bool(ok),
            "us_per_step_p10_p50_p90": [pct(0.1), pct(0.5), pct(0.9)],
            "single_call_latency_us": single_call_us,
            "bags_per_s": job_bags_per_step * args.steps / sec,
            "all_bytes_GBps": all_bytes_per_step * world * args.steps / sec / 1e9,
            "frac_of_hbm_peak": value / world / peak,
            "clocks": clocks.summary(),
            "e2e": e2e,
            "gpu_launches": timed_launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH.get((args.workload, args.group)),
                         "traffic_source": "dram__bytes_read+write of one ncu capture of this launch shape "
                                           "(profiles/spmdm_direct*_kernel__workload*_*.md)",
                         "peak_source": peak_src, "per_launch_us": per_launch_us,
                         "random_row_gather_ceiling_GBps": ceiling,
                         "frac_of_gather_ceiling": (achieved / ceiling) if ceiling else None,
                         "ceiling_note": "fbgemm_b200_probe_row_gather: the same rows read with the same lane "
                                         "layout and no arithmetic, one launch over all 32 batches",
                         "note": "achieved = gathered-row bytes per launch / (timed region / launches); launches "
                                 "of different streams overlap"},
            "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

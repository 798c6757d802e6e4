#!/usr/bin/env python
"""Benchmark of the quantized embedding-bag lookup on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload 0..4]

The default workload is the table-wise sharded multi-table configuration (64
mixed 8/4/2-bit tables, 16 384 bags per table, strong scaling over the N GPUs,
pooled rows redistributed batch-wise by the lookup kernels' own peer stores).
A *step* is ``--batches-per-step`` global batches (64 functor calls each) on
rotating pre-generated input sets, so that even the shortest driver run times
well over a thousand functor calls.  ``--workload 0|1|2`` times one of the
single-table configurations instead (a step = one CUDA-graph replay of
``--calls-per-step`` functor calls on rotating batches); at N = 1 the default
run carries all three as ``single_table`` sub-records.

Prints ONE JSON line:

* ``value``       gathered-row GB/s of the whole job, inputs resident in HBM,
                  device time (CUDA events), max over ranks.
* ``e2e``         the same metric through the host-pointer C-ABI calls
                  (``fbgemm_b200_multi_host_*`` / ``fbgemm_b200_spmdm_host_*``):
                  index arrays leave pinned host memory and the pooled rows
                  return to the host inside the timed region; tables resident.
* ``roofline``    HBM roofline of the lookup on gathered-row bytes per GPU.
* ``cpu_baseline`` the reference's CPU kernels timed on this box's host cores on
                  a bounded sample of the same workload (N = 1 only).
* ``results_ok``  pooled rows of sampled bags compared bit for bit with the CPU
                  oracle inside the run (on every rank, rows stored by peers
                  included), AND no lookup reported an error.

``--impl reference`` times only the reference's CPU path (all host threads) on
the same configuration, metric and step definition and prints the same line
shape with ``"impl": "reference"``; it never loads libfbgemm_b200.so.
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

_JSON_OUT = None


def claim_stdout():
    """stdout carries the one JSON line and nothing else: whatever libraries
    print there from now on (NCCL's version banner, for one) goes to stderr."""
    global _JSON_OUT
    if _JSON_OUT is None:
        sys.stdout.flush()
        _JSON_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _JSON_OUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()

FALLBACK_HBM_GBS = 6650.0
NUM_BATCHES = 32        # distinct pre-generated batches a single-table run rotates over
NUM_SETS = 4            # distinct pre-generated global batches a multi-table run rotates over
PARITY_BAGS = 64        # bags per table compared with the oracle inside the run
# DRAM bytes (read + write) of the lookup kernels per unit of work, from ncu captures
# (dram__bytes_read.sum + dram__bytes_write.sum; the files under profiles/ say how each was taken).
TRAFFIC = {
    # single-table workloads: DRAM bytes per functor call of the configuration's batch in the benchmark's steady state
    0: {"bytes_per_call": 25_902_699 + 5_179_565, "source": "profiles/lookup_kernels__workloads012_steady_state_dram.md"},
    1: {"bytes_per_call": 10_020_888 + 629_504, "source": "profiles/lookup_kernels__workloads012_steady_state_dram.md"},
    2: {"bytes_per_call": 13_405_040 + 4_003_784, "source": "profiles/lookup_kernels__workloads012_steady_state_dram.md"},
    # the 64-table configuration: DRAM bytes of all kernels of one global batch (captured at a quarter of the batch, x 4)
    3: {"bytes_per_global_batch": 4 * (2_174_574_080 + 178_803_456) / 2, "source": "profiles/lookup_kernels__default_workload_dram.md"},
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", type=int, default=3,
                    help="benchmark configuration 0..4: 8-bit, 4-bit, pruned 2-bit single tables; 64 mixed tables "
                         "(default); 256 large tables; 5: the kernels either side of the lookup (pruning lookups, index "
                         "remap, sequence lookup), one GPU")
    ap.add_argument("--batches-per-step", type=int, default=16, help="workloads 3/4: global batches per step")
    ap.add_argument("--calls-per-step", type=int, default=512, help="workloads 0-2: functor calls per step (one graph)")
    ap.add_argument("--streams", type=int, default=16, help="workloads 0-2: streams the graph spreads the calls over")
    ap.add_argument("--group", type=int, default=1, help="workloads 0-2: batches concatenated into one call")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink table rows (and, for workloads 0-2, the batch)")
    ap.add_argument("--tables-scale", type=float, default=1.0, help="workloads 3/4: fraction of the tables")
    ap.add_argument("--batch-scale", type=float, default=1.0, help="workloads 3/4: fraction of the batch")
    ap.add_argument("--batches-in-flight", type=int, default=0,
                    help="workloads 3/4: global batches in flight, each with its own output buffer, stream and counters "
                         "(default: as many as ranks, at least 2 and at most 8 - the more ranks, the shorter a rank's "
                         "share of a batch against the latency of the counters and of the peer stores; measured at "
                         "8 ranks: 0.2005 / 0.1926 / 0.1807 ms per global batch with 2 / 4 / 8 in flight)")
    ap.add_argument("--shard", default=None, metavar="K/G",
                    help="workload 3 on one GPU: only the tables that rank K of a G-rank table-wise plan owns (what that "
                         "rank's lookups take per global batch, with no store leaving the GPU)")
    ap.add_argument("--launch", default="streams", choices=["plan", "streams"],
                    help="workloads 3/4: one multi-table plan (a launch per kernel variant) or a launch per table")
    ap.add_argument("--redistribution", default="p2p", choices=["p2p", "nccl"],
                    help="workloads 3/4: peer stores from the lookup kernel, or NCCL all-to-all after it")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-pointer leg")
    ap.add_argument("--no-single", action="store_true", help="skip the single_table sub-records of the default run")
    ap.add_argument("--peer-ab", action="store_true",
                    help="workloads 3/4, N > 1: time the same steps again with every pooled row stored into the rank's own "
                         "buffer instead of its owner's (what the stores across NVLink cost)")
    ap.add_argument("--e2e-batches", type=int, default=12, help="workloads 3/4: global batches of the host-pointer leg")
    ap.add_argument("--e2e-steps", type=int, default=4, help="workloads 0-2: steps of the host-pointer leg")
    ap.add_argument("--cpu-seconds", type=float, default=4.0, help="wall-time bound of the CPU sample")
    ap.add_argument("--callers-only", choices=["hashmap", "array", "sequence", "remap"], default=None,
                    help="workload 5: one of the caller-side kernels instead of all")
    ap.add_argument("--caller-iters", type=int, default=20, help="workload 5: timed calls per kernel")
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

    def __init__(self, index: int, period_s: float = 0.005):
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


def pctl(sorted_vals, q):
    return sorted_vals[min(len(sorted_vals) - 1, int(q * len(sorted_vals)))] if sorted_vals else None


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


# ---- the oracle as the checker of sampled bags ----------------------------------------

def oracle_sample(oracle, bit_rate, dim, out_np, table, cit, indices, offsets, weights, normalize, bags):
    """Pool ``bags`` of one functor call on the CPU: the rows they name are
    copied back from the device table, compacted into a small table with
    re-numbered indices, and pooled by the oracle.  Returns [len(bags), dim]."""
    import torch

    off = offsets.cpu().numpy().astype(np.int64)
    pos = np.concatenate([np.arange(off[m], off[m + 1]) for m in bags]) if len(bags) else np.zeros(0, np.int64)
    lens = [off[m + 1] - off[m] for m in bags]
    pos_t = torch.from_numpy(pos).to(indices.device)
    idx = indices[pos_t].cpu().numpy().astype(np.int64)
    wts = weights[pos_t].cpu().numpy() if weights is not None else None
    dense = cit[torch.from_numpy(idx).to(cit.device)].cpu().numpy().astype(np.int64) if cit is not None else idx
    uniq, inv = np.unique(dense[dense >= 0], return_inverse=True)
    small = (table[torch.from_numpy(uniq).to(table.device)].cpu().numpy() if len(uniq)
             else np.zeros((1, table.shape[1]), np.uint8))
    new_off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    if cit is not None:
        mapping = np.full(max(len(idx), 1), -1, dtype=np.int32)
        mapping[:len(idx)][dense >= 0] = inv.astype(np.int32)
        ok, ref = oracle.spmdm_rowwise_sparse(bit_rate, dim, len(mapping), small, np.arange(len(idx), dtype=np.int64),
                                              mapping, new_off, wts, normalize)
    else:
        ok, ref = oracle.spmdm(bit_rate, dim, len(small), small, inv.astype(np.int64), new_off, wts, normalize, out_np)
    assert ok, "the oracle refused a sampled bag"
    return ref.reshape(-1)[:len(bags) * dim].reshape(len(bags), dim)


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    view = {2: np.uint16, 4: np.uint32}[a.dtype.itemsize]
    return a.shape == b.shape and bool((a.view(view) == b.view(view)).all())


# ---- CPU legs (the reference arm and cpu_baseline) -------------------------------------

class CpuTable:
    """One table of the CPU leg: its shape, host copy and host batches."""

    def __init__(self, bit_rate, dim, rows, out_half, normalize, host_table, host_cit, batches, row_bytes):
        self.bit_rate, self.dim, self.rows, self.normalize = bit_rate, dim, rows, normalize
        self.table, self.cit = host_table, host_cit
        out_dt = np.float16 if (out_half and host_cit is None) else np.float32
        self.batches = []
        for b in batches:
            self.batches.append({
                "indices": b.indices.cpu().numpy(), "offsets": b.offsets.cpu().numpy(),
                "weights": b.weights.cpu().numpy() if b.weights is not None else None,
                "B": b.output_size, "bytes": b.valid_rows * row_bytes,
                "out": np.zeros(b.output_size * dim, dtype=out_dt)})


def cpu_impl():
    """(object with batch_parallel/spmdm, kind, description): the reference's
    JIT kernels bundled in libtorch_cpu.so, else its scalar sources, else the
    oracle port."""
    from oracle import checker

    jit = checker.ReferenceJit()
    if jit.available:
        return jit, "reference", ("FBGEMM asmjit AVX2/AVX-512 kernels as bundled in libtorch_cpu.so; OpenMP threads "
                                  "over contiguous bag ranges")
    ref = checker.Reference()
    if ref.available:
        return ref, "reference", "FBGEMM scalar EmbeddingSpMDM*_ref compiled from the reference tree"
    return checker.Oracle(), "port", "plain-C oracle port (oracle/embedding_oracle.c)"


def run_cpu_batch(impl, tbl, hb, threads, pool):
    """One whole batch of one table, split over ``threads`` host threads
    (contiguous bag ranges, one functor call each: how the reference's callers
    and benchmarks parallelise this single-threaded kernel)."""
    if hasattr(impl, "batch_parallel"):
        return impl.batch_parallel(tbl.bit_rate, tbl.dim, tbl.rows, tbl.table, hb["indices"], hb["offsets"],
                                   hb["weights"], tbl.normalize, hb["out"], threads, tbl.cit)
    B = hb["B"]
    cuts = [B * t // threads for t in range(threads + 1)]

    def call(lo, hi):
        offs = hb["offsets"][lo:hi + 1]
        i0, i1 = int(offs[0]), int(offs[-1])
        idx = hb["indices"][i0:i1]
        wts = hb["weights"][i0:i1] if hb["weights"] is not None else None
        if tbl.cit is not None:
            return impl.spmdm_rowwise_sparse(tbl.bit_rate, tbl.dim, tbl.rows, tbl.table, idx, tbl.cit, offs, wts,
                                             tbl.normalize)[0]
        return impl.spmdm(tbl.bit_rate, tbl.dim, tbl.rows, tbl.table, idx, offs, wts, tbl.normalize,
                          hb["out"].dtype)[0]

    futs = [pool.submit(call, cuts[t], cuts[t + 1]) for t in range(threads) if cuts[t + 1] > cuts[t]]
    return all(f.result() for f in futs)


def time_cpu(tables, threads, calls_per_step, max_steps, max_seconds, warmup_steps=1):
    """Steps of ``calls_per_step`` functor calls (whole batches, round-robin
    over the tables and their rotating batches) until ``max_steps`` steps or
    ``max_seconds``.  Returns dict(seconds, steps, calls, bytes, bags, kind, desc)."""
    from concurrent.futures import ThreadPoolExecutor

    impl, kind, desc = cpu_impl()
    pool = None if hasattr(impl, "batch_parallel") else ThreadPoolExecutor(max_workers=threads)
    order = [(t, j) for j in range(max(len(t.batches) for t in tables)) for t in tables if j < len(t.batches)]
    at = 0

    def one_step(budget_end=None):
        nonlocal at
        nbytes = bags = calls = 0
        for _ in range(calls_per_step):
            tbl, j = order[at % len(order)]
            at += 1
            hb = tbl.batches[j]
            assert run_cpu_batch(impl, tbl, hb, threads, pool), "the CPU reference returned false on a valid batch"
            nbytes += hb["bytes"]
            bags += hb["B"]
            calls += 1
            if budget_end is not None and time.perf_counter() > budget_end:
                break
        return nbytes, bags, calls

    for _ in range(warmup_steps):   # JIT generation, page faults, caches
        one_step(time.perf_counter() + max(1.0, max_seconds / 4))
    t0 = time.perf_counter()
    tot_b = tot_bags = tot_calls = steps = 0
    while steps < max_steps and (time.perf_counter() - t0) < max_seconds:
        nb, bg, c = one_step(t0 + max_seconds if max_steps >= 10 ** 8 else None)
        tot_b, tot_bags, tot_calls, steps = tot_b + nb, tot_bags + bg, tot_calls + c, steps + 1
    dt = time.perf_counter() - t0
    if pool:
        pool.shutdown()
    return {"seconds": dt, "steps": steps, "calls": tot_calls, "bytes": tot_b, "bags": tot_bags, "kind": kind, "desc": desc}


# ---- single-table workloads (configurations 0, 1, 2) ------------------------------------

def run_single(args, cfg_index, dev, rank, world, steps, warmup, full, seed_shift=0):
    """Times one single-table configuration on this rank's GPU.  A step is one
    replay of a CUDA graph of ``calls_per_step`` functor calls spread over
    ``streams`` streams, the calls rotating over NUM_BATCHES distinct batches.
    Returns a record (dict); ``full`` adds the host-pointer leg, the CPU leg and
    the one-call latency."""
    import torch

    import fbgemm_b200 as F
    from fbgemm_b200 import workloads as W
    from oracle.checker import Oracle

    w = W.CONFIGS[cfg_index](dev, scale=args.scale, seed=W.SEED + 1000 * rank + seed_shift)
    base = [w.make_batch(s) for s in range(NUM_BATCHES * args.group)]
    batches = [concat_batches(base[i * args.group:(i + 1) * args.group]) if args.group > 1 else base[i]
               for i in range(NUM_BATCHES)]
    bytes_per_call = float(np.mean([W.algorithmic_bytes(w, b) for b in batches]))
    all_bytes_per_call = float(np.mean([W.all_bytes(w, b) for b in batches]))
    bags_per_call = batches[0].output_size
    cps = max(1, args.calls_per_step)
    kern = w.make_kernel()
    outs = [torch.zeros(b.output_size * w.dim, dtype=w.out_dtype, device=dev) for b in batches]

    def launch(i, stream=None):
        b = batches[i % NUM_BATCHES]
        kern.launch(b.output_size, b.index_size, w.rows, w.table, b.indices, b.offsets, b.weights,
                    outs[i % NUM_BATCHES], w.cit, slot=i % 256, stream=stream)

    # every batch once, eagerly; sampled bags of three of them against the oracle
    for i in range(NUM_BATCHES):
        launch(i)
    torch.cuda.synchronize()
    status_ok = all(F.status_read(s)[0] for s in range(256))
    oracle = Oracle()
    rng = np.random.default_rng(cfg_index + 17)
    out_np = np.float16 if w.out_dtype == torch.float16 else np.float32
    values_ok = True
    for i in (0, NUM_BATCHES // 2, NUM_BATCHES - 1):
        b = batches[i]
        bags = np.sort(rng.choice(b.output_size, min(PARITY_BAGS, b.output_size), replace=False))
        want = oracle_sample(oracle, w.bit_rate, w.dim, out_np, w.table, w.cit, b.indices, b.offsets, b.weights,
                             w.normalize_by_lengths, bags)
        got = outs[i].view(b.output_size, w.dim)[torch.from_numpy(bags).to(dev)].cpu().numpy()
        values_ok = values_ok and same_bits(got, want)

    streams = [torch.cuda.Stream(device=dev) for _ in range(max(1, args.streams))]
    graph = torch.cuda.CUDAGraph()
    captured = F.launch_count()
    with torch.cuda.graph(graph):
        cur = torch.cuda.current_stream()
        for s in streams:
            s.wait_stream(cur)
        for i in range(cps):
            with torch.cuda.stream(streams[i % len(streams)]):
                launch(i)
        for s in streams:
            cur.wait_stream(s)
    captured = int(F.launch_count() - captured)   # kernels of this library in one replay of the graph
    for _ in range(max(warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        torch.cuda.synchronize()
    with ClockSampler(dev.index) as clocks:
        marks[0].record()
        for r in range(steps):
            graph.replay()
            marks[r + 1].record()
        torch.cuda.synchronize()
    ms = marks[0].elapsed_time(marks[steps])
    per_step_ms = sorted(marks[r].elapsed_time(marks[r + 1]) for r in range(steps))
    status_ok = status_ok and all(F.status_read(s)[0] for s in range(256))
    peak, peak_src = measured_peak()
    per_call_us = ms * 1e3 / (steps * cps)
    value = bytes_per_call / (per_call_us * 1e-6) / 1e9
    traffic = TRAFFIC.get(cfg_index) if args.scale == 1.0 else None
    rec = {
        "workload": w.name, "baseline_config_index": cfg_index, "value": value, "unit": "GB/s",
        "frac": value / peak, "peak": peak, "peak_source": peak_src,
        "ms_per_call": per_call_us / 1e3, "ms_per_step": ms / steps, "steps": steps, "calls_per_step": cps,
        "timed_region_s": ms / 1e3,
        "ms_per_step_p10_p50_p90": [pctl(per_step_ms, 0.1), pctl(per_step_ms, 0.5), pctl(per_step_ms, 0.9)],
        "bags_per_s": bags_per_call / (per_call_us * 1e-6),
        "all_bytes_GBps": all_bytes_per_call / (per_call_us * 1e-6) / 1e9,
        "gathered_bytes_per_call": round(bytes_per_call), "bags_per_call": bags_per_call,
        "row_bytes": w.row_bytes, "table_MB": round(w.table.numel() / 1e6, 1),
        "traffic": (traffic["bytes_per_call"] * args.group) if traffic else None,
        "traffic_source": traffic["source"] if traffic else None,
        "results_ok": bool(status_ok and values_ok),
        "results_check": f"{min(PARITY_BAGS, bags_per_call)} sampled bags of 3 batches bit-equal to the CPU oracle; no "
                         "lookup reported an error",
        "gpu_launches": captured * steps,
        "clocks": clocks.summary(),
    }
    if not full:
        del w, batches, outs, graph
        torch.cuda.empty_cache()
        return rec

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
    rec["single_call_latency_us"] = sorted(lat)[len(lat) // 2]

    # ---- e2e: host buffers through the C ABI, the same step definition --------------
    rec["e2e"] = None
    if not args.no_e2e:
        import ctypes as C

        from fbgemm_b200 import _capi

        lanes = _capi.HOST_LANES
        hb = []
        for b in batches:
            pin = lambda t: t.cpu().pin_memory().numpy() if t is not None else None  # noqa: E731
            hb.append((pin(b.indices), pin(b.offsets), pin(b.weights),
                       torch.zeros(b.output_size * w.dim, dtype=w.out_dtype).pin_memory().numpy(), b))
        ctx = F.get_context(dev.index)
        host_tbl = w.table.cpu().numpy()
        ctx.register_table(host_tbl)     # the caller's table: one upload, resident under its host address
        host_key, cit_key, host_cit = host_tbl.ctypes.data, None, None
        if w.cit is not None:
            host_cit = w.cit.cpu().numpy()
            ctx.register_table(host_cit)
            cit_key = host_cit.ctypes.data

        # what a C or C++ caller holds anyway: the raw addresses of its arrays
        raw = [(x[0].ctypes.data, x[1].ctypes.data, x[2].ctypes.data if x[2] is not None else None, x[3].ctypes.data,
                x[4].output_size, x[4].index_size) for x in hb]
        host_submit = _capi.lib().fbgemm_b200_spmdm_host_submit
        cfg_ref = C.byref(kern.cfg)

        def submit(i):
            p_idx, p_off, p_w, p_out, osz, isz = raw[i % NUM_BATCHES]
            rc = host_submit(ctx.handle, i % lanes, cfg_ref, osz, isz, w.rows, host_key, p_idx, p_off, p_w, p_out, cit_key)
            if rc < 0:
                _capi.check(rc, "host_submit")

        host_s = [0.0, 0.0]   # host time inside submit / inside wait

        def run_calls(n):
            ok = True
            for i in range(n):
                if i >= lanes:
                    t = time.perf_counter()
                    ok = kern.host_wait(i % lanes) and ok
                    host_s[1] += time.perf_counter() - t
                t = time.perf_counter()
                submit(i)
                host_s[0] += time.perf_counter() - t
            for i in range(min(lanes, n)):
                ok = kern.host_wait((n + i) % lanes) and ok
            return ok

        e2e_steps = max(1, min(args.e2e_steps, steps))
        ok = run_calls(cps)   # warm-up step
        torch.cuda.synchronize()
        host_s[0] = host_s[1] = 0.0
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ok = run_calls(cps) and ok
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        # the rows that came back are the rows the device-pointer path produced
        idx, off, wts, out, b = hb[(cps - 1) % NUM_BATCHES]
        ok = ok and same_bits(out, outs[(cps - 1) % NUM_BATCHES].cpu().numpy())
        h2d = float(np.mean([x[0].nbytes + x[1].nbytes + (x[2].nbytes if x[2] is not None else 0) for x in hb]))
        d2h = float(np.mean([x[3].nbytes for x in hb])) + 16
        calls = e2e_steps * cps
        rec["e2e"] = {"value": bytes_per_call * calls / dt / 1e9, "unit": "GB/s",
                      "h2d_bytes_per_step": round(h2d * cps), "d2h_bytes_per_step": round(d2h * cps),
                      "steps": e2e_steps, "calls_per_step": cps, "ms_per_step": dt / e2e_steps * 1e3,
                      "ms_per_call": dt / calls * 1e3, "bags_per_s": bags_per_call * calls / dt, "results_ok": bool(ok),
                      "host_us_per_call": {"in_submit": host_s[0] / calls * 1e6, "blocked_in_wait": host_s[1] / calls * 1e6,
                                           "note": "one host thread issues every call; the time inside submit is checks, "
                                                   "pointer queries, one staging launch or three copies, the lookup, the "
                                                   "download and the status record.  Two or four submitting threads gave the "
                                                   "same rate, so the transfers bound the call, not this thread"},
                      "path": f"fbgemm_b200_spmdm_host_submit/wait, {lanes} pipelined lanes, pinned host buffers, table resident",
                      "timer": "host perf_counter bracketed by device synchronisation"}
        ctx.unregister_table(host_tbl)
        if host_cit is not None:
            ctx.unregister_table(host_cit)

    # ---- cpu_baseline ------------------------------------------------------------------
    rec["cpu_baseline"] = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        tbl = CpuTable(w.bit_rate, w.dim, w.rows, w.out_dtype == torch.float16, w.normalize_by_lengths,
                       w.table.cpu().numpy(), w.cit.cpu().numpy() if w.cit is not None else None, batches, w.row_bytes)
        r = time_cpu([tbl], threads, cps, 10 ** 9, args.cpu_seconds)
        r1 = time_cpu([tbl], 1, cps, 10 ** 9, min(3.0, args.cpu_seconds))
        rec["cpu_baseline"] = {
            "value": r["bytes"] / r["seconds"] / 1e9, "unit": "GB/s", "cores": threads, "kind": r["kind"],
            "sample": f"{r['calls']} whole batches in {r['seconds']:.1f} s after a warm-up, each split over {threads} "
                      f"host threads; {r['desc']}",
            "bags_per_s": r["bags"] / r["seconds"],
            "one_thread": {"value": r1["bytes"] / r1["seconds"] / 1e9, "unit": "GB/s",
                           "sample": f"{r1['calls']} whole batches in {r1['seconds']:.1f} s on one thread"}}
    return rec


def main_single(args):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=5))
    rec = run_single(args, args.workload, dev, rank, world, args.steps, args.warmup, full=True)
    ms, value, e2e = rec["timed_region_s"] * 1e3, rec["value"], rec.get("e2e")
    ok = rec["results_ok"]
    if world > 1:   # weak scaling: one table of the configuration per GPU, no exchange
        import torch.distributed as dist

        t = torch.tensor([ms, -float(ok), (e2e or {}).get("ms_per_step", 0.0)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ok = float(t[0]), float(t[1]) == -1.0
        value = rec["gathered_bytes_per_call"] * world * args.steps * rec["calls_per_step"] / (ms / 1e3) / 1e9
        if e2e:
            e2e["value"] = rec["gathered_bytes_per_call"] * world * e2e["calls_per_step"] / (float(t[2]) / 1e3) / 1e9
    if rank == 0:
        line = {
            "metric": "gathered_row_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": {0: "u8", 1: "u4", 2: "u2"}[args.workload] + "->f32 accumulate",
            "data": "synthetic",
            "config": {"workload": rec["workload"], "baseline_config_index": args.workload,
                       "calls_per_step": rec["calls_per_step"], "bags_per_call": rec["bags_per_call"],
                       "gathered_bytes_per_call": rec["gathered_bytes_per_call"], "row_bytes": rec["row_bytes"],
                       "table_MB": rec["table_MB"], "batches_per_call": args.group, "distinct_batches": NUM_BATCHES,
                       "launch": f"one CUDA graph of {rec['calls_per_step']} functor calls per step over {args.streams} streams",
                       "l2": "table (larger than the 126 MB L2) is the gathered input; calls rotate over distinct batches",
                       "sharding": "one table of this shape per GPU, no exchange" if world > 1 else "single table"},
            "results_ok": bool(ok), "results_check": rec["results_check"],
            "timed_region_s": ms / 1e3, "ms_per_call": rec["ms_per_call"],
            "ms_per_step_p10_p50_p90": rec["ms_per_step_p10_p50_p90"],
            "single_call_latency_us": rec.get("single_call_latency_us"),
            "bags_per_s": rec["bags_per_call"] * world * args.steps * rec["calls_per_step"] / (ms / 1e3),
            "all_bytes_GBps": rec["all_bytes_GBps"] * world, "clocks": rec["clocks"], "e2e": e2e,
            "gpu_launches": rec["gpu_launches"],
            "roofline": {"bound": "hbm", "achieved": rec["value"], "peak": rec["peak"], "unit": "GB/s",
                         "frac": rec["frac"], "traffic": rec["traffic"], "traffic_source": rec["traffic_source"],
                         "peak_source": rec["peak_source"],
                         "note": "achieved = gathered-row bytes per call / (timed region / calls), this rank; calls of "
                                 "different streams overlap; traffic = DRAM bytes per call from the ncu capture named"},
            "cpu_baseline": rec.get("cpu_baseline"),
        }
        emit(line)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


# ---- multi-table workloads (configurations 3 and 4) ----------------------------------

def multi_specs(args, world):
    """(specs, B, alpha, index dtype name, weighted, name, mean_len, costs)."""
    from fbgemm_b200 import workloads as W

    if args.workload == 3:
        specs = W.config3_tables(max(world, int(round(64 * args.tables_scale))), args.scale)
        return specs, int(16384 * args.batch_scale), 1.05, "int32", False, "mixed 8/4/2-bit", 30.0, "poisson"
    per_gpu = max(1, int(round(32 * args.tables_scale)))
    specs = W.config4_tables(per_gpu * world, args.scale)
    return specs, int(65536 * args.batch_scale), 1.1, "int64", True, "4-bit x128", 40.0, "fixed"


def make_input_sets(specs, tables, B, alpha, idt, weighted, mean_len, lengths_kind, dev, nsets):
    """``nsets`` global batches for the tables in ``tables``: sets[s][t] = Batch."""
    import torch

    from fbgemm_b200 import workloads as W

    tdt = torch.int32 if idt == "int32" else torch.int64
    perms = {t: W.row_permutation(specs[t].rows, dev, specs[t].seed + 5) for t in tables}
    sets = []
    for sidx in range(nsets):
        d = {}
        for t in tables:
            g = torch.Generator(device=dev).manual_seed(specs[t].seed + 77 * sidx)
            if lengths_kind == "poisson":
                lengths = torch.poisson(torch.full((B,), mean_len, device=dev), generator=g).to(torch.int64)
            else:
                lengths = torch.full((B,), int(mean_len), device=dev, dtype=torch.int64)
            off = W.offsets_from_lengths(lengths, tdt)
            n = int(off[-1])
            idx = W.zipf_indices(n, alpha, specs[t].rows, dev, specs[t].seed + 1000 + sidx, tdt, perms[t])
            wts = torch.rand(n, generator=g, device=dev) if weighted else None
            d[t] = W.Batch(idx, off, wts, B, n, n)
        sets.append(d)
    return sets


def main_multi(args):
    """Table-wise sharded multi-table lookup: every rank pools the global batch
    for the tables it owns and the kernels store the pooled rows batch-wise
    into the owning ranks' buffers.  One step = ``batches_per_step`` global
    batches over all tables, ordered between the ranks on the device."""
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
    from fbgemm_b200.sharding import ShardedLookup, TableWisePlan, expected_cost
    from oracle.checker import Oracle

    specs, B, alpha, idt, weighted, name, mean_len, lengths_kind = multi_specs(args, world)
    if args.shard:
        if args.workload != 3 or world != 1:
            raise SystemExit("--shard K/G sizes one rank's share of workload 3 on a single GPU")
        k, g = (int(x) for x in args.shard.split("/"))
        owner = TableWisePlan.balanced([expected_cost(s, B, mean_len) for s in specs], [s.dim for s in specs], g).owner
        specs = [s for t, s in enumerate(specs) if owner[t] == k]
        name += f", shard {k} of {g}"
    if args.workload == 3:
        plan = TableWisePlan.balanced([expected_cost(s, B, mean_len) for s in specs], [s.dim for s in specs], world)
    else:
        plan = TableWisePlan.balanced([1.0] * len(specs), [s.dim for s in specs], world)
    B -= B % world
    rows = B // world
    tnp = {"int32": np.int32, "int64": np.int64}[idt]
    p2p = args.redistribution == "p2p"
    nbuf = args.batches_in_flight if args.batches_in_flight > 0 else min(8, max(2, world))
    sl = ShardedLookup(specs, plan, rank, B, dev, torch.float16, mode=args.redistribution, num_buffers=nbuf,
                       weighted=weighted, index_dtype=tnp, offset_dtype=tnp)
    sets = make_input_sets(specs, sl.local, B, alpha, idt, weighted, mean_len, lengths_kind, dev, NUM_SETS)
    bytes_local = float(np.mean([sum(b.index_size * specs[t].row_bytes for t, b in d.items()) for d in sets]))
    # One lane per output buffer: its own stream (and side streams for the tables' launches), so that the counter
    # waits and the tail of one global batch overlap with the lookups of the next.
    lanes = [torch.cuda.Stream(device=dev) for _ in range(nbuf)]
    side = [[torch.cuda.Stream(device=dev) for _ in range(3)] for _ in range(nbuf)]
    bps = max(1, args.batches_per_step)

    plans = None
    if args.launch == "plan":   # one kernel launch per kernel variant instead of one per table
        plans = {(s, b): sl.make_plan(sets[s], buffer=b, slot=400 + s * nbuf + b) for s in range(NUM_SETS)
                 for b in range(nbuf)}
    launches_per_batch = (plans[(0, 0)].num_launches if plans else len(sl.local)) + (4 if p2p else 0)

    def make_step_calls(lookup):
        """One handle per output buffer that enqueues a whole ordered step with one call from the host, and its
        pointer arrays for every input set: the host side of a global batch is then a single C call."""
        if not (plans is None and lookup.local):
            return None, None
        calls_ = [lookup.make_step_call(b, slot=460 + b) for b in range(nbuf)]
        args_ = {s: calls_[0].device_args([sets[s][t].indices for t in lookup.local],
                                          [sets[s][t].offsets for t in lookup.local],
                                          [sets[s][t].weights for t in lookup.local] if weighted else None)
                 for s in range(NUM_SETS)}
        return calls_, args_

    step_calls, step_args = make_step_calls(sl)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
            torch.cuda.synchronize(dev)

    counter = [0]

    def global_batch():
        """One global batch: input set j % NUM_SETS into buffer j % 2, on that buffer's lane."""
        j = counter[0]
        counter[0] += 1
        s, b = j % NUM_SETS, j % nbuf
        with torch.cuda.stream(lanes[b]):
            streams = [lanes[b]] + side[b]
            if p2p and step_calls:
                # ack wait, the lookups over four streams, ready signal and wait, release: one call
                step_calls[b].step_device(step_args[s], True, lanes[b].cuda_stream)
            elif p2p:
                n = sl.step(sets[s], buffer=b, slot_base=(j % 4) * 100, streams=None if plans else streams,
                            plan=plans[(s, b)] if plans else None)
                sl.release(b, n)   # this benchmark's consumer has nothing to do with the rows
            else:
                if step_calls:
                    step_calls[b].step_device(step_args[s], False, lanes[b].cuda_stream)
                elif plans:
                    plans[(s, b)].launch(lanes[b].cuda_stream)
                else:
                    for st in side[b]:
                        st.wait_stream(lanes[b])
                    sl.launch(sets[s], buffer=b, slot_base=(j % 4) * 100, streams=[st.cuda_stream for st in streams])
                    for st in side[b]:
                        lanes[b].wait_stream(st)
                sl.exchange(b)
        return s, b

    def fork_lanes():
        cur = torch.cuda.current_stream()
        for ln in lanes:
            ln.wait_stream(cur)

    def join_lanes():
        cur = torch.cuda.current_stream()
        for ln in lanes:
            cur.wait_stream(ln)

    def status_ok():
        slots = list(range(400 + NUM_SETS * nbuf + 1)) + [460 + b for b in range(nbuf)]   # per-table, plans, step handles
        return all(F.status_read(s, dev.index)[0] for s in slots)

    # ---- parity inside the run: sampled bags of every table, on the rank that received them ----
    oracle = Oracle()
    rng = np.random.default_rng(777)
    sample = np.sort(rng.choice(B, min(PARITY_BAGS, B), replace=False))   # the same bags on every rank
    s0, b0 = global_batch()
    barrier()
    ok = status_ok()
    expected = {}
    for t in sl.local:
        bt = sets[s0][t]
        expected[t] = oracle_sample(oracle, specs[t].bit_rate, specs[t].dim, np.float16, sl.tables[t], None, bt.indices,
                                    bt.offsets, bt.weights, False, sample)
    if world > 1:
        import torch.distributed as dist

        gathered = [None] * world
        dist.all_gather_object(gathered, expected)
        expected = {}
        for d in gathered:
            expected.update(d)
    mine = [i for i, m in enumerate(sample) if rank * rows <= m < (rank + 1) * rows]
    got_rows = sl.out[b0][torch.from_numpy(sample[mine] - rank * rows).to(dev)].cpu().numpy() if mine else None
    values_ok = True
    for t in range(len(specs)):
        if mine:
            c0 = plan.column_start(t)
            values_ok = values_ok and same_bits(got_rows[:, c0:c0 + specs[t].dim], expected[t][mine])
    ok = ok and values_ok
    parity_rows = len(mine) * len(specs)

    # ---- value: inputs resident ------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        for _ in range(bps):
            global_batch()
    barrier()
    ok = ok and status_ok()
    before = F.launch_count()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(local_rank) as clocks:
        marks[0].record()
        fork_lanes()
        for k in range(args.steps):
            for _ in range(bps):
                global_batch()
            join_lanes()            # the step's mark waits for both lanes; the next step's batches follow without a gap
            marks[k + 1].record()
        torch.cuda.synchronize(dev)
    barrier()
    launches = int(F.launch_count() - before)
    ms = marks[0].elapsed_time(marks[args.steps])
    per_step_ms = sorted(marks[k].elapsed_time(marks[k + 1]) for k in range(args.steps))
    ok = ok and status_ok()

    # ---- host time to enqueue one global batch (nothing waited for: 8 batches fit the launch queue) ----
    barrier()
    fork_lanes()
    t_host = time.perf_counter()
    for _ in range(8):
        global_batch()
    enqueue_us = (time.perf_counter() - t_host) / 8 * 1e6
    join_lanes()
    barrier()
    ok = ok and status_ok()

    # ---- e2e: host index arrays in, this rank's [B/G, total_D] slice out --------------------
    e2e = None
    if not args.no_e2e and p2p and len(specs) >= world:
        sl_h = ShardedLookup(specs, plan, rank, B, dev, torch.float16, mode="p2p", num_buffers=nbuf, tables=sl.tables,
                             weighted=weighted, index_dtype=tnp, offset_dtype=tnp)
        caps = {t: max(sets[s][t].index_size for s in range(NUM_SETS)) for t in sl.local}
        calls = [sl_h.make_host_call(b, caps, slot=450 + b) for b in range(nbuf)]

        def host_views(arrays):
            """The arrays back to back in ONE page-locked block - how the reference's multi-table caller holds
            its indices, offsets and weights - and a view of the block per table."""
            if arrays[0] is None:
                return [None] * len(arrays)
            block = torch.empty(sum(a.numel() for a in arrays), dtype=arrays[0].dtype).pin_memory()
            views, at = [], 0
            for a in arrays:
                block[at:at + a.numel()].copy_(a)
                views.append(block[at:at + a.numel()].numpy())
                at += a.numel()
            return views

        host_sets = []
        for d in sets:
            cols = [host_views([getattr(d[t], name) for t in sl.local]) for name in ("indices", "offsets", "weights")]
            host_sets.append({t: (cols[0][k], cols[1][k], cols[2][k]) for k, t in enumerate(sl.local)})
        host_out = [torch.zeros((rows, plan.total_dim), dtype=torch.float16).pin_memory().numpy() for _ in range(nbuf)]

        def run_host(nb):
            good = True
            for j in range(nb):
                b = j % nbuf
                if j >= nbuf:
                    good = calls[b].wait()[0] and good
                hs = host_sets[j % NUM_SETS]
                calls[b].submit([hs[t][0] for t in sl.local], [hs[t][1] for t in sl.local],
                                [hs[t][2] for t in sl.local] if weighted else None, host_out[b])
            for j in range(nb, nb + min(nbuf, nb)):
                good = calls[j % nbuf].wait()[0] and good
            return good

        nb = max(nbuf, args.e2e_batches - args.e2e_batches % nbuf)
        good = run_host(nbuf * 2)    # warm-up
        barrier()
        t0 = time.perf_counter()
        good = run_host(nb) and good
        torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t0
        barrier()
        phases = np.mean([c.last_step_ms() for c in calls], axis=0)    # this rank's last timed step on each handle
        # one more step, untimed, on the input set whose sampled bags the oracle pooled above: the rows that come
        # back to the host are compared bit for bit
        hs = host_sets[s0]
        calls[0].submit([hs[t][0] for t in sl.local], [hs[t][1] for t in sl.local],
                        [hs[t][2] for t in sl.local] if weighted else None, host_out[0])
        good = calls[0].wait()[0] and good
        barrier()
        if mine:
            hb = host_out[0]
            for t in range(len(specs)):
                c0 = plan.column_start(t)
                good = good and same_bits(hb[sample[mine] - rank * rows][:, c0:c0 + specs[t].dim], expected[t][mine])
        h2d = float(np.mean([sum(a.nbytes for tup in hs.values() for a in tup if a is not None) for hs in host_sets]))
        d2h = float(host_out[0].nbytes + 16)
        red = torch.tensor([dt, -float(good), h2d, d2h], device=dev, dtype=torch.float64)
        if world > 1:
            import torch.distributed as dist

            mx = red[:2].clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            sm = red[2:].clone()
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            red = torch.cat([mx, sm])
        dt, good = float(red[0]), float(red[1]) == -1.0
        e2e = {"steps": nb / bps, "global_batches": nb, "ms_per_global_batch": dt / nb * 1e3,
               "ms_per_step": dt / nb * bps * 1e3, "unit": "GB/s",
               "h2d_bytes_per_step": round(float(red[2]) * bps), "d2h_bytes_per_step": round(float(red[3]) * bps),
               "results_ok": bool(good),
               "last_step_ms": {"uploads": float(phases[0]), "lookups_and_counters": float(phases[1]),
                                "download": float(phases[2]),
                                "note": "device time of the phases of rank 0's last step on each handle, averaged; "
                                        "the handles' phases overlap, so they add up to more than ms_per_global_batch"},
               "path": f"fbgemm_b200_multi_host_submit/wait on every rank, {nbuf} pipelined handles, per-table views of "
                       "one pinned indices, one offsets (and one weights) array per step: those go up, lookups with peer stores, ready/ack counters, "
                       "the rank's [B/G, total_D] slice down; tables resident",
               "timer": "host perf_counter bracketed by barriers and device synchronisation, max over ranks"}
        for c in calls:
            c.close()
        del sl_h, host_sets, host_out

    # ---- the same steps with no store leaving the GPU, and with every store leaving it (what the peer stores cost) ----
    peer_ab = None
    if args.peer_ab and p2p and world > 1:
        import torch.distributed as dist

        sl_main, main_calls, main_args = sl, step_calls, step_args
        peer_ab = {}
        for key, route in (("local_only_ms_per_global_batch", True), ("all_to_next_rank_ms_per_global_batch", "next")):
            sl = ShardedLookup(specs, plan, rank, B, dev, torch.float16, mode="p2p", num_buffers=nbuf,
                               tables=sl_main.tables, weighted=weighted, index_dtype=tnp, offset_dtype=tnp,
                               route_local=route)
            step_calls, step_args = make_step_calls(sl)
            for _ in range(3 * bps):
                global_batch()
            barrier()
            m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            m0.record()
            fork_lanes()
            for _ in range(args.steps * bps):
                global_batch()
            join_lanes()
            m1.record()
            torch.cuda.synchronize(dev)
            barrier()
            t_ms = torch.tensor([m0.elapsed_time(m1)], device=dev, dtype=torch.float64)
            dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
            peer_ab[key] = float(t_ms) / (args.steps * bps)
        sl, step_calls, step_args = sl_main, main_calls, main_args

    # ---- reduce over ranks ---------------------------------------------------------------------
    red = torch.tensor([ms, -float(ok)], device=dev, dtype=torch.float64)
    tot = torch.tensor([bytes_local, float(launches), float(parity_rows)], device=dev, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(red, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms, ok = float(red[0]), float(red[1]) == -1.0
    job_bytes, launches, parity_rows = float(tot[0]), int(tot[1]), int(tot[2])
    sec = ms / 1e3
    nbatches = args.steps * bps
    peak, peak_src = measured_peak()
    value = job_bytes * nbatches / sec / 1e9
    if e2e:
        e2e["value"] = job_bytes * e2e["global_batches"] / (e2e["ms_per_global_batch"] * e2e["global_batches"] / 1e3) / 1e9
        e2e["bags_per_s"] = len(specs) * B / (e2e["ms_per_global_batch"] / 1e3)

    # ---- cpu_baseline (one GPU only): the reference's kernels on a sample of the tables -----------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        pick = sl.local[:: max(1, len(sl.local) // 3)][:3]
        tabs = [CpuTable(specs[t].bit_rate, specs[t].dim, specs[t].rows, True, False, sl.tables[t].cpu().numpy(), None,
                         [sets[s][t] for s in range(NUM_SETS)], specs[t].row_bytes) for t in pick]
        r = time_cpu(tabs, threads, len(pick) * bps, 10 ** 9, args.cpu_seconds)
        cpu = {"value": r["bytes"] / r["seconds"] / 1e9, "unit": "GB/s", "cores": threads, "kind": r["kind"],
               "bags_per_s": r["bags"] / r["seconds"],
               "sample": f"tables {pick} of {len(specs)}: {r['calls']} whole-table batches of {B} bags in "
                         f"{r['seconds']:.1f} s after a warm-up, every batch split over {threads} host threads; "
                         f"{r['desc']}; stands for the whole table set by gathered bytes"}
        del tabs

    # ---- the single-table configurations as sub-records (one GPU only) ------------------------------
    single = None
    if world == 1 and not args.no_single and args.workload == 3:
        sets = None
        torch.cuda.empty_cache()
        single = [run_single(args, c, dev, rank, world, max(40, args.steps), 3, full=False) for c in (0, 1, 2)]

    if rank == 0:
        traffic = TRAFFIC.get(args.workload)
        traffic_ok = (traffic and args.scale == 1.0 and args.tables_scale == 1.0 and args.batch_scale == 1.0
                      and not args.shard)
        emit(({
            "metric": "gathered_row_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if args.workload == 3 else "weak", "vs_baseline": None,
            "dtype": "u8/u4/u2->f32 accumulate", "data": "synthetic",
            "config": {"workload": f"{len(specs)} tables {name}, table-wise over {world} GPU(s), batch {B} per table",
                       "baseline_config_index": args.workload, "tables": len(specs), "total_dim": plan.total_dim,
                       "batches_per_step": bps, "calls_per_step": bps * len(specs),
                       "bags_per_step": bps * len(specs) * B, "gathered_bytes_per_step": round(job_bytes * bps),
                       "distinct_input_sets": NUM_SETS,
                       "rows_scale": args.scale, "tables_scale": args.tables_scale, "batch_scale": args.batch_scale,
                       "table_GB_this_rank": round(sum(t.numel() for t in sl.tables.values()) / 1e9, 2),
                       "redistribution": ("pooled rows stored by the lookup kernels into the owning rank's buffer (peer "
                                          "stores), ready/ack counters between the ranks on the device" if p2p else
                                          "NCCL all_to_all_single after the lookups"),
                       "launch": (f"multi-table plan, {launches_per_batch} kernel launches per global batch" if plans else
                                  f"one launch per table over 4 streams ({launches_per_batch} kernel launches per "
                                  "global batch and rank, counters included)") + f"; {nbuf} global batches in flight, "
                                 "one per output buffer",
                       "l2": "tables are far larger than L2; the input sets rotate"},
            "results_ok": bool(ok),
            "results_check": f"{parity_rows} pooled rows (sampled bags x all tables, each on the rank whose buffer "
                             "received it, rows stored by peers included) bit-equal to the CPU oracle; no lookup or "
                             "counter wait reported an error",
            "timed_region_s": sec, "ms_per_global_batch": ms / nbatches,
            "ms_per_step_p10_p50_p90": [pctl(per_step_ms, 0.1), pctl(per_step_ms, 0.5), pctl(per_step_ms, 0.9)],
            "bags_per_s": len(specs) * B * nbatches / sec,
            "frac_of_hbm_peak": value / world / peak, "clocks": clocks.summary(),
            "gpu_launches": launches,
            "host_enqueue_us_per_global_batch": enqueue_us,
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak,
                         "traffic": traffic["bytes_per_global_batch"] / world if traffic_ok else None,
                         "traffic_source": traffic["source"] if traffic_ok else None, "peak_source": peak_src,
                         "note": "per GPU: gathered-row bytes of one global batch / device time per global batch (the "
                                 "tables' launches overlap on 4 streams); traffic = DRAM bytes of all lookup kernels of "
                                 "one global batch per GPU"},
            "e2e": e2e, "cpu_baseline": cpu, "single_table": single,
            "peer_store_ab": dict(peer_ab, peer_stores_ms_per_global_batch=ms / nbatches,
                                  note="the same lookups, counters and launch order with every pooled row stored into the "
                                       "rank's own buffer (no store crosses NVLink), with every row stored into the next "
                                       "rank's buffer (all of them cross it), and with the benchmark's routing, where "
                                       "(N-1)/N of each rank's rows are peer stores") if peer_ab else None}))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


# ---- the kernels either side of the pooled lookup (--workload 5) -------------------------------

def _caller_time(fn, iters, warm=3):
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    ev[0].record()
    for i in range(iters):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    ts = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(iters))
    return ts[len(ts) // 2] * 1e-3


def pruning_lookups(res, which, iters, dev):
    import torch

    import fbgemm_b200 as F
    from fbgemm_b200 import tbe

    rng = np.random.default_rng(5)
    T, B, E = 16, 16384, 4_000_000
    lengths = rng.poisson(30, T * B)
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    n = int(offsets[-1])
    indices = rng.integers(0, E, n).astype(np.int32)
    want = np.where(indices % 2 == 0, indices // 2, -1)   # the even sparse indices are the rows that were kept
    for idt, mdt in ((np.int32, np.int32), (np.int64, np.int64)):
        ib, mb = np.dtype(idt).itemsize, np.dtype(mdt).itemsize
        keys = np.arange(0, E, 2, dtype=idt)
        dense = np.arange(len(keys), dtype=idt)
        d_idx = torch.from_numpy(indices.astype(idt)).to(dev)
        d_off = torch.from_numpy(offsets.astype(idt)).to(dev)
        if which in (None, "hashmap"):
            cap = int(len(keys) / 0.8) + 1
            hto = np.arange(T + 1, dtype=np.int64) * cap
            table = np.full((T * cap, 2), -1, dtype=mdt)
            assert tbe.pruned_hashmap_insert(
                torch.from_numpy(np.tile(keys, T)), torch.from_numpy(np.tile(dense, T)),
                torch.from_numpy((np.arange(T + 1, dtype=np.int64) * len(keys)).astype(idt)), torch.from_numpy(table),
                torch.from_numpy(hto))
            d_tab, d_hto = torch.from_numpy(table).to(dev), torch.from_numpy(hto).to(dev)
            assert (tbe.pruned_hashmap_lookup(d_idx, d_off, d_tab, d_hto).cpu().numpy() == want).all()
            dt = _caller_time(lambda: tbe.pruned_hashmap_lookup(d_idx, d_off, d_tab, d_hto), iters)
            res[f"pruned_hashmap_lookup_index{ib * 8}_table{mb * 8}"] = {
                "positions": n, "us": round(dt * 1e6, 1), "Gpositions_s": round(n / dt / 1e9, 2),
                "alg_GBs": round(n * (2 * ib + 2 * mb) / dt / 1e9, 1), "table_MB": round(table.nbytes / 1e6)}
            del d_tab
        if which in (None, "array"):
            remap = np.full(T * E, -1, dtype=mdt)
            for t in range(T):
                remap[t * E:(t + 1) * E:2] = dense
            d_remap = torch.from_numpy(remap).to(dev)
            d_ro = torch.from_numpy(np.arange(T + 1, dtype=np.int64) * E).to(dev)
            assert (tbe.pruned_array_lookup(d_idx, d_off, d_remap, d_ro).cpu().numpy() == want).all()
            dt = _caller_time(lambda: tbe.pruned_array_lookup(d_idx, d_off, d_remap, d_ro), iters)
            res[f"pruned_array_lookup_index{ib * 8}_map{mb * 8}"] = {
                "positions": n, "us": round(dt * 1e6, 1), "Gpositions_s": round(n / dt / 1e9, 2),
                "alg_GBs": round(n * (2 * ib + mb) / dt / 1e9, 1), "map_MB": round(remap.nbytes / 1e6)}
            del d_remap


def sequence_lookup(res, iters, dev):
    import torch

    import fbgemm_b200 as F
    from fbgemm_b200 import tbe

    rng = np.random.default_rng(6)
    T, rows, D, B = 8, 2_000_000, 128, 32768
    for ty, name in ((tbe.SparseType.INT4, "int4"), (tbe.SparseType.INT8, "int8"), (tbe.SparseType.FP16, "fp16")):
        for out_ty, oname, ob in ((tbe.SparseType.FP16, "f16", 2), (tbe.SparseType.FP32, "f32", 4)):
            rb = tbe.padded_row_size_in_bytes(D, ty, 16)
            w = torch.randint(0, 256, (T * rows * rb,), dtype=torch.uint8, device=dev)
            lengths = rng.poisson(16, T * B)
            off = torch.from_numpy(np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)).to(dev)
            n = int(lengths.sum())
            idx = torch.randint(0, rows, (n,), dtype=torch.int32, device=dev)
            op = tbe.IntNBitSequenceEmbedding(w, [t * rows * rb for t in range(T)], [int(ty)] * T, D, 16, out_ty)
            out = torch.zeros((n, D), dtype=op.out_dtype, device=dev)
            dt = _caller_time(lambda: op.forward(idx, off, out), iters)
            assert F.status_read(0)[0]
            res[f"sequence_lookup_{name}_to_{oname}"] = {
                "positions": n, "us": round(dt * 1e6, 1), "alg_GBs": round(n * (rb + D * ob + 4) / dt / 1e9, 1),
                "row_bytes": rb, "out_row_bytes": D * ob}
            del w, out


def index_remap(res, iters, dev):
    import torch

    import fbgemm_b200 as F
    from fbgemm_b200 import tbe

    rng = np.random.default_rng(7)
    lengths = rng.poisson(30, 262144)
    off = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    n, U = int(off[-1]), 20_000_000
    mapping = np.where(rng.random(U) < 0.5, -1, 1).astype(np.int32)
    mapping[mapping > 0] = np.arange(int((mapping > 0).sum()), dtype=np.int32)
    d_map, d_off = torch.from_numpy(mapping).to(dev), torch.from_numpy(off).to(dev)
    d_idx = torch.randint(0, U, (n,), dtype=torch.int32, device=dev)
    d_w = torch.rand(n, device=dev)
    dt = _caller_time(lambda: F.compressed_indices_remap(d_idx, d_map, d_off, d_w), iters)
    res["compressed_indices_remap_weighted"] = {
        "positions": n, "us": round(dt * 1e6, 1), "Gpositions_s": round(n / dt / 1e9, 2),
        "alg_GBs": round(n * (4 + 4 + 4 + 0.5 * 8) / dt / 1e9, 1), "launches": 4,
        "note": "includes the status read-back the call waits for"}


def main_callers(args):
    """Timing of the pruning lookups, ``compressed_indices_remap`` and the
    sequence ("nobag") lookup on seeded synthetic inputs: CUDA events around
    each call on torch's current stream, median of ``--caller-iters`` calls
    after 3 warm-up calls.  ``alg_GBs`` counts the bytes a call has to move once
    (indices, one hash slot or map entry, the row, the output row), not the
    sectors it touches.  Shapes: 16 tables x 16384 bags x Poisson(30) indices
    with half of the keys present at a hash-table load factor of 0.8; 8 tables
    of 2 M rows x D = 128 and 32768 bags x Poisson(16) per table for the
    sequence lookup; 262144 bags x Poisson(30) over a 20 M-row map, half
    pruned, for the remap."""
    import torch

    dev = torch.device("cuda:0")
    res = {}
    only = args.callers_only
    if only in (None, "hashmap", "array"):
        pruning_lookups(res, only, args.caller_iters, dev)
    if only in (None, "sequence"):
        sequence_lookup(res, args.caller_iters, dev)
    if only in (None, "remap"):
        index_remap(res, args.caller_iters, dev)
    emit(({"metric": "caller_kernel_times", "unit": "us per call (median)", "n_gpus": 1, "data": "synthetic",
                      "config": {"workload": "pruning lookups, index remap and sequence lookup", "iters": args.caller_iters},
                      "records": res}))
    return 0


# ---- the reference arm: the reference's CPU path on the same configuration ---------------------

def reference_table(spec_bits, rows, dim, seed, dev):
    """The table of ``random_table`` (same seeded N(0,1) rows, drawn with torch
    on ``dev``), quantized on the host by the REFERENCE's own quantizers
    (FloatOrHalfToFused8BitRowwiseQuantizedSBFloat /
    FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf, src/QuantUtils.cc:534-718 of
    FBGEMM) over all host threads."""
    from concurrent.futures import ThreadPoolExecutor

    from fbgemm_b200 import workloads as W
    from oracle import checker

    ref = checker.Reference()
    quant = (lambda x: ref.quantize_8bit(x, use_ref=False)) if spec_bits == 8 else \
        (lambda x: ref.quantize_nbit(spec_bits, x, use_ref=False))
    if not ref.available:
        o = checker.Oracle()
        quant = o.quantize_8bit if spec_bits == 8 else (lambda x: o.quantize_nbit(spec_bits, x))
    out = np.empty((rows, W.fused_row_bytes(spec_bits, dim)), dtype=np.uint8)
    threads = os.cpu_count() or 1
    with ThreadPoolExecutor(max_workers=threads) as pool:
        for r0, x in W.random_rows(rows, dim, dev, seed):
            xh = x.cpu().numpy()
            cuts = [len(xh) * i // threads for i in range(threads + 1)]
            futs = [pool.submit(quant, xh[cuts[i]:cuts[i + 1]]) for i in range(threads) if cuts[i + 1] > cuts[i]]
            at = r0
            for f in futs:
                q = f.result()
                out[at:at + len(q)] = q
                at += len(q)
    return out


def main_reference(args):
    """``--impl reference``: the reference's CPU kernels on this box's host
    cores, same configuration, metric and step definition; rank 0 alone."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    import torch

    from fbgemm_b200 import workloads as W   # input generators only: the product library is never loaded here

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else torch.device("cpu")
    threads = os.cpu_count() or 1
    if args.workload in (0, 1, 2):
        maker = W.CONFIGS[args.workload]
        w = maker(dev, scale=args.scale, seed=W.SEED, table_maker=lambda r, d, b, device, s: torch.from_numpy(
            reference_table(b, r, d, s, device)))
        batches = [w.make_batch(s) for s in range(NUM_BATCHES)]
        tabs = [CpuTable(w.bit_rate, w.dim, w.rows, w.out_dtype == torch.float16, w.normalize_by_lengths,
                         w.table.numpy(), w.cit.cpu().numpy() if w.cit is not None else None, batches, w.row_bytes)]
        cps = max(1, args.calls_per_step)
        config = {"workload": w.name, "baseline_config_index": args.workload, "calls_per_step": cps,
                  "bags_per_call": batches[0].output_size, "row_bytes": w.row_bytes, "distinct_batches": NUM_BATCHES}
        sample = "the whole configuration"
        dtype = {0: "u8", 1: "u4", 2: "u2"}[args.workload] + "->f32 accumulate"
        scaling = "weak"
    else:
        specs, B, alpha, idt, weighted, name, mean_len, lengths_kind = multi_specs(args, 1)
        pick = list(range(len(specs)))[:: max(1, len(specs) // 3)][:3]
        tables = {t: reference_table(specs[t].bit_rate, specs[t].rows, specs[t].dim, specs[t].seed, dev) for t in pick}
        sets = make_input_sets(specs, pick, B, alpha, idt, weighted, mean_len, lengths_kind, dev, NUM_SETS)
        tabs = [CpuTable(specs[t].bit_rate, specs[t].dim, specs[t].rows, True, False, tables[t], None,
                         [sets[s][t] for s in range(NUM_SETS)], specs[t].row_bytes) for t in pick]
        cps = len(pick) * max(1, args.batches_per_step)
        config = {"workload": f"{len(specs)} tables {name}, batch {B} per table", "baseline_config_index": args.workload,
                  "tables": len(specs), "batches_per_step": args.batches_per_step, "calls_per_step": cps}
        sample = (f"tables {pick} of {len(specs)} at full size stand for the table set by gathered bytes: a step is "
                  f"{args.batches_per_step} batches of {B} bags of each of them")
        dtype = "u8/u4/u2->f32 accumulate"
        scaling = "strong" if args.workload == 3 else "weak"
    r = time_cpu(tabs, threads, cps, max(1, args.steps), 240.0, warmup_steps=max(1, args.warmup))
    gbs = r["bytes"] / r["seconds"] / 1e9
    emit(({
        "impl": "reference", "metric": "gathered_row_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": r["steps"], "warmup": max(1, args.warmup), "ms_per_step": r["seconds"] / max(r["steps"], 1) * 1e3,
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": config, "bags_per_s": r["bags"] / r["seconds"], "timed_region_s": r["seconds"],
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": r["kind"],
                         "sample": f"{sample}; {r['calls']} whole batches in {r['seconds']:.1f} s after {max(1, args.warmup)} "
                                   f"warm-up steps, each batch split over {threads} host threads; {r['desc']}; tables "
                                   "quantized by the reference's own quantizers from the seeded N(0,1) rows"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
    return 0


def relaunch_with_ranks(args) -> None:
    """``python bench.py --gpus N`` without a launcher: run the same command line
    as N ranks of one node (what ``python -m torch.distributed.run
    --nproc-per-node N bench.py --gpus N`` does) and leave with its exit code.
    The launcher picks its own free port (``--standalone``)."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
           f"--nproc-per-node={args.gpus}", os.path.abspath(__file__), *sys.argv[1:]]
    os.execv(sys.executable, cmd)


def main():
    args = parse_args()
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        relaunch_with_ranks(args)
    claim_stdout()
    if args.impl == "reference":
        return main_reference(args)
    import torch

    if not torch.cuda.is_available():
        emit(({"error": "no CUDA device: fbgemm_b200 has no CPU path"}))
        return 1
    if args.workload == 5:
        return main_callers(args)
    return main_multi(args) if args.workload in (3, 4) else main_single(args)


if __name__ == "__main__":
    sys.exit(main())

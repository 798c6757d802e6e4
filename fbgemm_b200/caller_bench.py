"""Timing of the kernels either side of the pooled lookup - the pruning
lookups, ``compressed_indices_remap`` and the sequence ("nobag") lookup - on
seeded synthetic inputs, one JSON object on stdout:

    python -m fbgemm_b200.caller_bench [--only hashmap|array|sequence|remap] [--iters N]

CUDA events around each call on torch's current stream, median of ``iters``
calls after 3 warm-up calls.  ``alg_GBs`` counts the bytes a call has to move
once (indices, one hash slot or map entry, the row, the output row), not the
sectors it touches.  Shapes: 16 tables x 16384 bags x Poisson(30) indices with
half of the keys present at a hash-table load factor of 0.8; 8 tables of 2 M
rows x D = 128 and 32768 bags x Poisson(16) per table for the sequence lookup;
262144 bags x Poisson(30) over a 20 M-row map, half pruned, for the remap.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

import fbgemm_b200 as F
from fbgemm_b200 import tbe


def _time(fn, iters, warm=3):
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
            dt = _time(lambda: tbe.pruned_hashmap_lookup(d_idx, d_off, d_tab, d_hto), iters)
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
            dt = _time(lambda: tbe.pruned_array_lookup(d_idx, d_off, d_remap, d_ro), iters)
            res[f"pruned_array_lookup_index{ib * 8}_map{mb * 8}"] = {
                "positions": n, "us": round(dt * 1e6, 1), "Gpositions_s": round(n / dt / 1e9, 2),
                "alg_GBs": round(n * (2 * ib + mb) / dt / 1e9, 1), "map_MB": round(remap.nbytes / 1e6)}
            del d_remap


def sequence_lookup(res, iters, dev):
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
            dt = _time(lambda: op.forward(idx, off, out), iters)
            assert F.status_read(0)[0]
            res[f"sequence_lookup_{name}_to_{oname}"] = {
                "positions": n, "us": round(dt * 1e6, 1), "alg_GBs": round(n * (rb + D * ob + 4) / dt / 1e9, 1),
                "row_bytes": rb, "out_row_bytes": D * ob}
            del w, out


def index_remap(res, iters, dev):
    rng = np.random.default_rng(7)
    lengths = rng.poisson(30, 262144)
    off = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    n, U = int(off[-1]), 20_000_000
    mapping = np.where(rng.random(U) < 0.5, -1, 1).astype(np.int32)
    mapping[mapping > 0] = np.arange(int((mapping > 0).sum()), dtype=np.int32)
    d_map, d_off = torch.from_numpy(mapping).to(dev), torch.from_numpy(off).to(dev)
    d_idx = torch.randint(0, U, (n,), dtype=torch.int32, device=dev)
    d_w = torch.rand(n, device=dev)
    dt = _time(lambda: F.compressed_indices_remap(d_idx, d_map, d_off, d_w), iters)
    res["compressed_indices_remap_weighted"] = {
        "positions": n, "us": round(dt * 1e6, 1), "Gpositions_s": round(n / dt / 1e9, 2),
        "alg_GBs": round(n * (4 + 4 + 4 + 0.5 * 8) / dt / 1e9, 1), "launches": 4,
        "note": "includes the status read-back the call waits for"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", choices=["hashmap", "array", "sequence", "remap"], default=None)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("fbgemm_b200.caller_bench needs a GPU")
    dev = torch.device("cuda:0")
    res = {}
    if args.only in (None, "hashmap", "array"):
        pruning_lookups(res, args.only, args.iters, dev)
    if args.only in (None, "sequence"):
        sequence_lookup(res, args.iters, dev)
    if args.only in (None, "remap"):
        index_remap(res, args.iters, dev)
    print(json.dumps(res))


if __name__ == "__main__":
    main()

"""Generates tests/golden/tbe_golden.npz from the REFERENCE's own table-batched
CPU operator and pruning lookups.

Run where the reference tree is available: oracle/Makefile (target ``tbe``)
renders the reference's template
fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp
and compiles it into oracle/_ref/libfbgemm_tbe_ref.so.

    python tests/golden/make_golden_tbe.py

Cases (seeded inputs and the reference's outputs):

* ``hash{i}_*``   pruned_hashmap_insert_unweighted_cpu then
                  pruned_hashmap_lookup_unweighted_cpu: int32/int64 indices x
                  int32/int64 tables, a table without a hash map, keys that
                  were never inserted, negative keys;
* ``arr{i}_*``    pruned_array_lookup_cpu: int32/int64 indices x int32/int64
                  arrays, one table without an array;
* ``op{i}_*``     int_nbit_split_embedding_codegen_forward_{unweighted,weighted}_cpu
                  over INT8/INT4/INT2 (and FP32/FP16/FP8) tables, both row
                  layouts, FP32/FP16/BF16 output, SUM and MEAN pooling;
* ``seq{i}_*``    int_nbit_split_embedding_nobag_codegen_forward_unweighted_cpu.

The fixture pins the CPU oracle (tests/test_oracle.py,
tests/test_pruned_lookup_cpu.py) and the CUDA kernels
(tests/test_pruned_lookup_gpu.py, tests/test_tbe_gpu.py,
tests/test_sequence_gpu.py); it travels with the repository, the reference tree
does not.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import build_op_inputs, pruning_case  # noqa: E402
from oracle import checker  # noqa: E402

# SparseType / PoolingMode values (fbgemm_gpu/include/fbgemm_gpu/embedding_common.h:20-34)
FP32, FP16, INT8, INT4, INT2, BF16, FP8 = range(7)
SUM, MEAN, NONE = range(3)
OUT_NP = {FP32: np.float32, FP16: np.uint16, BF16: np.uint16}


def main():
    if not os.path.exists(checker.TBE_SO):
        checker.build(("tbe",), checker.reference_root())
    ref = checker.ReferenceTbe()
    assert ref.available
    rng = np.random.default_rng(20260202)
    out = {}

    # ---- hash-map pruning -------------------------------------------------------
    n = 0
    for idt in (np.int32, np.int64):
        for hdt in (np.int32, np.int64):
            for T, B, max_len, lf, unpruned in ((1, 3, 6, 0.8, ()), (4, 9, 8, 0.8, (1,)), (3, 30, 10, 0.97, ())):
                indices, dense, offsets, table, hto = pruning_case(rng, T, B, max_len, idt, hdt, lf, unpruned)
                ref.pruned_hashmap_insert(T, B, indices, dense, offsets, table, hto)
                probe = indices.copy()   # a mix: inserted keys, keys never inserted, negative keys
                r = rng.random(len(probe))
                probe[r < 0.2] = np.iinfo(np.int32).max - rng.integers(0, 1000, int((r < 0.2).sum()))
                probe[r > 0.9] = -rng.integers(1, 50, int((r > 0.9).sum()))
                k = f"hash{n}_"
                out[k + "meta"] = np.array([T, B], dtype=np.int64)
                out[k + "indices"], out[k + "dense"], out[k + "offsets"] = indices, dense, offsets
                out[k + "hto"], out[k + "table"] = hto, table
                out[k + "lookup"] = ref.pruned_hashmap_lookup(T, B, indices, offsets, table, hto)
                out[k + "probe"] = probe
                out[k + "probe_lookup"] = ref.pruned_hashmap_lookup(T, B, probe, offsets, table, hto)
                n += 1
    out["n_hash"] = np.array(n)

    # ---- array pruning ----------------------------------------------------------
    m = 0
    for idt in (np.int32, np.int64):
        for rdt in (np.int32, np.int64):
            T, B = 4, 12
            lengths = rng.integers(0, 9, size=T * B)
            offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(idt)
            sizes = [50, 0, 200, 7]
            ro = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
            remap = rng.integers(-1, 40, size=int(ro[-1])).astype(rdt)
            indices = np.zeros(int(offsets[-1]), dtype=idt)
            for t in range(T):
                lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
                indices[lo:hi] = rng.integers(0, sizes[t] if sizes[t] else 1000, hi - lo)
            k = f"arr{m}_"
            out[k + "meta"] = np.array([T, B], dtype=np.int64)
            out[k + "indices"], out[k + "offsets"], out[k + "remap"], out[k + "ro"] = indices, offsets, remap, ro
            out[k + "lookup"] = ref.pruned_array_lookup(T, B, indices, offsets, remap, ro)
            m += 1
    out["n_arr"] = np.array(m)

    # ---- pooled operator ----------------------------------------------------------
    q = 0
    quant = ([INT4, INT8, INT2, INT4, INT8], [64, 128, 128, 32, 24], [120, 90, 100, 60, 40])
    mixed = ([FP16, INT4, FP32, FP8], [64, 64, 24, 36], [70, 60, 40, 50])
    for tys, dims, rows in (quant, mixed):
        for scale_bias_last in (False, True):
            for out_ty in (FP32, FP16, BF16):
                for weighted, pooling in ((False, SUM), (True, MEAN)):
                    if tys is mixed[0] and (not scale_bias_last or out_ty == BF16):
                        continue
                    idt = np.int32 if out_ty != FP32 else np.int64
                    B = 7
                    tables, blob, w_off, D_off, offsets, indices, weights = build_op_inputs(
                        rng, tys, dims, rows, B, 6, 16, scale_bias_last, idt, prune=FP8 not in tys)
                    total_D = int(D_off[-1])
                    res = ref.forward(blob, w_off, tys, D_off, total_D, indices, offsets, B, pooling, 16,
                                      weights if weighted else None, out_ty, scale_bias_last, False, 5, 15,
                                      (B, total_D), OUT_NP[out_ty])
                    k = f"op{q}_"
                    out[k + "meta"] = np.array([B, int(scale_bias_last), out_ty, int(weighted), pooling, 16], dtype=np.int64)
                    out[k + "tys"], out[k + "dims"], out[k + "rows"] = np.array(tys), np.array(dims), np.array(rows)
                    out[k + "blob"], out[k + "w_off"], out[k + "D_off"] = blob, w_off, D_off
                    out[k + "indices"], out[k + "offsets"], out[k + "weights"] = indices, offsets, weights
                    out[k + "out"] = res
                    q += 1
    out["n_op"] = np.array(q)

    # ---- sequence operator ----------------------------------------------------------
    s = 0
    for tys, D, rows in (([INT4, INT8, INT2], 64, [80, 50, 70]), ([FP16, INT8, FP32], 24, [40, 30, 20])):
        for scale_bias_last in (False, True):
            for out_ty in (FP32, FP16, BF16):
                if FP16 in tys and not scale_bias_last:
                    continue
                B = 5
                tables, blob, w_off, D_off, offsets, indices, _ = build_op_inputs(
                    rng, tys, [D] * len(tys), rows, B, 4, 16, scale_bias_last, np.int32)
                res = ref.forward(blob, w_off, tys, None, D, indices, offsets, B, NONE, 16, None, out_ty,
                                  scale_bias_last, True, -1, -1, (len(indices), D), OUT_NP[out_ty])
                k = f"seq{s}_"
                out[k + "meta"] = np.array([B, int(scale_bias_last), out_ty, D, 16], dtype=np.int64)
                out[k + "tys"], out[k + "rows"] = np.array(tys), np.array(rows)
                out[k + "blob"], out[k + "w_off"] = blob, w_off
                out[k + "indices"], out[k + "offsets"] = indices, offsets
                out[k + "out"] = res
                s += 1
    out["n_seq"] = np.array(s)

    path = os.path.join(HERE, "tbe_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes;", n, "hash-map,", m, "array,", q, "operator,", s, "sequence cases")


if __name__ == "__main__":
    main()

"""Generates tests/golden/lookup_golden.npz from the REFERENCE's own code.

Run where the reference tree is available (it is compiled into
oracle/_ref/libfbgemm_ref.so by oracle/Makefile):

    python tests/golden/make_golden.py

Every case holds seeded inputs and the outputs of the reference's scalar
functions (fbgemm::EmbeddingSpMDM_ref, EmbeddingSpMDMNBit_ref,
EmbeddingSpMDM[NBit]RowWiseSparse_ref, the two ...Ref quantizers and
compressed_indices_remap_ref).  The fixture pins both the CPU oracle
(tests/test_oracle.py) and the CUDA kernels (tests/test_golden_gpu.py); it
travels with the repository, the reference tree does not.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import lengths_indices_weights, mapping_table, random_fused_table  # noqa: E402
from oracle import checker  # noqa: E402


def main():
    if not os.path.exists(checker.REF_SO):
        checker.build(("ref",))
    ref = checker.Reference()
    assert ref.available
    rng = np.random.default_rng(20260101)
    out = {}
    n = 0
    # pooled lookups: (bit_rate, batch, rows, dim, avg_len)
    shapes = [(8, 10, 400, 128, 20), (8, 7, 300, 40, 9), (8, 5, 50, 7, 6), (4, 12, 500, 64, 30), (4, 6, 200, 86, 8),
              (4, 4, 64, 8, 4), (2, 9, 400, 128, 25), (2, 5, 100, 36, 7), (2, 3, 40, 16, 5)]
    for bit_rate, batch, rows, dim, avg_len in shapes:
        for variant in range(4):
            idt = (np.int32, np.int64)[variant % 2]
            odt = (np.int64, np.int32)[variant // 2]
            weighted = variant in (1, 2)
            positional = variant == 2
            normalize = variant in (2, 3)
            use_offsets = variant != 3
            out_dt = (np.float32, np.float16)[variant % 2]
            table = random_fused_table(rng, rows, dim, bit_rate)
            lengths, offsets, indices, weights, cnt = lengths_indices_weights(rng, batch, rows, avg_len, idt, odt)
            if positional:
                weights = rng.standard_normal(int(lengths.max()) + 1).astype(np.float32)
            ol = offsets if use_offsets else lengths
            ok, res = ref.spmdm(bit_rate, dim, rows, table, indices, ol, weights if weighted else None, normalize,
                                out_dt, positional, use_offsets, output_size=batch, index_size=cnt)
            assert ok
            k = f"lookup{n}_"
            out[k + "meta"] = np.array([bit_rate, batch, rows, dim, int(weighted), int(positional), int(normalize),
                                        int(use_offsets)], dtype=np.int64)
            out[k + "table"] = table
            out[k + "indices"] = indices
            out[k + "ol"] = ol
            out[k + "weights"] = weights
            out[k + "out"] = res[:batch * dim]
            n += 1
    out["n_lookup"] = np.array(n)
    # pruned lookups
    m = 0
    for bit_rate, batch, rows, dim, avg_len in [(8, 8, 300, 64, 12), (4, 8, 300, 128, 12), (2, 8, 300, 64, 12)]:
        for weighted in (False, True):
            mapping, dense = mapping_table(rng, rows, 0.5)
            table = random_fused_table(rng, dense, dim, bit_rate)
            lengths, offsets, indices, weights, cnt = lengths_indices_weights(rng, batch, rows, avg_len, np.int64,
                                                                              np.int32)
            ok, res = ref.spmdm_rowwise_sparse(bit_rate, dim, rows, table, indices, mapping, offsets,
                                               weights if weighted else None, True)
            assert ok
            k = f"sparse{m}_"
            out[k + "meta"] = np.array([bit_rate, batch, rows, dim, int(weighted)], dtype=np.int64)
            out[k + "table"] = table
            out[k + "mapping"] = mapping
            out[k + "indices"] = indices
            out[k + "offsets"] = offsets
            out[k + "weights"] = weights
            out[k + "out"] = res[:batch * dim]
            m += 1
    out["n_sparse"] = np.array(m)
    # quantizers
    q = 0
    for rows, cols in [(6, 128), (5, 64), (4, 8), (3, 20)]:
        x = (rng.standard_normal((rows, cols)) * rng.uniform(0.01, 50)).astype(np.float32)
        x[0] = 3.25  # a constant row: range 0
        out[f"quant{q}_x"] = x
        out[f"quant{q}_q8"] = ref.quantize_8bit(x)
        out[f"quant{q}_q4"] = ref.quantize_nbit(4, x)
        out[f"quant{q}_q2"] = ref.quantize_nbit(2, x)
        q += 1
    out["n_quant"] = np.array(q)
    # index remapping
    mapping, _ = mapping_table(rng, 200, 0.5)
    lengths, offsets, indices, weights, cnt = lengths_indices_weights(rng, 11, 200, 9, np.int32, np.int32)
    ri, ro, rw = ref.remap(indices, mapping, offsets, weights)
    out.update(remap_mapping=mapping, remap_indices=indices, remap_offsets=offsets, remap_weights=weights,
               remap_out_indices=ri, remap_out_offsets=ro, remap_out_weights=rw)
    path = os.path.join(HERE, "lookup_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes;", n, "lookups,", m, "pruned lookups,", q, "quantizer cases")


if __name__ == "__main__":
    main()

"""Generates tests/golden/lookup_ex_golden.npz from the REFERENCE's own code:
the lookups with the generators' remaining options - rows with fp16 scale,
bias FIRST and -1 as a pruned index (scale_bias_last = false, the layout of
table-batched embeddings), bf16 output, padded rows, and no_bag - and the
lookups on tables that are not row-wise quantized (fp32, fp16, bf16, fp8 rows),
also through a pruning map (fp32, fp16).

    python tests/golden/make_golden_ex.py

Outputs come from fbgemm::EmbeddingSpMDM_ref / EmbeddingSpMDMNBit_ref /
EmbeddingSpMDMFP8_ref / EmbeddingSpMDMRowWiseSparse_ref compiled
from the reference tree into oracle/_ref/libfbgemm_ref.so (oracle/Makefile).
The fixture pins the CPU oracle (tests/test_oracle.py) and the CUDA kernels
(tests/test_golden_gpu.py); it travels with the repository, the reference
tree does not.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import lengths_indices_weights, mapping_table, random_fused_table, random_plain_table  # noqa: E402
from oracle import checker  # noqa: E402

KINDS = ("f32", "f16", "bf16")


def main():
    if not os.path.exists(checker.REF_SO):
        checker.build(("ref",))
    ref = checker.Reference()
    assert ref.available
    rng = np.random.default_rng(20260202)
    out = {}
    n = 0
    # (bit_rate, batch, rows, dim, avg_len, row stride or None)
    shapes = [(8, 9, 300, 128, 14, None), (8, 6, 200, 40, 8, 48), (4, 10, 400, 64, 20, None), (4, 5, 150, 86, 7, 48),
              (2, 8, 300, 128, 18, None), (2, 4, 90, 36, 6, 16)]
    for bit_rate, batch, rows, dim, avg_len, stride in shapes:
        for variant in range(3):
            sb_last = variant == 2            # two cases of the new layout, one of the old with bf16 output
            kind = KINDS[(variant + 2) % 3] if not sb_last else "bf16"
            weighted = variant != 1
            normalize = variant == 1
            idt = (np.int32, np.int64)[variant % 2]
            table = random_fused_table(rng, rows, dim, bit_rate, None if sb_last else stride, not sb_last)
            _, offsets, indices, weights, cnt = lengths_indices_weights(rng, batch, rows, avg_len, idt, idt)
            if not sb_last:
                indices[rng.integers(0, cnt, max(1, cnt // 5))] = -1   # pruned rows
            ok, res = ref.spmdm_ex(bit_rate, dim, rows, table, indices, offsets, weights if weighted else None,
                                   normalize, kind, False, True, -1, table.shape[1], sb_last, False)
            assert ok
            k = f"ex{n}_"
            out[k + "meta"] = np.array([bit_rate, batch, rows, dim, int(weighted), int(normalize), int(sb_last), 0,
                                        KINDS.index(kind)], dtype=np.int64)
            out[k + "table"] = table
            out[k + "indices"] = indices
            out[k + "offsets"] = offsets
            out[k + "weights"] = weights
            out[k + "out"] = res[:batch * dim]
            n += 1
    # no_bag, 8-bit rows, both layouts
    for sb_last, kind, weighted, rows, dim, count in [(True, "f32", False, 120, 64, 33), (False, "f16", True, 80, 40, 21),
                                                      (True, "bf16", True, 60, 128, 17)]:
        table = random_fused_table(rng, rows, dim, 8, None, not sb_last)
        indices = rng.integers(0, rows, count).astype(np.int64)
        weights = rng.standard_normal(count).astype(np.float32)
        ok, res = ref.spmdm_ex(8, dim, rows, table, indices, None, weights if weighted else None, True, kind, False, True,
                               -1, -1, sb_last, True)
        assert ok
        k = f"ex{n}_"
        out[k + "meta"] = np.array([8, count, rows, dim, int(weighted), 1, int(sb_last), 1, KINDS.index(kind)],
                                   dtype=np.int64)
        out[k + "table"] = table
        out[k + "indices"] = indices
        out[k + "offsets"] = np.zeros(1, dtype=np.int64)
        out[k + "weights"] = weights
        out[k + "out"] = res[:count * dim]
        n += 1
    out["n_ex"] = np.array(n)
    # tables that are not row-wise quantized: fp32 / fp16 / bf16 / fp8 rows
    m = 0
    for in_kind, batch, rows, dim, avg_len, stride, kind, weighted, normalize, sb_last, no_bag in [
            ("f32", 9, 200, 64, 10, None, "f32", True, False, True, False),
            ("f32", 6, 100, 7, 5, 12, "bf16", False, True, False, False),
            ("f16", 8, 300, 128, 12, None, "f16", True, True, True, False),
            ("f16", 5, 80, 40, 6, 48, "f32", False, False, False, False),
            ("bf16", 7, 150, 64, 9, None, "bf16", True, False, True, False),
            ("fp8", 8, 250, 128, 11, None, "f32", True, False, True, False),
            ("fp8", 5, 90, 36, 7, 40, "f16", False, True, True, False),
            ("f32", 0, 120, 32, 0, None, "f16", True, False, True, True),
            ("f16", 0, 70, 96, 0, None, "f32", False, False, True, True)]:
        table = random_plain_table(rng, rows, dim, in_kind, stride)
        if no_bag:
            cnt = 25
            indices = rng.integers(0, rows, cnt).astype(np.int64)
            offsets = np.zeros(1, dtype=np.int64)
            weights = rng.standard_normal(cnt).astype(np.float32)
            batch = cnt
        else:
            _, offsets, indices, weights, cnt = lengths_indices_weights(rng, batch, rows, avg_len, np.int32, np.int32)
            if not sb_last:
                indices[rng.integers(0, cnt, max(1, cnt // 5))] = -1
        ebits, ebias = (5, 15) if (in_kind == "fp8" and m % 2) else (4, 7)
        ok, res = ref.spmdm_plain(in_kind, dim, rows, table, indices, None if no_bag else offsets,
                                  weights if weighted else None, normalize, kind, False, True, -1, table.shape[1],
                                  sb_last, no_bag, ebits, ebias)
        assert ok
        k = f"plain{m}_"
        out[k + "meta"] = np.array([("f32", "f16", "bf16", "fp8").index(in_kind), batch, rows, dim, int(weighted),
                                    int(normalize), int(sb_last), int(no_bag), KINDS.index(kind), ebits, ebias],
                                   dtype=np.int64)
        out[k + "table"] = table
        out[k + "indices"] = indices
        out[k + "offsets"] = offsets
        out[k + "weights"] = weights
        out[k + "out"] = res[:batch * dim]
        m += 1
    out["n_plain"] = np.array(m)
    # Pruned (row-wise sparse) lookups over float and fp16 rows: EmbeddingSpMDMRowWiseSparse_ref<float|float16|uint16_t>.
    # (in_kind, batch, uncompressed rows, dim, avg_len, sparsity, weighted, normalize, index type)
    q = 0
    for in_kind, batch, urows, dim, avg_len, sparsity, weighted, normalize, idt in [
            ("f32", 9, 400, 64, 10, 0.5, True, False, np.int64), ("f32", 6, 150, 7, 6, 0.8, False, True, np.int32),
            ("f16", 8, 300, 128, 12, 0.5, True, True, np.int32), ("f16", 5, 90, 40, 5, 0.2, False, False, np.int64),
            ("u16", 7, 200, 32, 8, 0.5, True, False, np.int32)]:
        cit, rows = mapping_table(rng, urows, sparsity)
        table = random_plain_table(rng, rows, dim, "f32" if in_kind == "f32" else "f16")
        _, offsets, indices, weights, cnt = lengths_indices_weights(rng, batch, urows, avg_len, idt, np.int32)
        ok, res = ref.spmdm_plain_rowwise_sparse(in_kind, dim, urows, table, indices, cit, offsets,
                                                 weights if weighted else None, normalize)
        assert ok
        k = f"sparse{q}_"
        out[k + "meta"] = np.array([("f32", "f16", "u16").index(in_kind), batch, urows, dim, int(weighted),
                                    int(normalize)], dtype=np.int64)
        out[k + "table"] = table
        out[k + "cit"] = cit
        out[k + "indices"] = indices
        out[k + "offsets"] = offsets
        out[k + "weights"] = weights
        out[k + "out"] = res[:batch * dim]
        q += 1
    out["n_sparse"] = np.array(q)
    path = os.path.join(HERE, "lookup_ex_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes;", n, "quantized-row cases,", m, "plain-row cases,", q,
          "pruned plain-row cases")


if __name__ == "__main__":
    main()

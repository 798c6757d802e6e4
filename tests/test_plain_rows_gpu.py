"""Lookups on tables that are not row-wise quantized (fp32 / fp16 / bf16 / FP8
rows), bit for bit against fixtures made by the reference's
EmbeddingSpMDM_ref<float|float16|uint16_t> / EmbeddingSpMDMFP8_ref
(tests/golden/make_golden_ex.py) and against the CPU oracle on the reference
tests' shapes."""
import os

import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from conftest import bits
from helpers import REFERENCE_SHAPES, lengths_indices_weights, mapping_table, random_plain_table
from test_oracle import IN_KINDS, KINDS
from test_variants_gpu import NP_KIND, TORCH_KIND, dev, out_bits

pytestmark = pytest.mark.gpu
EX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lookup_ex_golden.npz")
IN_NP = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16}


def generate(in_kind, dim, weighted, normalize, use_offsets, idt, odt, kind, sb_last, no_bag, stride, ebits=4, ebias=7):
    kw = dict(index_dtype=idt, offset_dtype=odt, out_dtype=NP_KIND[kind])
    if in_kind == "fp8":
        return F.GenerateEmbeddingSpMDMFP8WithStrides(dim, normalize, False, use_offsets, -1, stride, ebits, ebias,
                                                      kind == "bf16", **kw)
    return F.GenerateEmbeddingSpMDMWithStrides(dim, weighted, normalize, 16, False, use_offsets, -1, stride, sb_last,
                                               no_bag, kind == "bf16", in_kind == "bf16", in_dtype=IN_NP[in_kind], **kw)


def test_fixtures_made_by_the_reference(gpu_ctx):
    ex = np.load(EX)
    for i in range(int(ex["n_plain"])):
        k = f"plain{i}_"
        in_kind, count, rows, dim, weighted, normalize, sb_last, no_bag, kind, ebits, ebias = (int(v) for v in ex[k + "meta"])
        in_kind, kind = IN_KINDS[in_kind], KINDS[kind]
        table, idx, off = ex[k + "table"], ex[k + "indices"], ex[k + "offsets"]
        kern = generate(in_kind, dim, weighted, normalize, True, idx.dtype.type, off.dtype.type, kind, bool(sb_last),
                        bool(no_bag), table.shape[1], ebits, ebias)
        out = torch.zeros(count * dim, dtype=TORCH_KIND[kind], device="cuda")
        ok = kern(count, len(idx), rows, dev(table), dev(idx), None if no_bag else dev(off),
                  dev(ex[k + "weights"]) if weighted else None, out)
        assert ok, i
        np.testing.assert_array_equal(out_bits(out), bits(ex[k + "out"]), err_msg=f"case {i}")


@pytest.mark.parametrize("in_kind", IN_KINDS)
def test_reference_shapes(gpu_ctx, oracle, in_kind):
    rng = np.random.default_rng(6000 + IN_KINDS.index(in_kind))
    shapes = REFERENCE_SHAPES + [(6, 300, 1000, 12), (5, 200, 300, 9)]   # rows wider than one 1 KB tile as well
    for shape_i, (batch, rows, dim, avg_len) in enumerate(shapes):
        idt, odt = ((np.int32, np.int64), (np.int64, np.int32))[shape_i % 2]
        kind = KINDS[shape_i % 3]
        weighted, normalize, use_offsets = shape_i % 2 == 0, shape_i % 3 == 1, shape_i % 4 != 3
        sb_last = shape_i % 3 != 2 or in_kind == "fp8"
        stride = dim + (shape_i % 3)   # padded rows; odd strides take the element-wise kernel
        table = random_plain_table(rng, rows, dim, in_kind, stride)
        ebits, ebias = ((4, 7), (5, 15))[shape_i % 2]
        for corner in (None, "oob", "empty"):
            lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, odt, corner)
            if corner is None and not sb_last:
                indices[rng.integers(0, n, max(1, n // 5))] = -1
            ol = offsets if use_offsets else lengths
            ok_ref, ref = oracle.spmdm_plain(in_kind, dim, rows, table, indices, ol, weights if weighted else None,
                                             normalize, kind, False, use_offsets, -1, stride, sb_last, False, ebits,
                                             ebias, output_size=batch, index_size=n)
            kern = generate(in_kind, dim, weighted, normalize, use_offsets, idt, odt, kind, sb_last, False, stride, ebits,
                            ebias)
            out = torch.ones(batch * dim + 6, dtype=TORCH_KIND[kind], device="cuda")
            ok = kern(batch, n, rows, dev(table), dev(indices) if n else None, dev(ol),
                      dev(weights) if weighted and n else None, out)
            assert ok == ok_ref == (corner != "oob")
            assert (out[batch * dim:].float().cpu().numpy() == 1).all(), "wrote past the output"
            if ok:
                np.testing.assert_array_equal(out_bits(out)[:batch * dim], bits(ref[:batch * dim]), err_msg=str(shape_i))


def test_no_bag_and_fp8_formats(gpu_ctx, oracle):
    rng = np.random.default_rng(6100)
    for in_kind in ("f32", "f16", "bf16"):
        rows, dim, count = 200, 96, 150
        table = random_plain_table(rng, rows, dim, in_kind)
        indices = rng.integers(0, rows, count).astype(np.int64)
        weights = rng.standard_normal(count).astype(np.float32)
        ok_ref, ref = oracle.spmdm_plain(in_kind, dim, rows, table, indices, None, weights, True, "f16", False, True, -1,
                                         -1, True, True)
        kern = generate(in_kind, dim, True, True, True, np.int64, np.int64, "f16", True, True, -1)
        out = torch.zeros(count * dim, dtype=torch.float16, device="cuda")
        assert kern(count, count, rows, dev(table), dev(indices), None, dev(weights), out) and ok_ref
        np.testing.assert_array_equal(out_bits(out), bits(ref))
    # every FP8 bit pattern in a few exponent layouts
    table = np.arange(256, dtype=np.uint8).reshape(4, 64)
    idx = np.arange(4, dtype=np.int32)
    off = np.arange(5, dtype=np.int32)
    for ebits, ebias in ((4, 7), (5, 15), (3, 4), (2, 1)):
        ok_ref, ref = oracle.spmdm_plain("fp8", 64, 4, table, idx, off, None, False, "f32", False, True, -1, -1, True,
                                         False, ebits, ebias)
        kern = generate("fp8", 64, False, False, True, np.int32, np.int32, "f32", True, False, -1, ebits, ebias)
        out = torch.zeros(4 * 64, device="cuda")
        assert kern(4, 4, 4, dev(table), dev(idx), dev(off), None, out) and ok_ref
        np.testing.assert_array_equal(out_bits(out), bits(ref))


# ---- the same rows through a pruning map: GenerateEmbeddingSpMDMRowWiseSparse<float | float16> -------------

SPARSE_KINDS = ("f32", "f16", "u16")


def test_pruned_fixtures_made_by_the_reference(gpu_ctx):
    ex = np.load(EX)
    for i in range(int(ex["n_sparse"])):
        k = f"sparse{i}_"
        in_kind, batch, urows, dim, weighted, normalize = (int(v) for v in ex[k + "meta"])
        idx, off = ex[k + "indices"], ex[k + "offsets"]
        kern = F.GenerateEmbeddingSpMDMRowWiseSparse(dim, bool(weighted), bool(normalize), 16, False, True,
                                                     index_dtype=idx.dtype.type, offset_dtype=off.dtype.type,
                                                     in_dtype=np.float32 if in_kind == 0 else np.float16)
        out = torch.zeros(batch * dim, dtype=torch.float32, device="cuda")
        ok = kern(batch, len(idx), urows, dev(ex[k + "table"]), dev(idx), dev(off),
                  dev(ex[k + "weights"]) if weighted else None, out, dev(ex[k + "cit"]))
        assert ok, i
        np.testing.assert_array_equal(out_bits(out), bits(ex[k + "out"]), err_msg=f"case {i}")


@pytest.mark.parametrize("in_kind", ["f32", "f16"])
def test_pruned_reference_shapes(gpu_ctx, oracle, in_kind):
    rng = np.random.default_rng(6100 + SPARSE_KINDS.index(in_kind))
    for shape_i, (batch, urows, dim, avg_len) in enumerate(REFERENCE_SHAPES + [(6, 300, 1000, 12)]):
        idt, odt = ((np.int32, np.int64), (np.int64, np.int32))[shape_i % 2]
        weighted, normalize, use_offsets = shape_i % 2 == 0, shape_i % 3 == 1, shape_i % 4 != 3
        positional = weighted and shape_i % 4 == 2
        cit, rows = mapping_table(rng, urows, (0.5, 0.9, 0.0, 1.0)[shape_i % 4])
        table = random_plain_table(rng, max(rows, 1), dim, in_kind)
        kern = F.GenerateEmbeddingSpMDMRowWiseSparse(dim, weighted, normalize, 16, positional, use_offsets,
                                                     index_dtype=idt, offset_dtype=odt, in_dtype=IN_NP[in_kind])
        for corner in (None, "oob", "empty"):
            lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, urows, avg_len, idt, odt, corner)
            ol = offsets if use_offsets else lengths
            ok_ref, ref = oracle.spmdm_plain_rowwise_sparse(in_kind, dim, urows, table, indices, cit, ol,
                                                            weights if weighted else None, normalize, positional,
                                                            use_offsets)
            out = torch.zeros(batch * dim, dtype=torch.float32, device="cuda")
            ok = kern(batch, n, urows, dev(table), dev(indices) if n else None, dev(ol),
                      dev(weights) if weighted and n else None, out, dev(cit))
            assert ok == ok_ref == (corner != "oob")
            if ok:
                np.testing.assert_array_equal(out_bits(out), bits(ref), err_msg=f"shape {shape_i} {corner}")

"""The table-batched operator (fbgemm_b200/tbe.py) against the oracle, table by
table: the reference's operator is a loop over tables calling the generated
kernel with `output + D_start`, output_stride = total_D and the table's slice of
the T*B+1 offsets
(fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:343-473
of FBGEMM)."""
import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from fbgemm_b200 import tbe
from conftest import bits
from helpers import build_op_inputs

pytestmark = pytest.mark.gpu

KIND = {tbe.SparseType.FP32: "f32", tbe.SparseType.FP16: "f16", tbe.SparseType.BF16: "bf16"}
BITS = {tbe.SparseType.INT8: 8, tbe.SparseType.INT4: 4, tbe.SparseType.INT2: 2}
PLAIN = {tbe.SparseType.FP32: "f32", tbe.SparseType.FP16: "f16", tbe.SparseType.FP8: "fp8"}


@pytest.mark.parametrize("scale_bias_last", [False, True])
@pytest.mark.parametrize("out_ty", [tbe.SparseType.FP16, tbe.SparseType.BF16, tbe.SparseType.FP32])
def test_operator_matches_oracle_table_by_table(gpu_ctx, oracle, scale_bias_last, out_ty):
    rng = np.random.default_rng(8100 + int(out_ty) + 10 * scale_bias_last)
    tys = [tbe.SparseType.INT4, tbe.SparseType.INT8, tbe.SparseType.INT2, tbe.SparseType.INT4, tbe.SparseType.INT8]
    dims = [64, 128, 128, 32, 24]
    rows = [500, 300, 400, 200, 100]
    B, idt = 19, (np.int32 if out_ty != tbe.SparseType.FP32 else np.int64)
    for weighted, pooling in ((False, tbe.PoolingMode.SUM), (True, tbe.PoolingMode.MEAN)):
        tables, blob, w_off, D_off, offsets, indices, weights = build_op_inputs(
            rng, tys, dims, rows, B, 9, 16, scale_bias_last, idt)
        total_D = int(D_off[-1])
        tdt = torch.int32 if idt == np.int32 else torch.int64
        op = tbe.IntNBitTableBatchedEmbeddingBags(
            torch.from_numpy(blob).cuda(), w_off, np.array([int(t) for t in tys], np.uint8), D_off, total_D, pooling, 16,
            out_ty, scale_bias_last, weighted, tdt)
        d_idx, d_off, d_w = (torch.from_numpy(a).cuda() for a in (indices, offsets, weights))
        for use_plan in (False, True):
            out = op.forward(d_idx, d_off, d_w if weighted else None, slot=21, use_plan=use_plan)
            ok, info = F.status_read(21)
            assert ok, info
            got = out.cpu().view(torch.int32 if out.dtype == torch.float32 else torch.int16).numpy().view(
                np.uint32 if out.dtype == torch.float32 else np.uint16).reshape(B, total_D)
            for t in range(len(tys)):
                lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
                ok_ref, ref = oracle.spmdm_ex(BITS[tys[t]], dims[t], rows[t], tables[t], indices[lo:hi],
                                              offsets[t * B:(t + 1) * B + 1], weights[lo:hi] if weighted else None,
                                              pooling == tbe.PoolingMode.MEAN, KIND[out_ty], False, True, -1,
                                              tables[t].shape[1], scale_bias_last, False)
                assert ok_ref
                np.testing.assert_array_equal(np.ascontiguousarray(got[:, D_off[t]:D_off[t + 1]]).reshape(-1),
                                              bits(ref), err_msg=f"table {t}")


def test_function_form_and_bad_index(gpu_ctx, oracle):
    rng = np.random.default_rng(8200)
    tys, dims, rows = [tbe.SparseType.INT4, tbe.SparseType.INT2], [64, 64], [100, 50]
    tables, blob, w_off, D_off, offsets, indices, weights = build_op_inputs(rng, tys, dims, rows, 8, 5, 16, False, np.int32)
    args = (torch.from_numpy(blob).cuda(), w_off, np.array([int(t) for t in tys], np.uint8), D_off, int(D_off[-1]))
    out = tbe.int_nbit_split_embedding_codegen_forward(*args, torch.from_numpy(indices).cuda(),
                                                       torch.from_numpy(offsets).cuda(), tbe.PoolingMode.SUM, 16)
    assert F.status_read(0)[0] and out.shape == (8, 128) and out.dtype == torch.float16
    lo, hi = int(offsets[8]), int(offsets[16])
    ok_ref, ref = oracle.spmdm_ex(2, 64, 50, tables[1], indices[lo:hi], offsets[8:17], None, False, "f16", False, True,
                                  -1, tables[1].shape[1], False, False)
    got = out.cpu().view(torch.int16).numpy().view(np.uint16)[:, 64:]
    np.testing.assert_array_equal(np.ascontiguousarray(got).reshape(-1), bits(ref))
    indices[hi - 1] = 50   # one past the last row of table 1
    tbe.int_nbit_split_embedding_codegen_forward(*args, torch.from_numpy(indices).cuda(),
                                                 torch.from_numpy(offsets).cuda(), tbe.PoolingMode.SUM, 16)
    ok, info = F.status_read(0)
    assert not ok and info[0] == 1 and info[2] == hi - 1 and info[3] == 50


def test_operator_with_unquantized_and_fp8_tables(gpu_ctx, oracle):
    rng = np.random.default_rng(8300)
    tys = [tbe.SparseType.FP16, tbe.SparseType.INT4, tbe.SparseType.FP32, tbe.SparseType.FP8]
    dims, rows, B = [64, 64, 24, 36], [300, 200, 100, 150], 11
    tables, blob, w_off, D_off, offsets, indices, weights = build_op_inputs(rng, tys, dims, rows, B, 7, 16, True, np.int32)
    total_D = int(D_off[-1])
    op = tbe.IntNBitTableBatchedEmbeddingBags(torch.from_numpy(blob).cuda(), w_off, np.array([int(t) for t in tys], np.uint8),
                                              D_off, total_D, tbe.PoolingMode.SUM, 16, tbe.SparseType.FP32, True, True,
                                              torch.int32, 5, 15)
    out = op.forward(*(torch.from_numpy(a).cuda() for a in (indices, offsets, weights)), slot=22)
    ok, info = F.status_read(22)
    assert ok, info
    got = out.cpu().numpy().view(np.uint32)
    for t, ty in enumerate(tys):
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        if ty in PLAIN:
            eb = {"f32": 4, "f16": 2, "fp8": 1}[PLAIN[ty]]
            view = tables[t].reshape(-1).view({4: np.float32, 2: np.uint16, 1: np.uint8}[eb])
            ok_ref, ref = oracle.spmdm_plain(PLAIN[ty], dims[t], rows[t], view, indices[lo:hi], offsets[t * B:(t + 1) * B + 1],
                                             weights[lo:hi], False, "f32", False, True, -1, tables[t].shape[1] // eb, True,
                                             False, 5, 15)
        else:
            ok_ref, ref = oracle.spmdm_ex(BITS[ty], dims[t], rows[t], tables[t], indices[lo:hi],
                                          offsets[t * B:(t + 1) * B + 1], weights[lo:hi], False, "f32", False, True, -1,
                                          tables[t].shape[1], True, False)
        assert ok_ref
        np.testing.assert_array_equal(np.ascontiguousarray(got[:, D_off[t]:D_off[t + 1]]).reshape(-1), bits(ref),
                                      err_msg=f"table {t}")


def test_plan_cache_is_bounded(gpu_ctx):
    rng = np.random.default_rng(8400)
    tys, dims, rows, B = [tbe.SparseType.INT4, tbe.SparseType.INT8], [32, 64], [60, 50], 5
    tables, blob, w_off, D_off, offsets, indices, _ = build_op_inputs(rng, tys, dims, rows, B, 4, 16, False, np.int32)
    op = tbe.IntNBitTableBatchedEmbeddingBags(torch.from_numpy(blob).cuda(), w_off, np.array([int(t) for t in tys], np.uint8),
                                              D_off, 96, tbe.PoolingMode.SUM, 16, tbe.SparseType.FP16)
    d_idx, d_off = torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda()
    first = op.forward(d_idx, d_off, use_plan=True).clone()
    outs = [torch.zeros((B, 96), dtype=torch.float16, device="cuda") for _ in range(op.MAX_PLANS + 6)]
    for o in outs:
        op.forward(d_idx, d_off, output=o, use_plan=True)
    assert F.status_read(0)[0] and len(op._plans) == op.MAX_PLANS
    assert all(torch.equal(o, first) for o in outs)


def test_operator_matches_the_reference_operator_fixtures(gpu_ctx):
    """Outputs of the reference's own
    int_nbit_split_embedding_codegen_forward_{unweighted,weighted}_cpu
    (tests/golden/make_golden_tbe.py), bit for bit."""
    from helpers import load_golden

    g = load_golden("tbe_golden.npz")
    for i in range(int(g["n_op"])):
        k = f"op{i}_"
        B, sbl, out_ty, weighted, pooling, align = (int(x) for x in g[k + "meta"])
        indices, offsets = g[k + "indices"], g[k + "offsets"]
        tdt = torch.int32 if indices.dtype == np.int32 else torch.int64
        total_D = int(g[k + "D_off"][-1])
        op = tbe.IntNBitTableBatchedEmbeddingBags(
            torch.from_numpy(g[k + "blob"]).cuda(), g[k + "w_off"], g[k + "tys"].astype(np.uint8), g[k + "D_off"], total_D,
            pooling, align, out_ty, bool(sbl), bool(weighted), tdt, 5, 15)
        d_w = torch.from_numpy(g[k + "weights"]).cuda() if weighted else None
        for use_plan in (False, True):
            out = op.forward(torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda(), d_w, slot=23,
                             use_plan=use_plan)
            ok, info = F.status_read(23)
            assert ok, info
            got = out.cpu().view(torch.int32 if out.dtype == torch.float32 else torch.int16).numpy()
            want = g[k + "out"]
            np.testing.assert_array_equal(got.view(np.uint32 if out.dtype == torch.float32 else np.uint16),
                                          want.view(np.uint32) if want.dtype == np.float32 else want, err_msg=k)

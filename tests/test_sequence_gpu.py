"""The sequence ("nobag") form of the table-batched operator against the
oracle, table by table.  The reference
(fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:206-520
of FBGEMM, `nobag` branch) builds bags of one index per table and calls the
pooled kernel of the table's row type without weights, or - for INT8 / INT4
output - the kernels' no_bag forms, which copy row bytes; the oracle calls are
composed the same way here."""
import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from fbgemm_b200 import tbe
from conftest import bits
from test_tbe_gpu import BITS, KIND, PLAIN, build_op_inputs

pytestmark = pytest.mark.gpu
ST = tbe.SparseType


def reference_rows(oracle, ty, D, rows, table, idx, out_kind, scale_bias_last, fp8=(4, 7)):
    ones = np.ones(len(idx), dtype=idx.dtype)
    if ty in PLAIN:
        eb = {"f32": 4, "f16": 2, "fp8": 1}[PLAIN[ty]]
        view = table.reshape(-1).view({4: np.float32, 2: np.uint16, 1: np.uint8}[eb])
        return oracle.spmdm_plain(PLAIN[ty], D, rows, view, idx, ones, None, False, out_kind, False, False, -1,
                                  table.shape[1] // eb, scale_bias_last, False, fp8[0], fp8[1])
    return oracle.spmdm_ex(BITS[ty], D, rows, table, idx, ones, None, False, out_kind, False, False, -1,
                           table.shape[1], scale_bias_last, False)


@pytest.mark.parametrize("scale_bias_last", [False, True])
@pytest.mark.parametrize("out_ty", [ST.FP32, ST.FP16, ST.BF16])
@pytest.mark.parametrize("D,align", [(64, 16), (24, 1), (12, 1), (132, 4)])
def test_dequantized_rows_match_the_oracle(gpu_ctx, oracle, scale_bias_last, out_ty, D, align):
    rng = np.random.default_rng(9500 + int(out_ty) + 10 * scale_bias_last + D)
    tys = [ST.INT4, ST.INT8, ST.INT2, ST.FP16, ST.FP32, ST.FP8, ST.INT4]
    rows = [300, 200, 150, 100, 80, 120, 50]
    T, B = len(tys), 13
    idt = np.int64 if out_ty == ST.FP32 else np.int32
    tables, blob, w_off, _, offsets, indices, _ = build_op_inputs(rng, tys, [D] * T, rows, B, 5, align, scale_bias_last, idt)
    op = tbe.IntNBitSequenceEmbedding(torch.from_numpy(blob).cuda(), w_off, np.array([int(t) for t in tys], np.uint8), D,
                                      align, out_ty, scale_bias_last, 5, 15)
    out = op.forward(torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda(), slot=31)
    ok, info = F.status_read(31)
    got = out.cpu().view(torch.int32 if out.dtype == torch.float32 else torch.int16).numpy().view(
        np.uint32 if out.dtype == torch.float32 else np.uint16)
    assert got.shape == (len(indices), D)
    fp8_minus_one = False
    for t, ty in enumerate(tys):
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        idx = indices[lo:hi]
        if ty == ST.FP8 and not scale_bias_last:
            # -1 is no pruned row for FP8 tables: the reference returns false at the first one; check the rows before it
            bad = np.flatnonzero(idx == -1)
            fp8_minus_one = fp8_minus_one or len(bad) > 0
            keep = idx != -1
            ok_ref, ref = reference_rows(oracle, ty, D, rows[t], tables[t], idx[keep], KIND[out_ty], scale_bias_last, (5, 15))
            assert ok_ref
            np.testing.assert_array_equal(got[lo:hi][keep].reshape(-1), bits(ref)[:keep.sum() * D])
            assert (got[lo:hi][~keep] == 0).all()   # left as the zero fill
            continue
        ok_ref, ref = reference_rows(oracle, ty, D, rows[t], tables[t], idx, KIND[out_ty], scale_bias_last, (5, 15))
        assert ok_ref
        np.testing.assert_array_equal(got[lo:hi].reshape(-1), bits(ref)[:(hi - lo) * D], err_msg=f"table {t} {ty.name}")
    assert ok == (not fp8_minus_one), info


def test_int8_and_int4_output_are_row_copies(gpu_ctx, oracle):
    rng = np.random.default_rng(9600)
    B = 9
    for out_ty, ty, D, align, sbl in ((ST.INT8, ST.INT8, 32, 1, False), (ST.INT8, ST.INT8, 20, 16, False),
                                      (ST.INT8, ST.INT8, 24, 1, True), (ST.INT4, ST.INT4, 32, 1, False),
                                      (ST.INT4, ST.INT4, 30, 1, False)):
        tys, rows = [ty] * 3, [100, 60, 40]
        tables, blob, w_off, _, offsets, indices, _ = build_op_inputs(rng, tys, [D] * 3, rows, B, 6, align, sbl, np.int32)
        indices[indices < 0] = 0   # the row copies know no pruned index
        op = tbe.IntNBitSequenceEmbedding(torch.from_numpy(blob).cuda(), w_off, np.array([int(t) for t in tys], np.uint8),
                                          D, align, out_ty, sbl)
        out = op.forward(torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda(), slot=32)
        assert F.status_read(32)[0]
        got = out.cpu().numpy()
        for t in range(3):
            lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
            row_bytes = tables[t].shape[1]
            if out_ty == ST.INT8:
                assert got.shape[1] == D + 4
                ok_ref, ref = oracle.rows_copy(8, D, rows[t], tables[t], indices[lo:hi], D + 4, row_bytes)
                width = min(D + 4, row_bytes)
                np.testing.assert_array_equal(got[lo:hi, :width], ref[:hi - lo, :width])
                assert (got[lo:hi, width:] == 0).all()
            else:
                assert got.shape[1] == (D + 9) // 2 == row_bytes
                ok_ref, ref = oracle.rows_copy(4, D, rows[t], tables[t], indices[lo:hi], row_bytes, row_bytes)
                np.testing.assert_array_equal(got[lo:hi], ref[:hi - lo])
            assert ok_ref
    with pytest.raises(ValueError):
        tbe.IntNBitSequenceEmbedding(torch.zeros(64, dtype=torch.uint8, device="cuda"), [0], [int(ST.INT4)], 8, 1, ST.INT8)


def test_out_of_range_index_is_reported_and_lookup_function_dispatches(gpu_ctx, oracle):
    rng = np.random.default_rng(9700)
    tys, dims, rows, B = [ST.INT4, ST.INT8], [32, 32], [40, 30], 6
    tables, blob, w_off, D_off, offsets, indices, weights = build_op_inputs(rng, tys, dims, rows, B, 4, 16, False, np.int32)
    dev_w = torch.from_numpy(blob).cuda()
    d_idx, d_off = torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda()
    empty = torch.empty(0, dtype=torch.uint8, device="cuda")
    common = (dev_w, empty, None, w_off, np.array([int(t) for t in tys], np.uint8), D_off, 64, 0, 32, 32, 0, 0)
    seq = tbe.int_nbit_split_embedding_codegen_lookup_function(*common, d_idx, d_off, tbe.PoolingMode.NONE, None, ST.FP32,
                                                               row_alignment=16)
    assert F.status_read(0)[0] and seq.shape == (len(indices), 32) and seq.dtype == torch.float32
    lo, hi = int(offsets[B]), int(offsets[2 * B])
    ok_ref, ref = reference_rows(oracle, ST.INT8, 32, 30, tables[1], indices[lo:hi], "f32", False)
    np.testing.assert_array_equal(seq.cpu().numpy()[lo:hi].view(np.uint32).reshape(-1), bits(ref)[:(hi - lo) * 32])
    pooled = tbe.int_nbit_split_embedding_codegen_lookup_function(*common, d_idx, d_off, tbe.PoolingMode.SUM, None, ST.FP32,
                                                                  row_alignment=16)
    assert F.status_read(0)[0] and pooled.shape == (B, 64)
    ok_ref, ref = oracle.spmdm_ex(8, 32, 30, tables[1], indices[lo:hi], offsets[B:2 * B + 1], None, False, "f32", False, True,
                                  -1, tables[1].shape[1], False, False)
    np.testing.assert_array_equal(np.ascontiguousarray(pooled.cpu().numpy()[:, 32:]).view(np.uint32).reshape(-1), bits(ref))
    weighted = tbe.int_nbit_split_embedding_codegen_lookup_function(
        *common, d_idx, d_off, tbe.PoolingMode.SUM, torch.from_numpy(weights).cuda(), ST.FP32, row_alignment=16)
    ok_ref, ref = oracle.spmdm_ex(8, 32, 30, tables[1], indices[lo:hi], offsets[B:2 * B + 1], weights[lo:hi], False, "f32",
                                  False, True, -1, tables[1].shape[1], False, False)
    assert F.status_read(0)[0]
    np.testing.assert_array_equal(np.ascontiguousarray(weighted.cpu().numpy()[:, 32:]).view(np.uint32).reshape(-1), bits(ref))
    indices[hi - 1] = 30  # one past the last row of table 1
    tbe.int_nbit_split_embedding_codegen_lookup_function(*common, torch.from_numpy(indices).cuda(), d_off,
                                                         tbe.PoolingMode.NONE, None, ST.FP16, row_alignment=16)
    ok, info = F.status_read(0)
    assert not ok and info[:4] == [1, 1, hi - 1, 30]


def test_more_tables_than_fit_in_shared_memory(gpu_ctx, oracle):
    """Beyond 2047 tables the position -> table bisection reads the offsets from global memory."""
    rng = np.random.default_rng(9800)
    T, B, D, rows = 2100, 1, 8, 4
    tys = [ST.INT8] * T
    tables, blob, w_off, _, offsets, indices, _ = build_op_inputs(rng, tys, [D] * T, [rows] * T, B, 2, 4, True, np.int64)
    op = tbe.IntNBitSequenceEmbedding(torch.from_numpy(blob).cuda(), w_off, np.array([int(t) for t in tys], np.uint8), D, 4,
                                      ST.FP32, True)
    out = op.forward(torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda(), slot=33)
    assert F.status_read(33)[0]
    got = out.cpu().numpy().view(np.uint32)
    for t in range(0, T, 97):
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        if hi > lo:
            ok_ref, ref = reference_rows(oracle, ST.INT8, D, rows, tables[t], indices[lo:hi], "f32", True)
            assert ok_ref
            np.testing.assert_array_equal(got[lo:hi].reshape(-1), bits(ref)[:(hi - lo) * D])


def test_sequence_operator_matches_the_reference_operator_fixtures(gpu_ctx):
    """Outputs of the reference's own
    int_nbit_split_embedding_nobag_codegen_forward_unweighted_cpu
    (tests/golden/make_golden_tbe.py), bit for bit."""
    from helpers import load_golden

    g = load_golden("tbe_golden.npz")
    for i in range(int(g["n_seq"])):
        k = f"seq{i}_"
        B, sbl, out_ty, D, align = (int(x) for x in g[k + "meta"])
        op = tbe.IntNBitSequenceEmbedding(torch.from_numpy(g[k + "blob"]).cuda(), g[k + "w_off"],
                                          g[k + "tys"].astype(np.uint8), D, align, out_ty, bool(sbl))
        out = op.forward(torch.from_numpy(g[k + "indices"]).cuda(), torch.from_numpy(g[k + "offsets"]).cuda(), slot=34)
        ok, info = F.status_read(34)
        assert ok, info
        got = out.cpu().view(torch.int32 if out.dtype == torch.float32 else torch.int16).numpy()
        want = g[k + "out"]
        np.testing.assert_array_equal(got.view(np.uint32 if out.dtype == torch.float32 else np.uint16),
                                      want.view(np.uint32) if want.dtype == np.float32 else want, err_msg=k)

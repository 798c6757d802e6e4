"""Host logic of the table-batched operator mirror (no GPU): row sizes and
enumerations as the reference defines them."""
import pytest

from fbgemm_b200 import tbe


def test_enumerations_match_the_reference():
    # fbgemm_gpu/include/fbgemm_gpu/embedding_common.h:20-34
    assert [int(t) for t in (tbe.SparseType.FP32, tbe.SparseType.FP16, tbe.SparseType.INT8, tbe.SparseType.INT4,
                             tbe.SparseType.INT2, tbe.SparseType.BF16, tbe.SparseType.FP8)] == [0, 1, 2, 3, 4, 5, 6]
    assert [int(m) for m in (tbe.PoolingMode.SUM, tbe.PoolingMode.MEAN, tbe.PoolingMode.NONE)] == [0, 1, 2]


@pytest.mark.parametrize("dim,ty,align,sb,want", [
    (128, tbe.SparseType.INT8, 16, 4, 144),   # 128 + 4 = 132 -> 144
    (128, tbe.SparseType.INT8, 1, 8, 136),    # scale, bias last: fp32 pair, unpadded (the CPU default)
    (128, tbe.SparseType.INT4, 16, 4, 80),    # 64 + 4 = 68 -> 80
    (64, tbe.SparseType.INT4, 16, 4, 48),     # 32 + 4 = 36 -> 48
    (128, tbe.SparseType.INT2, 16, 4, 48),    # 32 + 4 = 36 -> 48
    (64, tbe.SparseType.INT2, 1, 4, 20),
    (24, tbe.SparseType.INT8, 16, 4, 32),
    (64, tbe.SparseType.FP16, 16, 4, 128),
])
def test_padded_row_size(dim, ty, align, sb, want):
    # nbit::padded_row_size_in_bytes, embedding_common.h:189-225
    assert tbe.padded_row_size_in_bytes(dim, ty, align, sb) == want


def test_row_sizes_of_unquantized_types():
    assert tbe.padded_row_size_in_bytes(64, tbe.SparseType.FP16, 16) == 128
    assert tbe.padded_row_size_in_bytes(30, tbe.SparseType.FP32, 16) == 128
    assert tbe.padded_row_size_in_bytes(36, tbe.SparseType.FP8, 16) == 48


def test_oracle_composition_matches_the_reference_operator():
    """The oracle's single-table lookups, composed table by table as the tests
    compose them, against outputs of the reference's own
    int_nbit_split_embedding_codegen_forward_{unweighted,weighted}_cpu and
    ..._nobag_... (fixtures made by tests/golden/make_golden_tbe.py)."""
    import numpy as np

    from helpers import load_golden, oracle_op_forward, oracle_sequence_forward
    from oracle.checker import Oracle

    oracle = Oracle()
    g = load_golden("tbe_golden.npz")
    assert int(g["n_op"]) >= 16 and int(g["n_seq"]) >= 9
    for i in range(int(g["n_op"])):
        k = f"op{i}_"
        B, sbl, out_ty, weighted, pooling, align = (int(x) for x in g[k + "meta"])
        got = oracle_op_forward(oracle, g[k + "tys"], g[k + "dims"], g[k + "rows"], g[k + "blob"], g[k + "w_off"],
                                g[k + "D_off"], g[k + "indices"], g[k + "offsets"], g[k + "weights"] if weighted else None,
                                B, pooling == 1, out_ty, bool(sbl), align, (5, 15))
        want = g[k + "out"]
        want = want.view(np.uint32) if want.dtype == np.float32 else want
        np.testing.assert_array_equal(got, want, err_msg=k)
    for i in range(int(g["n_seq"])):
        k = f"seq{i}_"
        B, sbl, out_ty, D, align = (int(x) for x in g[k + "meta"])
        got = oracle_sequence_forward(oracle, g[k + "tys"], D, g[k + "rows"], g[k + "blob"], g[k + "w_off"],
                                      g[k + "indices"], g[k + "offsets"], B, out_ty, bool(sbl), align)
        want = g[k + "out"]
        want = want.view(np.uint32) if want.dtype == np.float32 else want
        np.testing.assert_array_equal(got, want, err_msg=k)

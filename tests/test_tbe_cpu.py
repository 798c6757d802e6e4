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

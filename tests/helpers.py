"""Input builders shared by the CPU and GPU tests (seeded numpy)."""
import numpy as np

# (batch, table rows, embedding dim, average bag length): the shapes the
# reference's lookup tests run (test/EmbeddingSpMDM8BitTest.cc:20-43,
# test/EmbeddingSpMDMNBitTest.cc:21-46 of FBGEMM).
REFERENCE_SHAPES = [
    (1, 8, 8, 4), (2, 8, 16, 4), (10, 4000, 32, 100), (100, 4000, 32, 100), (10, 4000, 64, 100),
    (10, 4000, 128, 100), (4, 400, 256, 10), (4, 400, 512, 10), (10, 4000, 48, 100), (10, 4000, 40, 100),
    (10, 4000, 56, 100), (10, 4000, 2, 100), (10, 4000, 4, 100), (10, 4000, 7, 100), (10, 40, 16, 10),
    (10, 40, 86, 10), (10, 40, 8, 10), (10, 40, 96, 10), (10, 40, 164, 10),
]


def row_bytes(bit_rate, dim):
    epb = 8 // bit_rate
    return (dim + epb - 1) // epb + (8 if bit_rate == 8 else 4)


def random_fused_table(rng, rows, dim, bit_rate, stride=None, scale_bias_first=False):
    """Rows as the reference tests build them: small random payload values and
    N(0,1) scale/bias (test/EmbeddingSpMDM8BitTest.cc:120-154,
    test/EmbeddingSpMDMNBitTest.cc:137-166) - not quantizer output, so every
    payload bit pattern and awkward scales occur.  ``scale_bias_first`` builds
    the table-batched layout (the generators' scale_bias_last = false): fp16
    scale and bias in the first four bytes of the row, for 8-bit rows too."""
    epb = 8 // bit_rate
    data_bytes = (dim + epb - 1) // epb
    half_sb = bit_rate != 8 or scale_bias_first
    sb_bytes = 4 if half_sb else 8
    stride = stride or data_bytes + sb_bytes
    data_at, sb_at = (sb_bytes, 0) if scale_bias_first else (0, data_bytes)
    t = np.zeros((rows, stride), dtype=np.uint8)
    t[:, data_at:data_at + data_bytes] = rng.integers(0, 256, (rows, data_bytes), dtype=np.uint8)
    sb = rng.standard_normal((rows, 2)).astype(np.float32)
    if half_sb:
        t[:, sb_at:sb_at + 4] = sb.astype(np.float16).view(np.uint8).reshape(rows, 4)
    else:
        t[:, sb_at:sb_at + 8] = sb.view(np.uint8).reshape(rows, 8)
    return t


def lengths_indices_weights(rng, batch, rows, avg_len, index_dtype, offset_dtype, corner=None):
    """As GenerateLengthsIndicesWeights (test/EmbeddingSpMDMTestUtils.cc:18-95),
    seeded.  corner: None, 'empty', 'oob', 'unmatched+', 'unmatched-'."""
    hi = min(2 * avg_len + 1, rows)
    lengths = np.zeros(batch, dtype=np.int64) if corner == "empty" else rng.integers(1, hi + 1, batch)
    n = int(lengths.sum())
    indices = rng.integers(0, rows, n).astype(index_dtype)
    if corner != "empty":
        indices[0] = rows - 1  # probe the upper bound
    if corner == "oob":
        indices[rng.integers(0, n)] = rows
    if corner == "unmatched+":
        lengths[-1] += 1
    if corner == "unmatched-":
        lengths[-1] -= 1
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(offset_dtype)
    weights = rng.standard_normal(n).astype(np.float32)
    return lengths.astype(offset_dtype), offsets, indices, weights, n


def mapping_table(rng, rows, sparsity):
    """As CreateMappingTableForRowWiseSparsity (test/EmbeddingSpMDMTestUtils.cc:97-109)."""
    pruned = rng.random(rows) < sparsity
    m = np.full(rows, -1, dtype=np.int32)
    m[~pruned] = np.arange(int((~pruned).sum()), dtype=np.int32)
    return m, int((~pruned).sum())


def random_plain_table(rng, rows, dim, in_kind, stride=None):
    """A table that is not row-wise quantized, [rows, stride] elements:
    "f32" float32, "f16"/"bf16" uint16 bit patterns of N(0,1) values (plus a few
    subnormals and zeros), "fp8" every uint8 pattern."""
    stride = stride or dim
    x = rng.standard_normal((rows, stride)).astype(np.float32)
    x[rng.integers(0, rows, 3), rng.integers(0, stride, 3)] = 0.0
    if in_kind == "f32":
        return x
    if in_kind == "f16":
        x[0, 0] = 3e-7  # a half subnormal
        return x.astype(np.float16).view(np.uint16)
    if in_kind == "bf16":
        return (x.view(np.uint32) >> 16).astype(np.uint16)
    return rng.integers(0, 256, (rows, stride), dtype=np.uint8)

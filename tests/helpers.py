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


def pruning_case(rng, T, B, max_len, idt, hdt, load_factor=0.8, unpruned_tables=()):
    """The reference test's construction
    (fbgemm_gpu/test/tbe/utils/split_embeddings_utils_test.py:476-620) with
    ragged bags: unique sparse indices per table, half of them pruned (dense
    index -1); tables in ``unpruned_tables`` get no hash map."""
    lengths = rng.integers(0, max_len + 1, size=T * B)
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(idt)
    n = int(offsets[-1])
    indices = np.zeros(n, dtype=idt)
    dense = np.zeros(n, dtype=idt)
    capacities = []
    for t in range(T):
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        cnt = hi - lo
        space = max(4 * cnt, 16)
        indices[lo:hi] = rng.choice(space, size=cnt, replace=False).astype(idt)
        d = rng.integers(0, 1000, size=cnt).astype(idt)
        d[rng.random(cnt) < 0.5] = -1
        dense[lo:hi] = d
        capacities.append(0 if t in unpruned_tables else int(cnt / load_factor) + 1)
    hto = np.concatenate([[0], np.cumsum(capacities)]).astype(np.int64)
    table = np.full((int(hto[-1]), 2), -1, dtype=hdt)
    return indices, dense, offsets, table, hto


# SparseType values of the table-batched operator (fbgemm_gpu/include/fbgemm_gpu/embedding_common.h:20-32)
ST_FP32, ST_FP16, ST_INT8, ST_INT4, ST_INT2, ST_BF16, ST_FP8 = range(7)
ST_BITS = {ST_INT8: 8, ST_INT4: 4, ST_INT2: 2}
ST_PLAIN = {ST_FP32: "f32", ST_FP16: "f16", ST_FP8: "fp8"}


def padded_row_bytes(dim, ty, row_alignment, scale_bias_bytes=4):
    """nbit::padded_row_size_in_bytes (embedding_common.h:189-225)."""
    if ty in ST_PLAIN:
        unpadded = dim * {"f32": 4, "f16": 2, "fp8": 1}[ST_PLAIN[ty]]
    else:
        unpadded = dim * ST_BITS[ty] // 8 + scale_bias_bytes
    return (unpadded + row_alignment - 1) // row_alignment * row_alignment


def build_op_inputs(rng, tys, dims, rows, B, mean_len, row_alignment, scale_bias_last, idt, prune=True):
    """Tables, index arrays and per-sample weights of one call of the
    table-batched operator: T tables in one byte blob, T*B+1 offsets.  With
    scale and bias first an eighth of the indices are -1 (pruned rows) unless
    ``prune`` is false."""
    T = len(tys)
    tables, offs_w, blob = [], [], []
    at = 0
    for ty, D, R in zip(tys, dims, rows):
        ty = int(ty)
        sb = 8 if (ty == ST_INT8 and scale_bias_last) else 4
        stride = padded_row_bytes(D, ty, row_alignment, sb)
        if ty in ST_PLAIN:
            eb = {"f32": 4, "f16": 2, "fp8": 1}[ST_PLAIN[ty]]
            t = random_plain_table(rng, R, D, ST_PLAIN[ty], stride // eb)
            t = t.view(np.uint8).reshape(R, stride)
        else:
            t = random_fused_table(rng, R, D, ST_BITS[ty], stride, not scale_bias_last)
        tables.append(t)
        offs_w.append(at)
        blob.append(t.reshape(-1))
        at += t.size
    lengths = rng.poisson(mean_len, T * B)
    lengths[rng.integers(0, T * B, 3)] = 0
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(idt)
    indices = np.concatenate([rng.integers(0, rows[t], int(lengths[t * B:(t + 1) * B].sum())) for t in range(T)]).astype(idt)
    if not scale_bias_last and prune:
        indices[rng.integers(0, len(indices), len(indices) // 8)] = -1   # pruned rows
    weights = rng.standard_normal(len(indices)).astype(np.float32)
    D_offsets = np.concatenate([[0], np.cumsum(dims)]).astype(np.int32)
    return tables, np.concatenate(blob), np.array(offs_w, np.int64), D_offsets, offsets, indices, weights


ST_OUT_KIND = {ST_FP32: "f32", ST_FP16: "f16", ST_BF16: "bf16"}


def _as_bits(a):
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


def oracle_op_forward(oracle, tys, dims, rows, blob, w_off, D_off, indices, offsets, weights, B, pooling_mean, out_ty,
                      scale_bias_last, row_alignment, fp8=(4, 7)):
    """The table-batched pooled operator composed from the oracle's
    single-table lookups the way the reference composes its kernel calls
    (fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:343-473):
    table t pools offsets[t*B : (t+1)*B+1] into columns D_off[t]:D_off[t+1] of
    a [B, total_D] output.  Returns the output's bit patterns."""
    total_D = int(D_off[-1])
    out = np.zeros((B, total_D), dtype=np.uint32 if out_ty == ST_FP32 else np.uint16)
    for t, ty in enumerate(int(x) for x in tys):
        D, R = int(dims[t]), int(rows[t])
        sb = 8 if (ty == ST_INT8 and scale_bias_last) else 4
        stride = padded_row_bytes(D, ty, row_alignment, sb)
        table = blob[int(w_off[t]):int(w_off[t]) + R * stride].reshape(R, stride)
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        w = weights[lo:hi] if weights is not None else None
        if ty in ST_PLAIN:
            eb = {"f32": 4, "f16": 2, "fp8": 1}[ST_PLAIN[ty]]
            view = table.reshape(-1).view({4: np.float32, 2: np.uint16, 1: np.uint8}[eb])
            ok, ref = oracle.spmdm_plain(ST_PLAIN[ty], D, R, view, indices[lo:hi], offsets[t * B:(t + 1) * B + 1], w,
                                         pooling_mean, ST_OUT_KIND[out_ty], False, True, -1, stride // eb, scale_bias_last,
                                         False, fp8[0], fp8[1])
        else:
            ok, ref = oracle.spmdm_ex(ST_BITS[ty], D, R, table, indices[lo:hi], offsets[t * B:(t + 1) * B + 1], w,
                                      pooling_mean, ST_OUT_KIND[out_ty], False, True, -1, stride, scale_bias_last, False)
        assert ok, f"table {t}"
        out[:, int(D_off[t]):int(D_off[t + 1])] = _as_bits(ref)[:B * D].reshape(B, D)
    return out


def oracle_sequence_forward(oracle, tys, D, rows, blob, w_off, indices, offsets, B, out_ty, scale_bias_last,
                            row_alignment, fp8=(4, 7)):
    """The sequence ("nobag") operator composed from the oracle: every index
    position is a bag of one (…cpu_template.cpp:206-520, nobag branch).
    Returns [len(indices), D] bit patterns."""
    out = np.zeros((len(indices), D), dtype=np.uint32 if out_ty == ST_FP32 else np.uint16)
    for t, ty in enumerate(int(x) for x in tys):
        R = int(rows[t])
        sb = 8 if (ty == ST_INT8 and scale_bias_last) else 4
        stride = padded_row_bytes(D, ty, row_alignment, sb)
        table = blob[int(w_off[t]):int(w_off[t]) + R * stride].reshape(R, stride)
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        idx = indices[lo:hi]
        ones = np.ones(len(idx), dtype=idx.dtype)
        if ty in ST_PLAIN:
            eb = {"f32": 4, "f16": 2, "fp8": 1}[ST_PLAIN[ty]]
            view = table.reshape(-1).view({4: np.float32, 2: np.uint16, 1: np.uint8}[eb])
            ok, ref = oracle.spmdm_plain(ST_PLAIN[ty], D, R, view, idx, ones, None, False, ST_OUT_KIND[out_ty], False,
                                         False, -1, stride // eb, scale_bias_last, False, fp8[0], fp8[1])
        else:
            ok, ref = oracle.spmdm_ex(ST_BITS[ty], D, R, table, idx, ones, None, False, ST_OUT_KIND[out_ty], False, False,
                                      -1, stride, scale_bias_last, False)
        assert ok, f"table {t}"
        out[lo:hi] = _as_bits(ref)[:(hi - lo) * D].reshape(hi - lo, D)
    return out


def load_golden(name):
    import os

    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))

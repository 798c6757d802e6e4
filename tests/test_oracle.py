"""Pins the CPU oracle (oracle/embedding_oracle.c): against the reference's
known-answer vectors, against fixtures generated from the reference's own code,
and - when the reference checker library is present - live against the
reference's scalar functions and its asmjit kernels.  Runs without a GPU."""
import os

import numpy as np
import pytest

from conftest import bits
from helpers import (REFERENCE_SHAPES, lengths_indices_weights, mapping_table, random_fused_table,
                     random_plain_table)

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lookup_golden.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


# ---- known-answer vectors -----------------------------------------------------

# The fixed-number quantizer test of the reference
# (EmbeddingQuantizeFixedNumberTest, test/QuantUtilsTest.cc:550-667): two rows
# of four values whose fused encodings were worked out by hand there.
KAT_INPUT = np.array([[1, 1, 1, 1], [-64, -2.75, 61.625, 191]], dtype=np.float32)
KAT_SBFLOAT_8 = np.array([
    [0, 0, 0, 0, 0x00, 0x00, 0x00, 0x00, 0x00, 0x00, 0x80, 0x3f],   # scale 0, bias 1
    [0, 61, 126, 255, 0x00, 0x00, 0x80, 0x3f, 0x00, 0x00, 0x80, 0xc2],  # scale 1, bias -64
], dtype=np.uint8)
KAT_SBHALF = {
    8: np.array([[0, 0, 0, 0, 0x00, 0x3c, 0x00, 0x3c], [0, 61, 126, 255, 0x00, 0x3c, 0x00, 0xd4]], dtype=np.uint8),
    4: np.array([[0x00, 0x00, 0x00, 0x3c, 0x00, 0x3c], [0x40, 0xf7, 0x40, 0x4c, 0x00, 0xd4]], dtype=np.uint8),
    2: np.array([[0b00000000, 0x00, 0x3c, 0x00, 0x3c], [0b11010100, 0x50, 0x55, 0x00, 0xd4]], dtype=np.uint8),
}


def test_quantizer_known_answers(oracle):
    np.testing.assert_array_equal(oracle.quantize_8bit(KAT_INPUT), KAT_SBFLOAT_8)
    for bit_rate, want in KAT_SBHALF.items():
        np.testing.assert_array_equal(oracle.quantize_nbit(bit_rate, KAT_INPUT), want)


def test_lookup_of_known_answer_rows(oracle):
    """Pooling the hand-computed rows: row 1 dequantizes to scale*q + bias =
    q - 64 (8-bit) and 17*q - 64 (4-bit), so sums are exact integers."""
    idx = np.array([1, 1, 0], dtype=np.int64)
    off = np.array([0, 2, 3], dtype=np.int64)
    ok, out = oracle.spmdm(8, 4, 2, KAT_SBFLOAT_8, idx, off)
    assert ok
    np.testing.assert_array_equal(out.reshape(2, 4), [[-128, -6, 124, 382], [1, 1, 1, 1]])
    ok, out = oracle.spmdm(4, 4, 2, KAT_SBHALF[4], idx, off)
    assert ok
    np.testing.assert_array_equal(out.reshape(2, 4), [[-128, 8, 110, 382], [1, 1, 1, 1]])
    ok, out = oracle.spmdm(2, 4, 2, KAT_SBHALF[2], idx, off)
    assert ok
    np.testing.assert_array_equal(out.reshape(2, 4), [[-128, 42, 42, 382], [1, 1, 1, 1]])


def test_half_conversion_known_values(oracle):
    for f, h in [(1.0, 0x3c00), (-64.0, 0xd400), (17.0, 0x4c40), (85.0, 0x5550), (65504.0, 0x7bff),
                 (65520.0, 0x7c00), (2.0 ** -24, 0x0001), (2.0 ** -25, 0x0000), (0.0, 0x0000), (-0.0, 0x8000),
                 (61.625, 0x53b4), (float("inf"), 0x7c00)]:
        assert oracle.float_to_half(f) == h, f
    for h in (0x3c00, 0xd400, 0x0001, 0x03ff, 0x0400, 0x7bff, 0x8000):
        assert oracle.half_to_float(h) == float(np.array([h], dtype=np.uint16).view(np.float16)[0])


def test_half_conversion_matches_numpy_everywhere(oracle):
    halves = np.arange(0x7c00, dtype=np.uint16)  # every finite non-negative half
    want = halves.view(np.float16).astype(np.float32)
    got = np.array([oracle.half_to_float(int(h)) for h in halves[::7]], dtype=np.float32)
    np.testing.assert_array_equal(got, want[::7])
    rng = np.random.default_rng(5)
    f = np.concatenate([rng.standard_normal(3000) * 10.0 ** rng.integers(-8, 5, 3000),
                        want[::11] * 1.0004883]).astype(np.float32)
    with np.errstate(over="ignore"):
        want_h = f.astype(np.float16).view(np.uint16)
    got_h = np.array([oracle.float_to_half(float(x)) for x in f], dtype=np.uint16)
    np.testing.assert_array_equal(got_h, want_h)


# ---- fixtures generated from the reference ------------------------------------------

def test_oracle_matches_reference_fixtures(oracle, golden):
    for i in range(int(golden["n_lookup"])):
        k = f"lookup{i}_"
        bit_rate, batch, rows, dim, weighted, positional, normalize, use_offsets = golden[k + "meta"]
        want = golden[k + "out"]
        ok, got = oracle.spmdm(int(bit_rate), int(dim), int(rows), golden[k + "table"], golden[k + "indices"],
                               golden[k + "ol"], golden[k + "weights"] if weighted else None, bool(normalize),
                               want.dtype, bool(positional), bool(use_offsets), output_size=int(batch))
        assert ok
        np.testing.assert_array_equal(bits(got[:want.size]), bits(want))
    for i in range(int(golden["n_sparse"])):
        k = f"sparse{i}_"
        bit_rate, batch, rows, dim, weighted = golden[k + "meta"]
        ok, got = oracle.spmdm_rowwise_sparse(int(bit_rate), int(dim), int(rows), golden[k + "table"],
                                              golden[k + "indices"], golden[k + "mapping"], golden[k + "offsets"],
                                              golden[k + "weights"] if weighted else None, True)
        assert ok
        np.testing.assert_array_equal(bits(got), bits(golden[k + "out"]))
    for i in range(int(golden["n_quant"])):
        x = golden[f"quant{i}_x"]
        np.testing.assert_array_equal(oracle.quantize_8bit(x), golden[f"quant{i}_q8"])
        np.testing.assert_array_equal(oracle.quantize_nbit(4, x), golden[f"quant{i}_q4"])
        np.testing.assert_array_equal(oracle.quantize_nbit(2, x), golden[f"quant{i}_q2"])
    ri, ro, rw = oracle.remap(golden["remap_indices"], golden["remap_mapping"], golden["remap_offsets"],
                              golden["remap_weights"])
    np.testing.assert_array_equal(ri, golden["remap_out_indices"])
    np.testing.assert_array_equal(ro, golden["remap_out_offsets"])
    np.testing.assert_array_equal(rw, golden["remap_out_weights"])


KINDS = ("f32", "f16", "bf16")


def run_ex_fixture(lookups, ex, i):
    """One case of lookup_ex_golden.npz through `lookups.spmdm_ex`; returns (ok, got, want)."""
    k = f"ex{i}_"
    bit_rate, count, rows, dim, weighted, normalize, sb_last, no_bag, kind = (int(v) for v in ex[k + "meta"])
    table = ex[k + "table"]
    ok, got = lookups.spmdm_ex(bit_rate, dim, rows, table, ex[k + "indices"], None if no_bag else ex[k + "offsets"],
                               ex[k + "weights"] if weighted else None, bool(normalize), KINDS[kind], False, True, -1,
                               table.shape[1], bool(sb_last), bool(no_bag))
    return ok, got[:count * dim], ex[k + "out"]


def test_oracle_ex_matches_reference_fixtures(oracle):
    """Rows with scale, bias first and -1 as a pruned index, bf16 output,
    padded rows, no_bag: fixtures made by the reference's own functions."""
    ex = np.load(os.path.join(os.path.dirname(GOLDEN), "lookup_ex_golden.npz"))
    assert int(ex["n_ex"]) >= 20
    for i in range(int(ex["n_ex"])):
        ok, got, want = run_ex_fixture(oracle, ex, i)
        assert ok
        np.testing.assert_array_equal(bits(got), bits(want))


IN_KINDS = ("f32", "f16", "bf16", "fp8")


def run_plain_fixture(lookups, ex, i):
    """One plain-row case of lookup_ex_golden.npz through `lookups.spmdm_plain`."""
    k = f"plain{i}_"
    in_kind, count, rows, dim, weighted, normalize, sb_last, no_bag, kind, ebits, ebias = (int(v) for v in ex[k + "meta"])
    table = ex[k + "table"]
    ok, got = lookups.spmdm_plain(IN_KINDS[in_kind], dim, rows, table, ex[k + "indices"],
                                  None if no_bag else ex[k + "offsets"], ex[k + "weights"] if weighted else None,
                                  bool(normalize), KINDS[kind], False, True, -1, table.shape[1], bool(sb_last),
                                  bool(no_bag), ebits, ebias)
    return ok, got[:count * dim], ex[k + "out"]


def test_oracle_plain_rows_match_reference_fixtures(oracle):
    ex = np.load(os.path.join(os.path.dirname(GOLDEN), "lookup_ex_golden.npz"))
    assert int(ex["n_plain"]) >= 9
    for i in range(int(ex["n_plain"])):
        ok, got, want = run_plain_fixture(oracle, ex, i)
        assert ok
        np.testing.assert_array_equal(bits(got), bits(want))


SPARSE_KINDS = ("f32", "f16", "u16")


def run_sparse_plain_fixture(lookups, ex, i):
    """One pruned plain-row case of lookup_ex_golden.npz."""
    k = f"sparse{i}_"
    in_kind, batch, urows, dim, weighted, normalize = (int(v) for v in ex[k + "meta"])
    ok, got = lookups.spmdm_plain_rowwise_sparse(SPARSE_KINDS[in_kind], dim, urows, ex[k + "table"], ex[k + "indices"],
                                                 ex[k + "cit"], ex[k + "offsets"],
                                                 ex[k + "weights"] if weighted else None, bool(normalize))
    return ok, got[:batch * dim], ex[k + "out"]


def test_oracle_pruned_plain_rows_match_reference_fixtures(oracle):
    ex = np.load(os.path.join(os.path.dirname(GOLDEN), "lookup_ex_golden.npz"))
    assert int(ex["n_sparse"]) >= 5
    for i in range(int(ex["n_sparse"])):
        ok, got, want = run_sparse_plain_fixture(oracle, ex, i)
        assert ok
        np.testing.assert_array_equal(bits(got), bits(want))


# ---- live against the reference's own code ------------------------------------------

@pytest.mark.parametrize("bit_rate", [8, 4, 2])
def test_oracle_matches_reference_live(oracle, reference, bit_rate):
    rng = np.random.default_rng(40 + bit_rate)
    for shape_i, (batch, rows, dim, avg_len) in enumerate(REFERENCE_SHAPES):
        for corner in (None, "empty", "oob", "unmatched+", "unmatched-"):
            idt, odt = ((np.int32, np.int64), (np.int64, np.int32))[shape_i % 2]
            table = random_fused_table(rng, rows, dim, bit_rate)
            lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, odt, corner)
            for weighted, normalize, use_offsets, out_dt in ((False, False, True, np.float32),
                                                             (True, True, False, np.float16)):
                ol = offsets if use_offsets else lengths
                args = (bit_rate, dim, rows, table, indices, ol, weights if weighted else None, normalize, out_dt,
                        False, use_offsets)
                a = oracle.spmdm(*args, output_size=batch, index_size=n)
                b = reference.spmdm(*args, output_size=batch, index_size=n)
                assert a[0] == b[0] == (corner in (None, "empty"))
                if a[0]:
                    np.testing.assert_array_equal(bits(a[1]), bits(b[1]))
        mapping, dense = mapping_table(rng, rows, 0.7)
        table = random_fused_table(rng, max(dense, 1), dim, bit_rate)
        lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, np.int64, np.int64)
        a = oracle.spmdm_rowwise_sparse(bit_rate, dim, rows, table, indices, mapping, offsets, weights, True)
        b = reference.spmdm_rowwise_sparse(bit_rate, dim, rows, table, indices, mapping, offsets, weights, True)
        assert a[0] and b[0]
        np.testing.assert_array_equal(bits(a[1]), bits(b[1]))


def test_oracle_quantizers_match_reference_live(oracle, reference):
    rng = np.random.default_rng(77)
    for rows, cols in ((50, 128), (33, 64), (20, 8), (9, 36)):
        x = (rng.standard_normal((rows, cols)) * 10.0 ** rng.integers(-3, 3, (rows, 1))).astype(np.float32)
        x[3] = -1.5
        np.testing.assert_array_equal(oracle.quantize_8bit(x), reference.quantize_8bit(x))
        np.testing.assert_array_equal(oracle.quantize_8bit(x), reference.quantize_8bit(x, use_ref=False))
        for b in (2, 4):
            np.testing.assert_array_equal(oracle.quantize_nbit(b, x), reference.quantize_nbit(b, x))
            np.testing.assert_array_equal(oracle.quantize_nbit(b, x), reference.quantize_nbit(b, x, use_ref=False))


def test_reference_jit_matches_oracle(oracle):
    """The reference's asmjit kernels (reached through libtorch_cpu.so) are the
    timed CPU baseline; they agree bit for bit with the scalar restatement."""
    from oracle import checker

    jit = checker.ReferenceJit()
    if not jit.available:
        pytest.skip("oracle/_ref/libfbgemm_jit.so not built")
    rng = np.random.default_rng(99)
    for bit_rate, dim in ((8, 128), (4, 64), (2, 128), (8, 40), (4, 86)):
        rows, batch = 800, 40
        table = random_fused_table(rng, rows, dim, bit_rate)
        lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 20, np.int64, np.int64)
        for weighted, normalize, out_dt in ((False, False, np.float32), (True, True, np.float16)):
            a = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, weights if weighted else None, normalize,
                             out_dt)
            b = jit.spmdm(bit_rate, dim, rows, table, indices, offsets, weights if weighted else None, normalize,
                          out_dt)
            assert a[0] and b[0]
            np.testing.assert_array_equal(bits(a[1]), bits(b[1]))
            # the benchmark's CPU leg: the same batch split over OpenMP threads by bag ranges
            par = np.zeros_like(a[1])
            assert jit.batch_parallel(bit_rate, dim, rows, table, indices, offsets, weights if weighted else None,
                                      normalize, par, 3)
            np.testing.assert_array_equal(bits(par), bits(a[1]))


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
def test_oracle_ex_matches_reference_live(oracle, reference, bit_rate):
    rng = np.random.default_rng(140 + bit_rate)
    for shape_i, (batch, rows, dim, avg_len) in enumerate(REFERENCE_SHAPES[2:12]):
        for sb_last in (True, False):
            for corner in (None, "oob", "unmatched-"):
                idt = (np.int32, np.int64)[shape_i % 2]
                table = random_fused_table(rng, rows, dim, bit_rate, None, not sb_last)
                lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, idt, corner)
                if corner is None:
                    indices[rng.integers(0, n, max(1, n // 6))] = -1  # pruned when scale, bias come first; else an error
                for kind, weighted, normalize, use_offsets in (("f32", False, True, True), ("bf16", True, False, False),
                                                               ("f16", True, True, True)):
                    ol = offsets if use_offsets else lengths
                    args = (bit_rate, dim, rows, table, indices, ol, weights if weighted else None, normalize, kind,
                            False, use_offsets, -1, -1, sb_last, False)
                    a = oracle.spmdm_ex(*args, output_size=batch, index_size=n)
                    b = reference.spmdm_ex(*args, output_size=batch, index_size=n)
                    assert a[0] == b[0] == (corner is None and not sb_last)
                    if a[0]:
                        np.testing.assert_array_equal(bits(a[1]), bits(b[1]))
        if bit_rate == 8:
            for sb_last in (True, False):
                table = random_fused_table(rng, rows, dim, 8, None, not sb_last)
                indices = rng.integers(0, rows, 3 * batch).astype(np.int64)
                weights = rng.standard_normal(3 * batch).astype(np.float32)
                for kind, weighted in (("f32", True), ("f16", False), ("bf16", True)):
                    args = (8, dim, rows, table, indices, None, weights if weighted else None, True, kind, False, True,
                            -1, -1, sb_last, True)
                    a, b = oracle.spmdm_ex(*args), reference.spmdm_ex(*args)
                    assert a[0] and b[0]
                    np.testing.assert_array_equal(bits(a[1]), bits(b[1]))
                indices[5] = rows
                assert not oracle.spmdm_ex(8, dim, rows, table, indices, None, None, False, "f32", False, True, -1, -1,
                                           sb_last, True)[0]
                assert not reference.spmdm_ex(8, dim, rows, table, indices, None, None, False, "f32", False, True, -1, -1,
                                              sb_last, True)[0]


@pytest.mark.parametrize("in_kind", IN_KINDS)
def test_oracle_plain_rows_match_reference_live(oracle, reference, in_kind):
    rng = np.random.default_rng(240 + IN_KINDS.index(in_kind))
    for shape_i, (batch, rows, dim, avg_len) in enumerate(REFERENCE_SHAPES[2:14]):
        for corner in (None, "oob"):
            idt = (np.int32, np.int64)[shape_i % 2]
            sb_last = shape_i % 3 != 0
            table = random_plain_table(rng, rows, dim, in_kind)
            lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, idt, corner)
            if corner is None and not sb_last and in_kind != "fp8":
                indices[rng.integers(0, n, max(1, n // 6))] = -1
            ebits, ebias = ((4, 7), (5, 15))[shape_i % 2]
            for kind, weighted, normalize, use_offsets in (("f32", False, True, True), ("bf16", True, False, False),
                                                           ("f16", True, True, True)):
                ol = offsets if use_offsets else lengths
                args = (in_kind, dim, rows, table, indices, ol, weights if weighted else None, normalize, kind, False,
                        use_offsets, -1, -1, sb_last, False, ebits, ebias)
                a = oracle.spmdm_plain(*args, output_size=batch, index_size=n)
                b = reference.spmdm_plain(*args, output_size=batch, index_size=n)
                assert a[0] == b[0] == (corner is None)
                if a[0]:
                    np.testing.assert_array_equal(bits(a[1]), bits(b[1]))
        if in_kind != "fp8":
            table = random_plain_table(rng, rows, dim, in_kind)
            indices = rng.integers(0, rows, 2 * batch).astype(np.int64)
            weights = rng.standard_normal(2 * batch).astype(np.float32)
            args = (in_kind, dim, rows, table, indices, None, weights, True, "f16", False, True, -1, -1, True, True)
            a, b = oracle.spmdm_plain(*args), reference.spmdm_plain(*args)
            assert a[0] and b[0]
            np.testing.assert_array_equal(bits(a[1]), bits(b[1]))


@pytest.mark.parametrize("in_kind", SPARSE_KINDS)
def test_oracle_pruned_plain_rows_match_reference_live(oracle, reference, in_kind):
    rng = np.random.default_rng(270 + SPARSE_KINDS.index(in_kind))
    for shape_i, (batch, urows, dim, avg_len) in enumerate(REFERENCE_SHAPES[2:12]):
        cit, rows = mapping_table(rng, urows, (0.5, 0.9, 0.0)[shape_i % 3])
        table = random_plain_table(rng, max(rows, 1), dim, "f32" if in_kind == "f32" else "f16")
        for corner in (None, "oob", "unmatched+"):
            idt, odt = ((np.int32, np.int64), (np.int64, np.int32))[shape_i % 2]
            lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, urows, avg_len, idt, odt, corner)
            for weighted, normalize, positional, use_offsets in ((False, True, False, True), (True, False, False, False),
                                                                 (True, True, True, True)):
                args = (in_kind, dim, urows, table, indices, cit, offsets if use_offsets else lengths,
                        weights if weighted else None, normalize, positional, use_offsets)
                a = oracle.spmdm_plain_rowwise_sparse(*args)
                b = reference.spmdm_plain_rowwise_sparse(*args)
                assert a[0] == b[0] == (corner is None)
                if a[0]:
                    np.testing.assert_array_equal(bits(a[1]), bits(b[1]))

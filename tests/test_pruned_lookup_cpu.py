"""Index remapping of table-batched pruned tables, CPU side: the oracle's
restatement of pruned_hashmap_insert / pruned_hashmap_lookup /
pruned_array_lookup (fbgemm_gpu/codegen/inference/
embedding_forward_quantized_cpu_template.cpp:102-204, :524-659 of FBGEMM)
against fixtures made by the reference's own compiled functions
(tests/golden/make_golden_tbe.py; live against that library where it was
built), the property the reference's own test checks
(fbgemm_gpu/test/tbe/utils/split_embeddings_utils_test.py:476-620), the hash
against an independent statement of the MurmurHash3 finalisers, and the
library's host-side insert against the oracle's (same table bytes)."""
import ctypes as C

import numpy as np
import pytest

from fbgemm_b200 import _capi
from helpers import pruning_case


def fmix32(h):
    h &= 0xFFFFFFFF
    h ^= h >> 16
    h = (h * 0x85EBCA6B) & 0xFFFFFFFF
    h ^= h >> 13
    h = (h * 0xC2B2AE35) & 0xFFFFFFFF
    h ^= h >> 16
    return h


def fmix64(k):
    m = 2 ** 64 - 1
    k &= m
    k ^= k >> 33
    k = (k * 0xFF51AFD7ED558CCD) & m
    k ^= k >> 33
    k = (k * 0xC4CEB9FE1A85EC53) & m
    k ^= k >> 33
    return k


def test_hash_is_the_murmur3_finaliser(oracle):
    rng = np.random.default_rng(77)
    for key in [0, 1, 2, 0x7FFFFFFF, 0xFFFFFFFF, 12345678] + [int(x) for x in rng.integers(0, 2 ** 31, 20)]:
        assert oracle.pruned_hash(key, 4) == fmix32(key)
    for key in [0, 1, 2 ** 63 - 1, 2 ** 64 - 1, 0x123456789ABCDEF] + [int(x) for x in rng.integers(0, 2 ** 62, 20)]:
        assert oracle.pruned_hash(key, 8) == fmix64(key)
    assert fmix32(1) == 0x514E28B7  # the published finaliser's value for 1


@pytest.mark.parametrize("idt", [np.int32, np.int64])
@pytest.mark.parametrize("hdt", [np.int32, np.int64])
def test_insert_then_lookup(oracle, idt, hdt):
    rng = np.random.default_rng(500 + np.dtype(idt).itemsize + 3 * np.dtype(hdt).itemsize)
    for T, B, max_len in ((1, 1, 5), (3, 7, 8), (5, 40, 20), (2, 300, 6)):
        indices, dense, offsets, table, hto = pruning_case(rng, T, B, max_len, idt, hdt, unpruned_tables=(1,))
        assert oracle.pruned_hashmap_insert(T, B, indices, dense, offsets, table, hto)
        got = oracle.pruned_hashmap_lookup(T, B, indices, offsets, table, hto)
        want = dense.copy()
        if T > 1:  # table 1 has no hash table: its indices pass through
            lo, hi = int(offsets[B]), int(offsets[2 * B])
            want[lo:hi] = indices[lo:hi]
        np.testing.assert_array_equal(got, want)
        # keys that were never inserted are pruned rows
        absent = np.full_like(indices, np.iinfo(np.int32).max)
        got = oracle.pruned_hashmap_lookup(T, B, absent, offsets, table, hto)
        want = np.full_like(indices, -1)
        if T > 1:
            want[lo:hi] = absent[lo:hi]
        np.testing.assert_array_equal(got, want)


def test_slot_layout_follows_hash_and_linear_probing(oracle):
    # three keys with the same first slot in a table of 5: they sit in consecutive slots in insertion order
    cap = 5
    keys, k = [], 0
    while len(keys) < 3:
        if fmix32(k) % cap == 3:
            keys.append(k)
        k += 1
    indices = np.array(keys, dtype=np.int32)
    dense = np.array([10, 11, 12], dtype=np.int32)
    offsets = np.array([0, 3], dtype=np.int32)
    table = np.full((cap, 2), -1, dtype=np.int64)
    assert oracle.pruned_hashmap_insert(1, 1, indices, dense, offsets, table, np.array([0, cap]))
    assert table[3].tolist() == [keys[0], 10] and table[4].tolist() == [keys[1], 11] and table[0].tolist() == [keys[2], 12]
    # a full table that lacks the key: the probe gives up with -1 (the reference would not return)
    full = np.array([[1, 1], [2, 2], [3, 3]], dtype=np.int64)
    got = oracle.pruned_hashmap_lookup(1, 1, np.array([99], dtype=np.int32), np.array([0, 1], dtype=np.int32), full,
                                       np.array([0, 3]))
    assert got.tolist() == [-1]


@pytest.mark.parametrize("idt", [np.int32, np.int64])
def test_array_lookup(oracle, idt):
    rng = np.random.default_rng(640)
    T, B = 4, 30
    lengths = rng.integers(0, 9, size=T * B)
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(idt)
    sizes = [50, 0, 200, 7]
    ro = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    remap = rng.integers(-1, 40, size=int(ro[-1])).astype(np.int64)
    indices = np.zeros(int(offsets[-1]), dtype=idt)
    want = np.zeros_like(indices)
    for t in range(T):
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        indices[lo:hi] = rng.integers(0, max(sizes[t], 1000 if sizes[t] == 0 else sizes[t]), hi - lo)
        want[lo:hi] = indices[lo:hi] if sizes[t] == 0 else remap[ro[t] + indices[lo:hi]]
    ok, got = oracle.pruned_array_lookup(T, B, indices, offsets, remap, ro)
    assert ok
    np.testing.assert_array_equal(got, want)
    indices[int(offsets[-1]) - 1] = 7  # one past table 3's array
    ok, got = oracle.pruned_array_lookup(T, B, indices, offsets, remap, ro)
    assert not ok and got[-1] == -1


@pytest.mark.parametrize("idt", [np.int32, np.int64])
@pytest.mark.parametrize("hdt", [np.int32, np.int64])
def test_library_insert_builds_the_same_table(oracle, idt, hdt):
    """The host-side insert the library ships fills the table exactly as the
    oracle's restatement does (it needs no GPU)."""
    rng = np.random.default_rng(900 + np.dtype(idt).itemsize + 3 * np.dtype(hdt).itemsize)
    lib = _capi.lib()
    for T, B, max_len in ((1, 4, 5), (4, 25, 12), (3, 200, 7)):
        indices, dense, offsets, table, hto = pruning_case(rng, T, B, max_len, idt, hdt, unpruned_tables=(0,))
        ours = table.copy()
        assert oracle.pruned_hashmap_insert(T, B, indices, dense, offsets, table, hto)
        rc = lib.fbgemm_b200_pruned_hashmap_insert_host(
            T, B, indices.ctypes.data, dense.ctypes.data, offsets.ctypes.data, indices.dtype.itemsize,
            ours.ctypes.data, ours.dtype.itemsize, hto.ctypes.data)
        assert rc == 1
        np.testing.assert_array_equal(ours, table)
    # a table with no free slot: returns 0 instead of probing for ever
    indices = np.arange(4, dtype=idt)
    dense = np.arange(4, dtype=idt)
    offsets = np.array([0, 4], dtype=idt)
    small = np.full((3, 2), -1, dtype=hdt)
    hto = np.array([0, 3], dtype=np.int64)
    rc = lib.fbgemm_b200_pruned_hashmap_insert_host(1, 1, indices.ctypes.data, dense.ctypes.data, offsets.ctypes.data,
                                                    indices.dtype.itemsize, small.ctypes.data, small.dtype.itemsize,
                                                    hto.ctypes.data)
    assert rc == 0 and (small[:, 0] != -1).all()
    assert lib.fbgemm_b200_pruned_hashmap_insert_host(0, 1, None, None, None, 4, None, 8, None) < 0


def test_oracle_matches_the_reference_fixtures(oracle):
    """oracle_pruned_* against tables and answers produced by the reference's
    own pruned_hashmap_insert_unweighted_cpu, pruned_hashmap_lookup_unweighted_cpu
    and pruned_array_lookup_cpu (tests/golden/make_golden_tbe.py)."""
    from helpers import load_golden

    g = load_golden("tbe_golden.npz")
    assert int(g["n_hash"]) >= 12 and int(g["n_arr"]) >= 4
    for i in range(int(g["n_hash"])):
        k = f"hash{i}_"
        T, B = (int(x) for x in g[k + "meta"])
        table = np.full_like(g[k + "table"], -1)
        assert oracle.pruned_hashmap_insert(T, B, g[k + "indices"], g[k + "dense"], g[k + "offsets"], table, g[k + "hto"])
        np.testing.assert_array_equal(table, g[k + "table"], err_msg=k)   # same slots, not only the same answers
        np.testing.assert_array_equal(
            oracle.pruned_hashmap_lookup(T, B, g[k + "indices"], g[k + "offsets"], table, g[k + "hto"]), g[k + "lookup"])
        np.testing.assert_array_equal(
            oracle.pruned_hashmap_lookup(T, B, g[k + "probe"], g[k + "offsets"], table, g[k + "hto"]),
            g[k + "probe_lookup"])
    for i in range(int(g["n_arr"])):
        k = f"arr{i}_"
        T, B = (int(x) for x in g[k + "meta"])
        ok, got = oracle.pruned_array_lookup(T, B, g[k + "indices"], g[k + "offsets"], g[k + "remap"], g[k + "ro"])
        assert ok
        np.testing.assert_array_equal(got, g[k + "lookup"], err_msg=k)


@pytest.mark.parametrize("idt", [np.int32, np.int64])
@pytest.mark.parametrize("hdt", [np.int32, np.int64])
def test_oracle_matches_the_compiled_reference_live(oracle, idt, hdt):
    """Fresh random cases against the reference's compiled template, where that
    library was built (it needs the reference tree at build time)."""
    from oracle import checker

    ref = checker.ReferenceTbe()
    if not ref.available:
        pytest.skip("oracle/_ref/libfbgemm_tbe_ref.so not built")
    rng = np.random.default_rng(4100 + np.dtype(idt).itemsize + 3 * np.dtype(hdt).itemsize)
    for T, B, max_len, lf in ((1, 1, 5, 0.8), (5, 40, 20, 0.5), (3, 200, 9, 0.95)):
        indices, dense, offsets, table, hto = pruning_case(rng, T, B, max_len, idt, hdt, lf,
                                                           unpruned_tables=(1,) if T > 1 else ())
        ours = table.copy()
        ref.pruned_hashmap_insert(T, B, indices, dense, offsets, table, hto)
        assert oracle.pruned_hashmap_insert(T, B, indices, dense, offsets, ours, hto)
        np.testing.assert_array_equal(ours, table)
        for probe in (indices, indices[::-1].copy(), np.full_like(indices, 2 ** 31 - 1), -indices - 1):
            np.testing.assert_array_equal(oracle.pruned_hashmap_lookup(T, B, probe, offsets, ours, hto),
                                          ref.pruned_hashmap_lookup(T, B, probe, offsets, table, hto))

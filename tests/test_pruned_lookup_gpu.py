"""pruned_hashmap_lookup / pruned_array_lookup on the GPU against the CPU
oracle (bit-exact: integer work) and the property the reference's own test
checks (fbgemm_gpu/test/tbe/utils/split_embeddings_utils_test.py:476-620 of
FBGEMM): insert, then every inserted index looks up its dense index and any
other index -1."""
import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from fbgemm_b200 import tbe
from helpers import pruning_case

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("idt", [np.int32, np.int64])
@pytest.mark.parametrize("hdt", [np.int32, np.int64])
def test_hashmap_lookup_against_the_oracle(gpu_ctx, oracle, idt, hdt):
    rng = np.random.default_rng(1500 + np.dtype(idt).itemsize + 3 * np.dtype(hdt).itemsize)
    for T, B, max_len, lf in ((1, 1, 5, 0.8), (3, 7, 8, 0.8), (5, 40, 20, 0.5), (2, 3000, 6, 0.8), (64, 200, 30, 0.95),
                              (2500, 1, 3, 0.8)):  # the last: more tables than the kernel stages in shared memory
        indices, dense, offsets, table, hto = pruning_case(rng, T, B, max_len, idt, hdt, lf,
                                                           unpruned_tables=(1,) if T > 1 else ())
        ti, td, to = torch.from_numpy(indices), torch.from_numpy(dense), torch.from_numpy(offsets)
        tt, th = torch.from_numpy(table), torch.from_numpy(hto)
        assert tbe.pruned_hashmap_insert(ti, td, to, tt, th)      # fills `table` in place (shared memory with tt)
        want = oracle.pruned_hashmap_lookup(T, B, indices, offsets, table, hto)
        got = tbe.pruned_hashmap_lookup(ti.cuda(), to.cuda(), tt.cuda(), th.cuda())
        np.testing.assert_array_equal(got.cpu().numpy(), want)
        expect = dense.copy()
        if T > 1:
            lo, hi = int(offsets[B]), int(offsets[2 * B])
            expect[lo:hi] = indices[lo:hi]
        np.testing.assert_array_equal(want, expect)
        # absent keys, negative keys
        for fill in (np.iinfo(np.int32).max, -1, -5):
            other = np.full_like(indices, fill)
            want = oracle.pruned_hashmap_lookup(T, B, other, offsets, table, hto)
            got = tbe.pruned_hashmap_lookup(dev(other), to.cuda(), tt.cuda(), th.cuda())
            np.testing.assert_array_equal(got.cpu().numpy(), want)
        assert F.status_read(0)[0]


def test_a_full_table_without_the_key_ends_with_minus_one(gpu_ctx):
    full = np.array([[1, 1], [2, 2], [3, 3]], dtype=np.int64)
    got = tbe.pruned_hashmap_lookup(dev(np.array([99, 2], dtype=np.int32)), dev(np.array([0, 2], dtype=np.int32)),
                                    dev(full), dev(np.array([0, 3], dtype=np.int64)))
    assert got.cpu().tolist() == [-1, 2]


def test_positions_outside_the_offsets_are_left_alone(gpu_ctx, oracle):
    rng = np.random.default_rng(1600)
    indices, dense, offsets, table, hto = pruning_case(rng, 3, 10, 6, np.int64, np.int64)
    assert oracle.pruned_hashmap_insert(3, 10, indices, dense, offsets, table, hto)
    shift, tail = 11, 5
    idx2 = np.concatenate([np.zeros(shift, np.int64), indices, np.zeros(tail, np.int64)])
    off2 = offsets + shift
    ctx = F.get_context(0)
    out = torch.full((len(idx2),), -7, dtype=torch.int64, device="cuda")
    from fbgemm_b200 import _capi
    d_idx, d_off, d_table, d_hto = dev(idx2), dev(off2), dev(table), dev(hto)
    rc = _capi.lib().fbgemm_b200_pruned_hashmap_lookup(
        ctx.handle, 3, 10, d_idx.data_ptr(), d_off.data_ptr(), 8, len(idx2), d_table.data_ptr(), 8,
        d_hto.data_ptr(), out.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    got = out.cpu().numpy()
    assert (got[:shift] == -7).all() and (got[len(idx2) - tail:] == -7).all()
    np.testing.assert_array_equal(got[shift:shift + len(indices)], dense)


@pytest.mark.parametrize("idt", [np.int32, np.int64])
@pytest.mark.parametrize("rdt", [np.int32, np.int64])
def test_array_lookup_against_the_oracle(gpu_ctx, oracle, idt, rdt):
    rng = np.random.default_rng(1700 + np.dtype(idt).itemsize + 3 * np.dtype(rdt).itemsize)
    for T, B, max_len in ((1, 1, 4), (4, 30, 8), (16, 2000, 12)):
        lengths = rng.integers(0, max_len + 1, size=T * B)
        offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(idt)
        sizes = [0 if t % 4 == 1 else int(rng.integers(5, 5000)) for t in range(T)]
        ro = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        remap = rng.integers(-1, 4000, size=max(int(ro[-1]), 1)).astype(rdt)
        indices = np.zeros(int(offsets[-1]), dtype=idt)
        for t in range(T):
            lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
            indices[lo:hi] = rng.integers(0, sizes[t] if sizes[t] else 100000, hi - lo)
        ok, want = oracle.pruned_array_lookup(T, B, indices, offsets, remap, ro)
        assert ok
        got = tbe.pruned_array_lookup(dev(indices), dev(offsets), dev(remap), dev(ro), slot=3)
        np.testing.assert_array_equal(got.cpu().numpy(), want)
        assert F.status_read(3)[0]
        if len(indices) and sizes[-1]:
            indices[-1] = sizes[-1]  # one past the last table's array: reported, -1, nothing read
            ok, want = oracle.pruned_array_lookup(T, B, indices, offsets, remap, ro)
            assert not ok
            got = tbe.pruned_array_lookup(dev(indices), dev(offsets), dev(remap), dev(ro), slot=3)
            np.testing.assert_array_equal(got.cpu().numpy(), want)
            ok_gpu, info = F.status_read(3)
            assert not ok_gpu and info[2] == len(indices) - 1


def test_remap_then_lookup_equals_the_minus_one_lookup(gpu_ctx, oracle):
    """The table-batched flow: hash-map remapping, then the table-batched
    lookup in which -1 is a pruned row, against the oracle on the dense indices."""
    rng = np.random.default_rng(1800)
    T, B, D, rows = 3, 64, 32, 500
    indices, dense, offsets, table, hto = pruning_case(rng, T, B, 10, np.int32, np.int64)
    dense = np.where(dense >= 0, dense % rows, -1).astype(np.int32)
    assert oracle.pruned_hashmap_insert(T, B, indices, dense, offsets, table, hto)
    got = tbe.pruned_hashmap_lookup(dev(indices), dev(offsets), dev(table), dev(hto))
    np.testing.assert_array_equal(got.cpu().numpy(), dense)
    row_bytes = tbe.padded_row_size_in_bytes(D, tbe.SparseType.INT4, 16)
    weights = rng.integers(0, 256, size=(T, rows, row_bytes), dtype=np.uint8)
    weights[:, :, 1] &= 0x3B  # keep the fp16 scale and bias finite
    weights[:, :, 3] &= 0x3B
    op = tbe.IntNBitTableBatchedEmbeddingBags(
        dev(weights.reshape(-1)), [t * rows * row_bytes for t in range(T)], [tbe.SparseType.INT4] * T,
        [t * D for t in range(T + 1)], T * D, tbe.PoolingMode.SUM, 16, tbe.SparseType.FP32)
    out = op.forward(got, dev(offsets)).cpu().numpy()
    for t in range(T):
        lo, hi = int(offsets[t * B]), int(offsets[(t + 1) * B])
        ok, want = oracle.spmdm_ex(4, D, rows, weights[t].reshape(-1), dense[lo:hi], offsets[t * B:(t + 1) * B + 1],
                                   None, False, "f32", False, True, -1, row_bytes, False, False)
        assert ok
        np.testing.assert_array_equal(np.ascontiguousarray(out[:, t * D:(t + 1) * D]).view(np.uint32).reshape(-1),
                                      want.view(np.uint32))


@pytest.mark.parametrize("idt", [np.int32, np.int64])
@pytest.mark.parametrize("hdt", [np.int32, np.int64])
def test_insert_on_the_device(gpu_ctx, oracle, idt, hdt):
    """The table a kernel fills by compare-and-swap need not equal the host-built one slot for slot, but
    it holds the same keys, and both the GPU lookup and the oracle's lookup read the same answers from it."""
    rng = np.random.default_rng(1900 + np.dtype(idt).itemsize + 3 * np.dtype(hdt).itemsize)
    for T, B, max_len, lf in ((1, 1, 5, 0.8), (4, 50, 12, 0.8), (3, 4000, 8, 0.95), (2, 2000, 10, 1.0)):
        indices, dense, offsets, table, hto = pruning_case(rng, T, B, max_len, idt, hdt, lf,
                                                           unpruned_tables=(1,) if T > 1 else ())
        d_idx, d_dense, d_off, d_hto = dev(indices), dev(dense), dev(offsets), dev(hto)
        d_table = dev(table) if table.size else torch.empty((0, 2), dtype=torch.int64 if hdt == np.int64 else torch.int32,
                                                            device="cuda")
        assert tbe.pruned_hashmap_insert(d_idx, d_dense, d_off, d_table, d_hto, slot=5)
        built = d_table.cpu().numpy()
        host = table.copy()
        assert oracle.pruned_hashmap_insert(T, B, indices, dense, offsets, host, hto)
        for t in range(T):   # the same keys with the same dense indices in every table
            lo, hi = int(hto[t]), int(hto[t + 1])
            got = {int(k): int(v) for k, v in built[lo:hi] if k != -1}
            want = {int(k): int(v) for k, v in host[lo:hi] if k != -1}
            assert got == want
            assert int((built[lo:hi, 0] != -1).sum()) == len(want)   # no key twice
        expect = oracle.pruned_hashmap_lookup(T, B, indices, offsets, host, hto)
        np.testing.assert_array_equal(oracle.pruned_hashmap_lookup(T, B, indices, offsets, built, hto), expect)
        np.testing.assert_array_equal(tbe.pruned_hashmap_lookup(d_idx, d_off, d_table, d_hto).cpu().numpy(), expect)
        other = np.full_like(indices, np.iinfo(np.int32).max)
        np.testing.assert_array_equal(tbe.pruned_hashmap_lookup(dev(other), d_off, d_table, d_hto).cpu().numpy(),
                                      oracle.pruned_hashmap_lookup(T, B, other, offsets, host, hto))
    # a table with fewer slots than keys: reported, nothing written outside it
    indices = np.arange(6, dtype=idt)
    small = torch.full((4, 2), -1, dtype=torch.int64 if hdt == np.int64 else torch.int32, device="cuda")
    ok = tbe.pruned_hashmap_insert(dev(indices), dev(indices.copy()), dev(np.array([0, 6], dtype=idt)), small,
                                   dev(np.array([0, 4], dtype=np.int64)), slot=5)
    assert not ok and int((small[:, 0] != -1).sum()) == 4


def test_lookups_match_the_reference_fixtures(gpu_ctx):
    """The kernels against tables built, and answers given, by the reference's
    own pruned_hashmap_insert/lookup_unweighted_cpu and pruned_array_lookup_cpu
    (tests/golden/make_golden_tbe.py); the host-side insert the library ships
    against the reference's table, slot for slot."""
    from helpers import load_golden

    g = load_golden("tbe_golden.npz")
    for i in range(int(g["n_hash"])):
        k = f"hash{i}_"
        T, B = (int(x) for x in g[k + "meta"])
        table, hto, offsets = g[k + "table"], g[k + "hto"], g[k + "offsets"]
        for probe, want in ((g[k + "indices"], g[k + "lookup"]), (g[k + "probe"], g[k + "probe_lookup"])):
            got = tbe.pruned_hashmap_lookup(dev(probe), dev(offsets), dev(table), dev(hto), slot=7)
            np.testing.assert_array_equal(got.cpu().numpy(), want, err_msg=k)
        built = torch.full(table.shape, -1, dtype=torch.from_numpy(table).dtype)
        assert tbe.pruned_hashmap_insert(torch.from_numpy(g[k + "indices"]), torch.from_numpy(g[k + "dense"]),
                                         torch.from_numpy(offsets), built, torch.from_numpy(hto))
        np.testing.assert_array_equal(built.numpy(), table, err_msg=k)
        # the device-built table gives the reference's answers too
        d_built = torch.full(table.shape, -1, dtype=built.dtype, device="cuda")
        assert tbe.pruned_hashmap_insert(dev(g[k + "indices"]), dev(g[k + "dense"]), dev(offsets), d_built, dev(hto), slot=7)
        got = tbe.pruned_hashmap_lookup(dev(g[k + "probe"]), dev(offsets), d_built, dev(hto), slot=7)
        np.testing.assert_array_equal(got.cpu().numpy(), g[k + "probe_lookup"], err_msg=k)
    for i in range(int(g["n_arr"])):
        k = f"arr{i}_"
        got = tbe.pruned_array_lookup(dev(g[k + "indices"]), dev(g[k + "offsets"]), dev(g[k + "remap"]), dev(g[k + "ro"]),
                                      slot=7)
        np.testing.assert_array_equal(got.cpu().numpy(), g[k + "lookup"], err_msg=k)
    assert F.status_read(7)[0]

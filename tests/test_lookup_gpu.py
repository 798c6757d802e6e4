"""Parity of the CUDA lookups with the CPU oracle, through the C ABI.

Modelled on the reference's own differential tests
(test/EmbeddingSpMDM8BitTest.cc, test/EmbeddingSpMDMNBitTest.cc of FBGEMM): the
same shapes, weighting modes, corner cases and overrun sentries, with the
coin-flipped options (index/offset width, normalize, offsets-vs-lengths)
enumerated from a seed instead.  The bar is the reference's: EXPECT_EQ on every
element, i.e. bit-exact fp32 and fp16.
"""
import ctypes as C
import itertools
import os

import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from fbgemm_b200 import _capi
from helpers import REFERENCE_SHAPES, lengths_indices_weights, mapping_table, random_fused_table, row_bytes
from conftest import bits

pytestmark = pytest.mark.gpu

SENTRIES = 10


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_kernel(bit_rate, dim, has_weight, normalize, positional, use_offsets, idt, odt, out_dt, **strides):
    if bit_rate == 8:
        return F.GenerateEmbeddingSpMDMWithStrides(
            dim, has_weight, normalize, 16, positional, use_offsets, index_dtype=idt, offset_dtype=odt,
            out_dtype=out_dt, **strides)
    return F.GenerateEmbeddingSpMDMNBitWithStrides(
        bit_rate, dim, has_weight, normalize, 16, positional, use_offsets, index_dtype=idt, offset_dtype=odt,
        out_dtype=out_dt, **strides)


def run_case(oracle, rng, bit_rate, shape, weighting, corner, out_dt, idt, odt, normalize, use_offsets):
    batch, rows, dim, avg_len = shape
    table = random_fused_table(rng, rows, dim, bit_rate)
    lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, odt, corner)
    has_weight = weighting != "unweighted"
    positional = weighting == "positional"
    if positional:
        weights = rng.standard_normal(max(int(lengths.max()), 1) + 1).astype(np.float32)
    ol = offsets if use_offsets else lengths
    ok_ref, out_ref = oracle.spmdm(bit_rate, dim, rows, table, indices, ol, weights if has_weight else None,
                                   normalize, out_dt, positional, use_offsets, output_size=batch, index_size=n)
    kern = make_kernel(bit_rate, dim, has_weight, normalize, positional, use_offsets, idt, odt, out_dt)
    tdt = torch.float16 if out_dt == np.float16 else torch.float32
    out = torch.ones(batch * dim + SENTRIES, dtype=tdt, device="cuda")
    d_idx = dev(indices) if n else None  # the reference passes nullptr for empty indices
    ok = kern(batch, n, rows, dev(table), d_idx, dev(ol), dev(weights) if has_weight else None, out)
    assert ok == ok_ref
    expected_false = corner in ("oob", "unmatched+", "unmatched-")
    assert ok == (not expected_false)
    got = out.cpu().numpy()
    assert (got[batch * dim:] == 1).all(), "wrote past the output"
    if ok:
        np.testing.assert_array_equal(bits(got[:batch * dim]), bits(out_ref[:batch * dim]))


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
@pytest.mark.parametrize("weighting", ["unweighted", "weighted", "positional"])
@pytest.mark.parametrize("out_dt", [np.float32, np.float16])
def test_reference_shapes(gpu_ctx, oracle, bit_rate, weighting, out_dt):
    rng = np.random.default_rng(1000 + bit_rate)
    flips = itertools.cycle(itertools.product([np.int32, np.int64], [np.int32, np.int64], [False, True], [True, False]))
    for shape in REFERENCE_SHAPES:
        idt, odt, normalize, use_offsets = next(flips)
        run_case(oracle, rng, bit_rate, shape, weighting, None, out_dt, idt, odt, normalize, use_offsets)


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
@pytest.mark.parametrize("corner", ["empty", "oob", "unmatched+", "unmatched-"])
def test_corner_cases(gpu_ctx, oracle, bit_rate, corner):
    rng = np.random.default_rng(2000 + bit_rate)
    flips = itertools.cycle(itertools.product([np.int64, np.int32], [np.int64, np.int32], [True, False], [True, False]))
    for shape in REFERENCE_SHAPES[::3]:
        idt, odt, normalize, use_offsets = next(flips)
        for weighting in ("unweighted", "weighted"):
            run_case(oracle, rng, bit_rate, shape, weighting, corner, np.float32, idt, odt, normalize, use_offsets)


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
def test_all_option_combinations_small(gpu_ctx, oracle, bit_rate):
    """Every index/offset width x normalize x offsets-vs-lengths x output type
    on one ragged shape with empty bags in the middle."""
    rng = np.random.default_rng(3000 + bit_rate)
    rows, dim, batch = 300, 72, 33
    table = random_fused_table(rng, rows, dim, bit_rate)
    lengths = rng.integers(0, 50, batch)
    lengths[[3, 4, 17]] = 0
    n = int(lengths.sum())
    w = rng.standard_normal(n).astype(np.float32)
    d_table, d_w = dev(table), dev(w)
    for idt, odt, normalize, use_offsets, out_dt, has_weight in itertools.product(
            [np.int32, np.int64], [np.int32, np.int64], [False, True], [True, False], [np.float32, np.float16],
            [False, True]):
        indices = rng.integers(0, rows, n).astype(idt)
        ol = (np.concatenate([[0], np.cumsum(lengths)]) if use_offsets else lengths).astype(odt)
        ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, ol, w if has_weight else None, normalize,
                                   out_dt, False, use_offsets, output_size=batch, index_size=n)
        kern = make_kernel(bit_rate, dim, has_weight, normalize, False, use_offsets, idt, odt, out_dt)
        out = torch.zeros(batch * dim, dtype=torch.float16 if out_dt == np.float16 else torch.float32, device="cuda")
        ok = kern(batch, n, rows, d_table, dev(indices), dev(ol), d_w if has_weight else None, out)
        assert ok and ok_ref
        np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(ref))


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
def test_offsets_not_zero_based(gpu_ctx, oracle, bit_rate):
    """A multi-table caller passes a slice of a global offsets array together
    with pre-advanced indices/weights: only differences of offsets matter."""
    rng = np.random.default_rng(4000 + bit_rate)
    rows, dim, batch = 500, 64, 20
    table = random_fused_table(rng, rows, dim, bit_rate)
    lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 12, np.int32, np.int64)
    shifted = offsets + 123457
    ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, weights, False, np.float32)
    kern = make_kernel(bit_rate, dim, True, False, False, True, np.int32, np.int64, np.float32)
    out = torch.zeros(batch * dim, device="cuda")
    assert kern(batch, n, rows, dev(table), dev(indices), dev(shifted), dev(weights), out) and ok_ref
    np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(ref))


@pytest.mark.parametrize("bit_rate", [8, 4])
def test_offsets_stepping_backwards_return_false(gpu_ctx, oracle, bit_rate):
    """offsets = [0, 5, 3, 8] with 8 indices: the last offset matches, every
    bag stays inside the index array, yet the reference (which walks the array
    with a running position) runs past the end and returns false."""
    rng = np.random.default_rng(4100 + bit_rate)
    rows, dim = 300, 32
    table = random_fused_table(rng, rows, dim, bit_rate)
    indices = rng.integers(0, rows, 8).astype(np.int64)
    for odt in (np.int32, np.int64):
        offsets = np.array([0, 5, 3, 8], dtype=odt)
        ok_ref, _ = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, None, False, np.float32)
        assert not ok_ref
        kern = make_kernel(bit_rate, dim, False, False, False, True, np.int64, odt, np.float32)
        out = torch.zeros(3 * dim, device="cuda")
        assert not kern(3, 8, rows, dev(table), dev(indices), dev(offsets), None, out)
        _capi.lib().fbgemm_b200_set_kernel_choice(1)   # the generic kernel
        try:
            assert not kern(3, 8, rows, dev(table), dev(indices), dev(offsets), None, out)
        finally:
            _capi.lib().fbgemm_b200_set_kernel_choice(0)


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
def test_strides(gpu_ctx, oracle, bit_rate):
    """output_stride > block_size (a column slice of a wider output) and
    input_stride > fused row size (padded rows); columns outside the slice
    must stay untouched."""
    rng = np.random.default_rng(5000 + bit_rate)
    rows, dim, batch = 400, 96, 17
    for in_pad, out_stride, out_dt in ((0, 200, np.float32), (12, 96, np.float16), (28, 131, np.float32)):
        in_stride = row_bytes(bit_rate, dim) + in_pad
        table = random_fused_table(rng, rows, dim, bit_rate, stride=in_stride)
        lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 9, np.int64, np.int32)
        ref_buf = np.full(batch * out_stride, 7, dtype=out_dt)
        ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, weights, True, out_dt, False, True,
                                   out_stride, in_stride, out=ref_buf)
        kern = make_kernel(bit_rate, dim, True, True, False, True, np.int64, np.int32, out_dt,
                           output_stride=out_stride, input_stride=in_stride)
        out = torch.full((batch * out_stride,), 7, dtype=torch.float16 if out_dt == np.float16 else torch.float32,
                         device="cuda")
        assert kern(batch, n, rows, dev(table), dev(indices), dev(offsets), dev(weights), out) and ok_ref
        np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(ref))


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
def test_misaligned_table_pointer(gpu_ctx, oracle, bit_rate):
    """A table that starts at an odd address takes the byte-wise staging path."""
    rng = np.random.default_rng(6000 + bit_rate)
    rows, dim, batch = 200, 64, 9
    table = random_fused_table(rng, rows, dim, bit_rate)
    lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 7, np.int64, np.int64)
    ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, None, False, np.float32)
    for shift in (1, 2, 4, 8):
        buf = torch.zeros(table.size + 64, dtype=torch.uint8, device="cuda")
        buf[shift:shift + table.size] = torch.from_numpy(table.reshape(-1)).cuda()
        view = buf[shift:shift + table.size]
        kern = make_kernel(bit_rate, dim, False, False, False, True, np.int64, np.int64, np.float32)
        out = torch.zeros(batch * dim, device="cuda")
        assert kern(batch, n, rows, view, dev(indices), dev(offsets), None, out) and ok_ref
        np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(ref))


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
@pytest.mark.parametrize("weighting", ["unweighted", "weighted", "positional"])
def test_rowwise_sparse(gpu_ctx, oracle, bit_rate, weighting):
    """Pruned tables (test/EmbeddingSpMDMNBitTest.cc rowwiseSparseTest): a -1 in
    the mapping skips the row but keeps its weight slot and its place in the
    bag length."""
    rng = np.random.default_rng(7000 + bit_rate)
    flips = itertools.cycle(itertools.product([np.int32, np.int64], [np.int64, np.int32], [True, False], [True, False]))
    for shape in REFERENCE_SHAPES:
        batch, rows, dim, avg_len = shape
        idt, odt, normalize, use_offsets = next(flips)
        mapping, n_dense = mapping_table(rng, rows, 0.7)
        table = random_fused_table(rng, max(n_dense, 1), dim, bit_rate)
        for corner in (None, "oob", "unmatched-"):
            lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, odt, corner)
            has_weight = weighting != "unweighted"
            positional = weighting == "positional"
            if positional:
                weights = rng.standard_normal(int(lengths.max()) + 1).astype(np.float32)
            ol = offsets if use_offsets else lengths
            ok_ref, ref = oracle.spmdm_rowwise_sparse(
                bit_rate, dim, rows, table, indices, mapping, ol, weights if has_weight else None, normalize,
                positional, use_offsets, output_size=batch, index_size=n)
            if bit_rate == 8:
                kern = F.GenerateEmbeddingSpMDMRowWiseSparse(dim, has_weight, normalize, 16, positional, use_offsets,
                                                             index_dtype=idt, offset_dtype=odt)
            else:
                kern = F.GenerateEmbeddingSpMDMNBitRowWiseSparse(bit_rate, dim, has_weight, normalize, 16, positional,
                                                                 use_offsets, index_dtype=idt, offset_dtype=odt)
            out = torch.ones(batch * dim + SENTRIES, device="cuda")
            ok = kern(batch, n, rows, dev(table), dev(indices), dev(ol), dev(weights) if has_weight else None, out,
                      dev(mapping))
            assert ok == ok_ref == (corner is None)
            got = out.cpu().numpy()
            assert (got[batch * dim:] == 1).all()
            if ok:
                np.testing.assert_array_equal(bits(got[:batch * dim]), bits(ref[:batch * dim]))


def test_long_bags_and_wide_rows(gpu_ctx, oracle):
    """Bags longer than one staging wave and the widest supported rows."""
    rng = np.random.default_rng(8000)
    for bit_rate, dim in ((8, 1024), (4, 1024), (2, 1024), (8, 640), (4, 520), (2, 36)):
        rows, batch = 300, 6
        table = random_fused_table(rng, rows, dim, bit_rate)
        lengths = np.array([0, 1, 700, 64, 65, 129])
        offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
        n = int(offsets[-1])
        indices = rng.integers(0, rows, n).astype(np.int64)
        weights = rng.standard_normal(n).astype(np.float32)
        ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, weights, True, np.float32)
        kern = make_kernel(bit_rate, dim, True, True, False, True, np.int64, np.int64, np.float32)
        out = torch.zeros(batch * dim, device="cuda")
        assert kern(batch, n, rows, dev(table), dev(indices), dev(offsets), dev(weights), out) and ok_ref
        np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(ref))


def test_unsupported_block_size_is_rejected_at_generation():
    with pytest.raises(Exception):
        F.GenerateEmbeddingSpMDM(2048, False, False)


def test_host_pointer_path(gpu_ctx, oracle):
    """The functor called with host (numpy) buffers: table made resident on
    first use, per-call arrays staged, result written to the host buffer."""
    rng = np.random.default_rng(9000)
    for bit_rate, out_dt, out_stride in ((8, np.float32, -1), (4, np.float16, -1), (2, np.float32, 150)):
        rows, dim, batch = 1000, 128, 50
        table = random_fused_table(rng, rows, dim, bit_rate)
        lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 15, np.int64, np.int64)
        ostride = dim if out_stride == -1 else out_stride
        ref_buf = np.full(batch * ostride, 3, dtype=out_dt)
        ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, weights, False, out_dt, False, True,
                                   out_stride, -1, out=ref_buf)
        kern = make_kernel(bit_rate, dim, True, False, False, True, np.int64, np.int64, out_dt,
                           output_stride=out_stride)
        out = np.full(batch * ostride, 3, dtype=out_dt)
        for _ in range(2):  # second call hits the resident table
            assert kern(batch, n, rows, table, indices, offsets, weights, out) and ok_ref
            np.testing.assert_array_equal(bits(out), bits(ref))
        bad = indices.copy()
        bad[5] = rows
        assert kern(batch, n, rows, table, bad, offsets, weights, out) is False
        assert kern(batch, n, rows, table, indices, offsets, weights, out) is True  # status was cleared
        gpu_ctx.unregister_table(table)


def test_host_pipeline_lanes(gpu_ctx, oracle):
    rng = np.random.default_rng(9100)
    rows, dim, batch = 2000, 64, 64
    table = random_fused_table(rng, rows, dim, 4)
    gpu_ctx.register_table(table)
    kern = make_kernel(4, dim, True, False, False, True, np.int32, np.int32, np.float16)
    jobs = []
    for lane in range(4):
        lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 20, np.int32, np.int32)
        out = np.zeros(batch * dim, dtype=np.float16)
        kern.host_submit(lane, batch, n, rows, table, indices, offsets, weights, out)
        jobs.append((lane, offsets, indices, weights, out))
    for lane, offsets, indices, weights, out in jobs:
        assert kern.host_wait(lane)
        _, ref = oracle.spmdm(4, dim, rows, table, indices, offsets, weights, False, np.float16)
        np.testing.assert_array_equal(bits(out), bits(ref))
    gpu_ctx.unregister_table(table)


def test_host_pipeline_with_pinned_upload_dominant_calls(gpu_ctx, oracle):
    """Page-locked caller arrays whose uploads outweigh the rows coming back
    (long bags, narrow rows): the inputs are read in place by the staging
    kernel and the status record is written by a kernel.  Every lane, a bad
    index on one of them, and the lane clean again afterwards."""
    rng = np.random.default_rng(9150)
    rows, dim, batch = 3000, 32, 24
    table = random_fused_table(rng, rows, dim, 4)
    gpu_ctx.register_table(table)
    kern = make_kernel(4, dim, True, False, False, True, np.int64, np.int64, np.float16)
    pin = lambda a: torch.from_numpy(a).pin_memory().numpy()  # noqa: E731
    jobs = []
    for lane in range(_capi.HOST_LANES):
        lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 60, np.int64, np.int64)
        assert indices.nbytes + offsets.nbytes + weights.nbytes > batch * dim * 2   # uploads are the larger transfer
        if lane == 5:
            indices = indices.copy()
            indices[11] = rows + 3
        indices, offsets, weights = pin(indices), pin(offsets), pin(weights)
        out = torch.zeros(batch * dim, dtype=torch.float16).pin_memory().numpy()
        kern.host_submit(lane, batch, n, rows, table, indices, offsets, weights, out)
        jobs.append((lane, offsets, indices, weights, out, n))
    for lane, offsets, indices, weights, out, n in jobs:
        ok = kern.host_wait(lane)
        assert ok == (lane != 5)
        if ok:
            _, ref = oracle.spmdm(4, dim, rows, table, indices, offsets, weights, False, np.float16)
            np.testing.assert_array_equal(bits(out), bits(ref))
    lane, offsets, indices, weights, out, n = jobs[4]
    kern.host_submit(5, batch, n, rows, table, indices, offsets, weights, out)     # lane 5 again, good indices
    assert kern.host_wait(5)
    gpu_ctx.unregister_table(table)


def test_async_launch_and_status_slots(gpu_ctx, oracle):
    rng = np.random.default_rng(9200)
    rows, dim, batch = 500, 32, 40
    table = random_fused_table(rng, rows, dim, 8)
    lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 10, np.int64, np.int64)
    kern = make_kernel(8, dim, False, False, False, True, np.int64, np.int64, np.float32)
    d_table, d_off = dev(table), dev(offsets)
    good, bad = dev(indices), indices.copy()
    bad[7] = -1
    out1 = torch.zeros(batch * dim, device="cuda")
    out2 = torch.zeros(batch * dim, device="cuda")
    kern.launch(batch, n, rows, d_table, good, d_off, None, out1, slot=5)
    kern.launch(batch, n, rows, d_table, dev(bad), d_off, None, out2, slot=6)
    ok5, _ = F.status_read(5)
    ok6, info = F.status_read(6)
    assert ok5 and not ok6
    assert info[0] == 1 and info[2] == 7 and info[3] == -1  # BAD_INDEX at position 7, value -1
    ok6_again, _ = F.status_read(6)
    assert ok6_again  # reading clears the slot
    _, ref = oracle.spmdm(8, dim, rows, table, indices, offsets, None, False, np.float32)
    np.testing.assert_array_equal(bits(out1.cpu().numpy()), bits(ref))


def test_resident_copy_is_checked_against_the_callers_table(gpu_ctx, oracle):
    """A resident copy is keyed by the host address alone, and an address can
    come back with another table behind it.  A call that needs more bytes than
    the registered copy holds, or whose host table no longer has the registered
    contents, is refused before any kernel runs (explicit registration) or gets
    a fresh copy (a copy the library made on its own)."""
    rng = np.random.default_rng(9300)
    rows, dim, batch = 400, 64, 20
    big = random_fused_table(rng, 2 * rows, dim, 4)
    lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 8, np.int32, np.int32)
    kern = make_kernel(4, dim, False, False, False, True, np.int32, np.int32, np.float32)
    out = np.zeros(batch * dim, dtype=np.float32)
    # explicit registration of the first half only, then a call that addresses the whole array
    gpu_ctx.register_table(big[:rows])
    assert kern(batch, n, rows, big, indices, offsets, None, out)
    before = F.launch_count()
    with pytest.raises(_capi.Fbgemmb200Error, match="register it again"):
        kern(batch, n, 2 * rows, big, indices, offsets, None, out)
    # same size, other contents behind the same address: refused as well
    big[:rows] = random_fused_table(rng, rows, dim, 4)
    with pytest.raises(_capi.Fbgemmb200Error, match="register it again"):
        kern(batch, n, rows, big, indices, offsets, None, out)
    assert F.launch_count() == before          # nothing ran
    gpu_ctx.register_table(big[:rows])         # registering again is the cure
    assert kern(batch, n, rows, big, indices, offsets, None, out)
    _, ref = oracle.spmdm(4, dim, rows, big, indices, offsets, None, False, np.float32)
    np.testing.assert_array_equal(bits(out), bits(ref))
    gpu_ctx.unregister_table(big)
    # a copy made by the call itself follows the caller's memory
    table = random_fused_table(rng, rows, dim, 4)
    assert kern(batch, n, rows, table, indices, offsets, None, out)
    table[:] = random_fused_table(rng, rows, dim, 4)
    assert kern(batch, n, rows, table, indices, offsets, None, out)
    _, ref = oracle.spmdm(4, dim, rows, table, indices, offsets, None, False, np.float32)
    np.testing.assert_array_equal(bits(out), bits(ref))
    gpu_ctx.unregister_table(table)


def test_lengths_mode_on_two_streams_does_not_share_scratch(gpu_ctx, oracle):
    """Lengths-mode launches on different streams overlap: each stream has its
    own scanned offsets."""
    rng = np.random.default_rng(9400)
    rows, dim = 3000, 64
    table = random_fused_table(rng, rows, dim, 4)
    d_table = dev(table)
    kern = make_kernel(4, dim, False, False, False, False, np.int32, np.int32, np.float32)
    streams = [torch.cuda.Stream() for _ in range(3)]
    jobs = []
    for rep in range(4):
        for i, s in enumerate(streams):
            batch = 2000 + 700 * i
            lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 6 + 3 * i, np.int32, np.int32)
            d_len, d_idx = dev(lengths), dev(indices)
            out = torch.zeros(batch * dim, device="cuda")
            torch.cuda.synchronize()
            jobs.append((lengths, indices, n, batch, d_len, d_idx, out, 70 + i, s))
    for lengths, indices, n, batch, d_len, d_idx, out, slot, s in jobs:
        kern.launch(batch, n, rows, d_table, d_idx, d_len, None, out, slot=slot, stream=s.cuda_stream)
    torch.cuda.synchronize()
    for i in range(3):
        assert F.status_read(70 + i)[0]
    for lengths, indices, n, batch, d_len, d_idx, out, slot, s in jobs:
        _, ref = oracle.spmdm(4, dim, rows, table, indices, lengths, None, False, np.float32, False, False)
        np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(ref))


def test_null_pointers_and_reserved_slots_are_refused_on_the_host(gpu_ctx):
    lib = _capi.lib()
    kern = make_kernel(4, 64, False, False, False, True, np.int32, np.int32, np.float32)
    t = torch.zeros(64 * 36, dtype=torch.uint8, device="cuda")
    idx = torch.zeros(8, dtype=torch.int32, device="cuda")
    off = torch.arange(0, 9, dtype=torch.int32, device="cuda")
    out = torch.zeros(8 * 64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    args = lambda **kw: [gpu_ctx.handle, C.byref(kern.cfg), 8, 8, 64, kw.get("t", t.data_ptr()), kw.get("i", idx.data_ptr()),  # noqa: E731
                         kw.get("o", off.data_ptr()), None, kw.get("out", out.data_ptr()), None, kw.get("slot", 3), st]
    before = F.launch_count()
    for bad in (dict(t=None), dict(i=None), dict(o=None), dict(out=None), dict(slot=_capi.USER_SLOTS),
                dict(slot=_capi.STATUS_SLOTS - 1)):
        assert lib.fbgemm_b200_spmdm_launch(*args(**bad)) == _capi.EINVAL, bad
    assert F.launch_count() == before
    assert lib.fbgemm_b200_spmdm_launch(*args()) == 0 and F.status_read(3)[0]

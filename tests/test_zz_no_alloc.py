"""The lookup entry point for callers that must not allocate device memory
(servers whose own allocator owns the whole GPU, request loops that forbid
cudaMalloc after start-up).  It keeps its scratch - the scanned offsets of the
lengths flavour and the status record - in a fixed device array of the library
instead of a cudaMalloc'ed buffer.

Checked here, through the C ABI: two calls in a row (the second with fewer and
different bags, so anything left in the shared array by the first call would
show) give exactly the rows of the regular entry point ``fbgemm_b200_spmdm``;
an input error is reported and then cleared; a call beyond the stated maximum
is refused.  The file name sorts last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from fbgemm_b200 import _capi
from helpers import random_fused_table
from conftest import bits

pytestmark = pytest.mark.gpu


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _call_pair(ctx, cfg, batch, n, rows, table, indices, lengths, weights, dim, out_dtype, cit=None):
    """Run the regular and the no-allocation entry point on the same device
    buffers; return (ok_regular, rows_regular, ok_noalloc, rows_noalloc)."""
    lib = _capi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    d = [dev(table), dev(indices), dev(lengths), dev(weights), dev(cit)]
    ptr = [None if t is None else t.data_ptr() for t in d]
    want = torch.full((batch * dim,), 5, dtype=out_dtype, device="cuda")
    got = torch.full((batch * dim,), 9, dtype=out_dtype, device="cuda")
    ok_regular = lib.fbgemm_b200_spmdm(ctx.handle, C.byref(cfg), batch, n, rows, ptr[0], ptr[1], ptr[2], ptr[3],
                                       want.data_ptr(), ptr[4], stream)
    ok_noalloc = lib.fbgemm_b200_spmdm_lengths_noalloc(C.byref(cfg), batch, n, rows, ptr[0], ptr[1], ptr[2], ptr[3],
                                                       got.data_ptr(), ptr[4], stream)
    assert ok_regular >= 0 and ok_noalloc >= 0, _capi.last_error()
    return ok_regular, want.cpu().numpy(), ok_noalloc, got.cpu().numpy()


@pytest.mark.parametrize("bit_rate,out_dtype", [(8, torch.float32), (4, torch.float16), (2, torch.float32)])
def test_no_alloc_entry_matches_regular_entry_twice(gpu_ctx, oracle, bit_rate, out_dtype):
    rng = np.random.default_rng(100 + bit_rate)
    rows, dim = 3000, 64
    table = random_fused_table(rng, rows, dim, bit_rate)
    cfg = _capi.SpmdmConfig(bit_rate=bit_rate, index_bytes=8, offset_bytes=4,
                            out_dtype=_capi.OUT_F16 if out_dtype == torch.float16 else _capi.OUT_F32,
                            block_size=dim, output_stride=-1, input_stride=-1, has_weight=1,
                            normalize_by_lengths=1, is_weight_positional=0, use_offsets=0)
    # first call: many bags (several scan tiles); second call: fewer, other bags
    for batch in (9000, 700):
        lengths = rng.integers(0, 12, batch).astype(np.int32)
        n = int(lengths.sum())
        indices = rng.integers(0, rows, n).astype(np.int64)
        weights = rng.standard_normal(n).astype(np.float32)
        ok_r, want, ok_n, got = _call_pair(gpu_ctx, cfg, batch, n, rows, table, indices, lengths, weights, dim,
                                           out_dtype)
        assert ok_r == 1 and ok_n == 1
        np.testing.assert_array_equal(bits(got), bits(want))
        # and directly against the CPU oracle's lengths flavour
        ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, lengths, weights, True,
                                   np.float16 if out_dtype == torch.float16 else np.float32, False, False)
        assert ok_ref
        np.testing.assert_array_equal(bits(got), bits(ref))


def test_no_alloc_entry_reports_and_clears_errors(gpu_ctx):
    rng = np.random.default_rng(7)
    rows, dim, batch = 500, 32, 300
    table = random_fused_table(rng, rows, dim, 8)
    cfg = _capi.SpmdmConfig(bit_rate=8, index_bytes=4, offset_bytes=8, out_dtype=_capi.OUT_F32, block_size=dim,
                            output_stride=-1, input_stride=-1, has_weight=0, normalize_by_lengths=0,
                            is_weight_positional=0, use_offsets=0)
    lengths = rng.integers(1, 9, batch).astype(np.int64)
    n = int(lengths.sum())
    good = rng.integers(0, rows, n).astype(np.int32)
    bad = good.copy()
    bad[n // 2] = rows  # one index out of range
    ok_r, _, ok_n, _ = _call_pair(gpu_ctx, cfg, batch, n, rows, table, bad, lengths, None, dim, torch.float32)
    assert ok_r == 0 and ok_n == 0
    # the error record lives in the shared array: the next call must start clean
    ok_r, want, ok_n, got = _call_pair(gpu_ctx, cfg, batch, n, rows, table, good, lengths, None, dim, torch.float32)
    assert ok_r == 1 and ok_n == 1
    np.testing.assert_array_equal(bits(got), bits(want))
    # lengths that do not add up to index_size
    ok_r, _, ok_n, _ = _call_pair(gpu_ctx, cfg, batch, n - 1, rows, table, good, lengths, None, dim, torch.float32)
    assert ok_r == 0 and ok_n == 0


def test_no_alloc_entry_refuses_sizes_beyond_its_maximum(gpu_ctx):
    cfg = _capi.SpmdmConfig(bit_rate=8, index_bytes=8, offset_bytes=8, out_dtype=_capi.OUT_F32, block_size=16,
                            output_stride=-1, input_stride=-1, has_weight=0, normalize_by_lengths=0,
                            is_weight_positional=0, use_offsets=0)
    lib = _capi.lib()
    t = torch.zeros(64, dtype=torch.uint8, device="cuda")
    rc = lib.fbgemm_b200_spmdm_lengths_noalloc(C.byref(cfg), _capi.NOALLOC_MAX_BAGS + 1, 0, 1, t.data_ptr(),
                                               t.data_ptr(), t.data_ptr(), None, t.data_ptr(), None, None)
    assert rc == _capi.EINVAL
    assert "FBGEMM_B200_NOALLOC_MAX_BAGS" in _capi.last_error()
    cfg.use_offsets = 1  # the entry point is the lengths flavour only
    rc = lib.fbgemm_b200_spmdm_lengths_noalloc(C.byref(cfg), 4, 0, 1, t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                               None, t.data_ptr(), None, None)
    assert rc == _capi.EINVAL
    # configurations without lengths, and null pointers, are refused before any kernel is enqueued
    before = F.launch_count()
    cfg.use_offsets = 0
    cfg.no_bag = 1
    rc = lib.fbgemm_b200_spmdm_lengths_noalloc(C.byref(cfg), 4, 4, 1, t.data_ptr(), t.data_ptr(), None, None,
                                               t.data_ptr(), None, None)
    assert rc == _capi.EINVAL
    cfg.no_bag = 0
    for args in ((t.data_ptr(), t.data_ptr(), None, t.data_ptr()), (None, t.data_ptr(), t.data_ptr(), t.data_ptr()),
                 (t.data_ptr(), None, t.data_ptr(), t.data_ptr()), (t.data_ptr(), t.data_ptr(), t.data_ptr(), None)):
        rc = lib.fbgemm_b200_spmdm_lengths_noalloc(C.byref(cfg), 4, 4, 1, args[0], args[1], args[2], None, args[3],
                                                   None, None)
        assert rc == _capi.EINVAL, args
    cfg.offset_bytes = 3
    rc = lib.fbgemm_b200_spmdm_lengths_noalloc(C.byref(cfg), 4, 4, 1, t.data_ptr(), t.data_ptr(), t.data_ptr(), None,
                                               t.data_ptr(), None, None)
    assert rc == _capi.EINVAL
    assert F.launch_count() == before

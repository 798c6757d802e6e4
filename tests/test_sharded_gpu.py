"""Table-wise sharding on GPUs: the peer-routing of the sharded launch on one
GPU (two "peers" that are both local buffers), and the real thing on two GPUs
when the box has them (p2p stores over NVLink and the NCCL baseline, both
against the oracle)."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from fbgemm_b200 import _capi
from conftest import bits
from helpers import lengths_indices_weights, random_fused_table

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("bit_rate,out_dt", [(8, np.float32), (4, np.float16), (2, np.float16)])
def test_sharded_launch_routes_bags_to_peers(gpu_ctx, oracle, bit_rate, out_dt):
    """Bags [0, 40) go to 'peer' 0, [40, 80) to peer 1, [80, 100) to peer 2, each
    at its own column offset of a wider row, as the batch-wise layout wants."""
    rng = np.random.default_rng(bit_rate)
    rows, dim, batch, per_peer, total_dim, col = 700, 64, 100, 40, 200, 72
    table = random_fused_table(rng, rows, dim, bit_rate)
    lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 12, np.int32, np.int32)
    ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, weights, False, out_dt)
    ref = ref.reshape(batch, dim)
    tdt = torch.float16 if out_dt == np.float16 else torch.float32
    bufs = [torch.full((per_peer, total_dim), 7, dtype=tdt, device="cuda") for _ in range(3)]
    esize = 2 if out_dt == np.float16 else 4
    ptrs = (C.c_void_p * 3)(*[b.data_ptr() + col * esize for b in bufs])
    kw = dict(index_dtype=np.int32, offset_dtype=np.int32, out_dtype=out_dt, output_stride=total_dim)
    kern = (F.GenerateEmbeddingSpMDMWithStrides(dim, True, False, **kw) if bit_rate == 8 else
            F.GenerateEmbeddingSpMDMNBitWithStrides(bit_rate, dim, True, False, **kw))
    d = [torch.from_numpy(a).cuda() for a in (table, indices, offsets, weights)]
    rc = _capi.lib().fbgemm_b200_spmdm_launch_sharded(
        gpu_ctx.handle, C.byref(kern.cfg), batch, n, rows, d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(),
        d[3].data_ptr(), ptrs, 3, per_peer, 9, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _capi.last_error()
    ok, _ = F.status_read(9)
    assert ok and ok_ref
    for peer, buf in enumerate(bufs):
        got = buf.cpu().numpy()
        lo, hi = peer * per_peer, min(batch, (peer + 1) * per_peer)
        np.testing.assert_array_equal(bits(got[:hi - lo, col:col + dim]), bits(ref[lo:hi]))
        assert (got[:, :col] == 7).all() and (got[:, col + dim:] == 7).all()   # other columns untouched
        assert (got[hi - lo:] == 7).all()                                        # rows past the batch untouched


def test_two_gpu_sharded_lookup_matches_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.join(ROOT, "tests", "sharded_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "SHARDED_OK" in res.stdout


def test_peer_counters_signal_wait_and_time_out(gpu_ctx):
    """A wait whose counters were published passes; a wait on a counter that
    nobody writes gives up after its time limit with a status record naming
    the laggard - no hang, no trap - and the context keeps working."""
    import time

    lib = _capi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    flags = torch.zeros(4, dtype=torch.int64, device="cuda")
    arr = (C.c_void_p * 3)(*[flags.data_ptr() + 8 * i for i in range(3)])
    assert lib.fbgemm_b200_peer_signal(gpu_ctx.handle, arr, 3, 5, stream) == 0
    assert lib.fbgemm_b200_peer_wait(gpu_ctx.handle, flags.data_ptr(), 3, 5, 1000, 40, stream) == 0
    ok, info = F.status_read(40)
    assert ok and flags.cpu().tolist() == [5, 5, 5, 0]
    # word 3 stays at 0: the wait for 1 runs out (50 ms limit)
    t0 = time.perf_counter()
    assert lib.fbgemm_b200_peer_wait(gpu_ctx.handle, flags.data_ptr(), 4, 1, 50_000, 40, stream) == 0
    ok, info = F.status_read(40)
    dt = time.perf_counter() - t0
    assert not ok and info == [_capi.STATUS_PEER_TIMEOUT, 3, 0, 1]
    assert 0.04 < dt < 5.0
    # the slot was cleared by the read and the context is usable
    assert lib.fbgemm_b200_peer_wait(gpu_ctx.handle, flags.data_ptr(), 3, 5, 1000, 40, stream) == 0
    assert F.status_read(40)[0]
    # argument checks happen on the host
    assert lib.fbgemm_b200_peer_wait(gpu_ctx.handle, flags.data_ptr(), 3, 5, 0, 40, stream) < 0
    assert lib.fbgemm_b200_peer_wait(gpu_ctx.handle, flags.data_ptr() + 4, 3, 5, 10, 40, stream) < 0
    assert lib.fbgemm_b200_peer_signal(gpu_ctx.handle, arr, 9, 5, stream) < 0


def _specs_and_batches(B, seed=0, tables=5):
    from fbgemm_b200.workloads import TableSpec

    specs = [TableSpec(900 + 150 * t, (64, 128, 32)[t % 3], (8, 4, 2)[t % 3], 300 + t) for t in range(tables)]
    rng = np.random.default_rng(seed)
    host = {}
    for t, s in enumerate(specs):
        lengths = rng.integers(0, 15, B)
        off = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
        host[t] = (rng.integers(0, s.rows, int(off[-1])).astype(np.int32), off)
    return specs, host


def _oracle_rows(oracle, specs, plan, tables, host, rows_lo, rows_hi):
    want = np.zeros((rows_hi - rows_lo, plan.total_dim), dtype=np.float16)
    for t, s in enumerate(specs):
        idx, off = host[t]
        ok, ref = oracle.spmdm(s.bit_rate, s.dim, s.rows, tables[t], idx[off[rows_lo]:off[rows_hi]],
                               off[rows_lo:rows_hi + 1], None, False, np.float16)
        assert ok
        c0 = plan.column_start(t)
        want[:, c0:c0 + s.dim] = ref.reshape(rows_hi - rows_lo, s.dim)
    return want


def test_ordered_steps_and_host_call_on_one_gpu(gpu_ctx, oracle):
    """World size 1: the device-ordered step (ack wait, lookups, ready signal,
    ready wait, release) over two buffers, and the host-pointer multi-table
    call with its counters, both against the oracle."""
    from fbgemm_b200.sharding import ShardedLookup, TableWisePlan
    from fbgemm_b200.workloads import Batch

    B, dev = 64, torch.device("cuda", 0)
    specs, _ = _specs_and_batches(B)
    plan = TableWisePlan([0] * len(specs), [s.dim for s in specs], 1)
    sl = ShardedLookup(specs, plan, 0, B, dev, torch.float16, mode="p2p", num_buffers=2)
    tables = {t: sl.tables[t].cpu().numpy() for t in sl.local}
    streams = [torch.cuda.Stream() for _ in range(2)]
    for step in range(5):
        _, host = _specs_and_batches(B, seed=10 + step)
        batches = {t: Batch(torch.from_numpy(host[t][0]).cuda(), torch.from_numpy(host[t][1]).cuda(), None, B,
                            len(host[t][0]), len(host[t][0])) for t in sl.local}
        buf = step % 2
        n = sl.step(batches, buffer=buf, slot_base=50, streams=streams)
        got = sl.out[buf].cpu().numpy()      # the copy is ordered after the ready wait on this stream
        sl.release(buf, n)
        assert n == step // 2 + 1
        for i in range(len(sl.local)):
            ok, info = F.status_read(50 + i)
            assert ok, info
        want = _oracle_rows(oracle, specs, plan, tables, host, 0, B)
        np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))
    # host arrays in, host rows out
    sl2 = ShardedLookup(specs, plan, 0, B, dev, torch.float16, mode="p2p", num_buffers=1, tables=sl.tables)
    call = sl2.make_host_call(0, {t: 2000 for t in sl2.local}, slot=60)
    out_host = torch.zeros((B, plan.total_dim), dtype=torch.float16).pin_memory().numpy()
    with pytest.raises(_capi.Fbgemmb200Error):
        call.last_step_ms()              # nothing has been waited for yet
    for step in range(3):
        _, host = _specs_and_batches(B, seed=20 + step)
        call.submit([host[t][0] for t in sl2.local], [host[t][1] for t in sl2.local], None, out_host)
        ok, info = call.wait()
        assert ok, info
        phases = call.last_step_ms()     # uploads, lookups, download of the step just waited for
        assert len(phases) == 3 and all(0.0 <= ms < 1000.0 for ms in phases) and sum(phases) > 0.0
        want = _oracle_rows(oracle, specs, plan, tables, host, 0, B)
        np.testing.assert_array_equal(out_host.view(np.uint16), want.view(np.uint16))
    # more indices than the handle was built for: refused on the host, nothing enqueued
    big = np.zeros(2001, dtype=np.int32)
    with pytest.raises(_capi.Fbgemmb200Error):
        call.submit([big] * len(sl2.local), [host[t][1] for t in sl2.local], None, out_host)
    # a bad index makes the step false and the next step is clean again
    _, host = _specs_and_batches(B, seed=30)
    host[2][0][5] = specs[2].rows
    call.submit([host[t][0] for t in sl2.local], [host[t][1] for t in sl2.local], None, out_host)
    ok, info = call.wait()
    assert not ok and info[0] == 1 and info[3] == specs[2].rows
    _, host = _specs_and_batches(B, seed=31)
    call.submit([host[t][0] for t in sl2.local], [host[t][1] for t in sl2.local], None, out_host)
    assert call.wait()[0]
    call.close()


@pytest.mark.parametrize("layout", ["one_block", "shared_offsets", "odd_start", "reversed"])
def test_host_call_with_arrays_that_touch_in_host_memory(gpu_ctx, oracle, layout):
    """The host-pointer multi-table call sends arrays that touch or overlap in
    host memory as one copy.  one_block: per-table views of one pinned indices
    and one pinned offsets array; shared_offsets: the reference caller's form,
    ONE offsets array of T*B+1 positions into ONE indices array, table t's
    view starting at element t*B (neighbours share an element); odd_start:
    the block starts 4 bytes past a 16-byte line; reversed: the views of the
    block are handed over last table first (nothing to merge)."""
    from fbgemm_b200.sharding import ShardedLookup, TableWisePlan

    B, dev = 64, torch.device("cuda", 0)
    specs, host = _specs_and_batches(B, seed=40)
    T = len(specs)
    plan = TableWisePlan([0] * T, [s.dim for s in specs], 1)
    sl = ShardedLookup(specs, plan, 0, B, dev, torch.float16, mode="p2p", num_buffers=1)
    tables = {t: sl.tables[t].cpu().numpy() for t in sl.local}
    call = sl.make_host_call(0, {t: 2000 for t in sl.local}, slot=70)
    out_host = torch.zeros((B, plan.total_dim), dtype=torch.float16).pin_memory().numpy()
    pad = 1 if layout == "odd_start" else 0
    n_idx = sum(len(host[t][0]) for t in range(T))
    idx_block = torch.zeros(n_idx + pad, dtype=torch.int32).pin_memory().numpy()[pad:]
    idx_views, at = [], 0
    for t in range(T):
        n = len(host[t][0])
        idx_block[at:at + n] = host[t][0]
        idx_views.append(idx_block[at:at + n])
        at += n
    if layout == "shared_offsets":
        off_block = torch.zeros(T * B + 1, dtype=torch.int32).pin_memory().numpy()
        at = 0
        for t in range(T):
            off_block[t * B:(t + 1) * B + 1] = host[t][1] + at
            at += len(host[t][0])
        off_views = [off_block[t * B:(t + 1) * B + 1] for t in range(T)]
    else:
        off_block = torch.zeros(T * (B + 1) + pad, dtype=torch.int32).pin_memory().numpy()[pad:]
        for t in range(T):
            off_block[t * (B + 1):(t + 1) * (B + 1)] = host[t][1]
        off_views = [off_block[t * (B + 1):(t + 1) * (B + 1)] for t in range(T)]
    order = list(range(T))
    if layout == "reversed":
        # the handle's tables keep their order; what changes is where each table's arrays lie
        idx_block2 = torch.zeros(n_idx, dtype=torch.int32).pin_memory().numpy()
        at = n_idx
        for t in range(T):
            n = len(host[t][0])
            at -= n
            idx_block2[at:at + n] = host[t][0]
            idx_views[t] = idx_block2[at:at + n]
    for _ in range(2):
        out_host[:] = 0
        call.submit([idx_views[t] for t in order], [off_views[t] for t in order], None, out_host)
        ok, info = call.wait()
        assert ok, info
        want = _oracle_rows(oracle, specs, plan, tables, host, 0, B)
        np.testing.assert_array_equal(out_host.view(np.uint16), want.view(np.uint16))
    call.close()


def test_device_array_steps_of_the_multi_table_handle(gpu_ctx, oracle):
    """``fbgemm_b200_multi_host_step_device``: the ordered step on device arrays
    in one call - ack wait, lookups over the handle's streams, ready signal and
    wait - with the release either inside the call or after the consumer."""
    from fbgemm_b200.sharding import ShardedLookup, TableWisePlan

    B, dev = 64, torch.device("cuda", 0)
    specs, _ = _specs_and_batches(B)
    plan = TableWisePlan([0] * len(specs), [s.dim for s in specs], 1)
    sl = ShardedLookup(specs, plan, 0, B, dev, torch.float16, mode="p2p", num_buffers=2)
    tables = {t: sl.tables[t].cpu().numpy() for t in sl.local}
    calls = [sl.make_step_call(b, slot=80 + b) for b in range(2)]
    stream = torch.cuda.Stream()
    for step in range(6):
        _, host = _specs_and_batches(B, seed=50 + step)
        idx = [torch.from_numpy(host[t][0]).cuda() for t in sl.local]
        off = [torch.from_numpy(host[t][1]).cuda() for t in sl.local]
        b = step % 2
        args = calls[b].device_args(idx, off, None)
        stream.wait_stream(torch.cuda.current_stream())
        release_inside = step >= 4
        n = calls[b].step_device(args, release_inside, stream.cuda_stream)
        assert n == step // 2 + 1
        with torch.cuda.stream(stream):
            got = sl.out[b].cpu().numpy()          # ordered after the ready wait
        if not release_inside:
            calls[b].release(n, stream.cuda_stream)
        ok, info = F.status_read(80 + b)
        assert ok, info
        want = _oracle_rows(oracle, specs, plan, tables, host, 0, B)
        np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))
    # a bad index is reported in the handle's slot, and the next step is clean
    _, host = _specs_and_batches(B, seed=60)
    host[1][0][3] = -5
    idx = [torch.from_numpy(host[t][0]).cuda() for t in sl.local]
    off = [torch.from_numpy(host[t][1]).cuda() for t in sl.local]
    calls[0].step_device(calls[0].device_args(idx, off, None), True, stream.cuda_stream)
    stream.synchronize()
    ok, info = F.status_read(80)
    assert not ok and info[0] == 1 and info[3] == -5
    with pytest.raises(_capi.Fbgemmb200Error):
        calls[0].release(99, stream.cuda_stream)      # not a step of this handle
    for c in calls:
        c.close()

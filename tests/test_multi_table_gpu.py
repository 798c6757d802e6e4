"""Several tables pooled by one call (fbgemm_b200_multi_plan_*): every table's
output must equal, bit for bit, what the oracle computes for that table alone -
the reference's multi-table caller is a loop of independent functor calls
(fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:343-473
of FBGEMM), each writing `output + D_start` with output_stride = total_D."""
import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from conftest import bits
from helpers import lengths_indices_weights, mapping_table, random_fused_table
from test_lookup_gpu import dev, make_kernel

pytestmark = pytest.mark.gpu

# (bit_rate, dim, rows, batch, avg_len, weighted, normalize, index dtype, offset dtype)
TABLES = [
    (8, 128, 900, 37, 12, False, False, np.int64, np.int64),
    (4, 64, 700, 50, 20, True, False, np.int32, np.int32),
    (4, 64, 300, 21, 9, True, False, np.int32, np.int32),     # same kernel variant as the one before
    (2, 128, 500, 64, 30, False, True, np.int64, np.int32),
    (8, 40, 200, 10, 6, True, True, np.int32, np.int64),
    (4, 86, 150, 13, 10, False, False, np.int64, np.int64),   # odd payload width: not a direct-kernel shape
    (2, 64, 100, 0, 0, False, False, np.int32, np.int32),     # no bags at all
    (8, 256, 400, 9, 70, False, False, np.int32, np.int32),
]


def build_inputs(seed):
    rng = np.random.default_rng(seed)
    tables = []
    for bit_rate, dim, rows, batch, avg_len, weighted, normalize, idt, odt in TABLES:
        table = random_fused_table(rng, rows, dim, bit_rate)
        if batch:
            _, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, odt)
        else:
            offsets, indices, weights, n = np.zeros(1, dtype=odt), np.zeros(0, dtype=idt), np.zeros(0, np.float32), 0
        tables.append(dict(bit_rate=bit_rate, dim=dim, rows=rows, batch=batch, weighted=weighted, normalize=normalize,
                           idt=idt, odt=odt, table=table, offsets=offsets, indices=indices, weights=weights, n=n))
    return tables


@pytest.mark.parametrize("out_dt", [np.float32, np.float16])
def test_plan_matches_oracle_table_by_table(gpu_ctx, oracle, out_dt):
    tables = build_inputs(7100)
    tdt = torch.float16 if out_dt == np.float16 else torch.float32
    calls, outs, keep = [], [], []
    for t in tables:
        kern = make_kernel(t["bit_rate"], t["dim"], t["weighted"], t["normalize"], False, True, t["idt"], t["odt"], out_dt)
        out = torch.full((max(t["batch"], 1) * t["dim"] + 8,), 7.0, dtype=tdt, device="cuda")
        d = [dev(t["table"]), dev(t["indices"]) if t["n"] else None, dev(t["offsets"]),
             dev(t["weights"]) if t["weighted"] and t["n"] else None]
        keep.append(d)
        calls.append((kern, t["batch"], t["n"], t["rows"], d[0], d[1], d[2], d[3], out, None))
        outs.append(out)
    plan = F.MultiTablePlan(calls, slot=11)
    # 7 tables with bags; the two 4-bit D=64 tables share a launch, the odd one goes alone
    assert 1 <= plan.num_launches < sum(1 for t in tables if t["batch"])
    before = F.launch_count()
    plan.launch()
    plan.launch()  # a plan can be launched again
    ok, info = F.status_read(11)
    assert ok, info
    assert F.launch_count() - before == 2 * plan.num_launches
    for t, out in zip(tables, outs):
        got = out.cpu().numpy()
        assert (got[t["batch"] * t["dim"]:] == 7).all(), "wrote past the output"
        if not t["batch"]:
            continue
        ok_ref, ref = oracle.spmdm(t["bit_rate"], t["dim"], t["rows"], t["table"], t["indices"], t["offsets"],
                                   t["weights"] if t["weighted"] else None, t["normalize"], out_dt)
        assert ok_ref
        np.testing.assert_array_equal(bits(got[:t["batch"] * t["dim"]]), bits(ref[:t["batch"] * t["dim"]]))
    plan.close()


def test_plan_columns_of_one_output_and_pruned_table(gpu_ctx, oracle):
    """Tables writing side by side into one [B, total_D] output
    (output_stride = total_D), plus a row-wise sparse table with its own output."""
    rng = np.random.default_rng(7200)
    batch = 33
    dims = [(8, 64), (4, 128), (2, 64), (4, 128)]
    total = sum(d for _, d in dims)
    out = torch.zeros(batch * total, dtype=torch.float16, device="cuda")
    calls, expect, col, keep = [], [], 0, []
    for bit_rate, dim in dims:
        rows = 600
        table = random_fused_table(rng, rows, dim, bit_rate)
        _, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 15, np.int32, np.int32)
        kern = make_kernel(bit_rate, dim, True, False, False, True, np.int32, np.int32, np.float16, output_stride=total)
        d = (dev(table), dev(indices), dev(offsets), dev(weights))
        keep.append(d)
        calls.append((kern, batch, n, rows, d[0], d[1], d[2], d[3], out.view(-1)[col:], None))
        ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, weights, False, np.float16)
        assert ok_ref
        expect.append((col, dim, ref.reshape(batch, dim)))
        col += dim
    # the pruned table
    prows, pdim = 800, 64
    mapping, dense = mapping_table(rng, prows, 0.6)
    ptable = random_fused_table(rng, max(dense, 1), pdim, 4)
    _, poffsets, pindices, _, pn = lengths_indices_weights(rng, batch, prows, 15, np.int64, np.int64)
    pk = F.GenerateEmbeddingSpMDMNBitRowWiseSparse(4, pdim, False, True, index_dtype=np.int64, offset_dtype=np.int64)
    pout = torch.zeros(batch * pdim, device="cuda")
    d = (dev(ptable), dev(pindices), dev(poffsets), dev(mapping))
    calls.append((pk, batch, pn, prows, d[0], d[1], d[2], None, pout, d[3]))
    plan = F.MultiTablePlan(calls, slot=12)
    plan.launch()
    ok, info = F.status_read(12)
    assert ok, info
    got = out.cpu().numpy().reshape(batch, total)
    for c0, dim, ref in expect:
        np.testing.assert_array_equal(bits(np.ascontiguousarray(got[:, c0:c0 + dim])), bits(ref))
    ok_ref, pref = oracle.spmdm_rowwise_sparse(4, pdim, prows, ptable, pindices, mapping, poffsets, None, True)
    assert ok_ref
    np.testing.assert_array_equal(bits(pout.cpu().numpy()), bits(pref))


def test_plan_reports_a_bad_index_and_peer_layout(gpu_ctx, oracle):
    """num_peers = 2 on one GPU: bag b goes to row b % bags_per_peer of buffer
    b // bags_per_peer.  Then an out-of-range index in one of the tables makes
    the whole call report false."""
    rng = np.random.default_rng(7300)
    batch, half = 40, 20
    dims = [(4, 64), (4, 64), (8, 128)]
    total = sum(d for _, d in dims)
    bufs = [torch.zeros(half * total, dtype=torch.float16, device="cuda") for _ in range(2)]
    calls, peer_ptrs, expect, col, keep, bad = [], [], [], 0, [], None
    for i, (bit_rate, dim) in enumerate(dims):
        rows = 500
        table = random_fused_table(rng, rows, dim, bit_rate)
        _, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 10, np.int64, np.int32)
        kern = make_kernel(bit_rate, dim, False, False, False, True, np.int64, np.int32, np.float16, output_stride=total)
        d = [dev(table), dev(indices), dev(offsets)]
        keep.append(d)
        calls.append((kern, batch, n, rows, d[0], d[1], d[2], None, None, None))
        peer_ptrs.append([b.data_ptr() + 2 * col for b in bufs])
        ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, None, False, np.float16)
        expect.append((col, dim, ref.reshape(batch, dim)))
        col += dim
        if i == 1:
            bad = (d[1], n, rows)
    plan = F.MultiTablePlan(calls, slot=13, peer_ptrs=peer_ptrs, bags_per_peer=half)
    plan.launch()
    ok, info = F.status_read(13)
    assert ok, info
    got = np.concatenate([b.cpu().numpy().reshape(half, total) for b in bufs])
    for c0, dim, ref in expect:
        np.testing.assert_array_equal(bits(np.ascontiguousarray(got[:, c0:c0 + dim])), bits(ref))
    idx, n, rows = bad
    idx[n // 2] = rows  # one past the last row
    plan.launch()
    ok, info = F.status_read(13)
    assert not ok and info[0] == 1 and info[2] == n // 2 and info[3] == rows

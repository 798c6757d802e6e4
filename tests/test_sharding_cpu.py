"""Host-side logic of the table-wise sharding, on CPU: the placement plan and
the batch-wise redistribution of pooled rows, the latter run as two gloo ranks
(the same code runs over NCCL on GPUs)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fbgemm_b200.sharding import TableWisePlan, assemble_columns, exchange_pooled, expected_cost
from fbgemm_b200.workloads import TableSpec, config3_tables, config4_tables, fused_row_bytes


def test_plan_balances_cost_not_count():
    specs = config3_tables()
    assert len(specs) == 64
    assert {s.bit_rate for s in specs} <= {8, 4, 2} and {s.dim for s in specs} <= {64, 128, 256}
    assert all(1_000_000 <= s.rows <= 20_000_000 for s in specs)
    costs = [expected_cost(s, 16384, 30.0) for s in specs]
    for world in (1, 2, 4, 8):
        plan = TableWisePlan.balanced(costs, [s.dim for s in specs], world)
        loads = [sum(costs[t] for t in plan.tables_of(r)) for r in range(world)]
        assert sum(len(plan.tables_of(r)) for r in range(world)) == 64
        assert max(loads) <= 1.10 * (sum(costs) / world)          # within 10 % of perfect
        assert plan.total_dim == sum(s.dim for s in specs)
        # the columns of all tables tile [0, total_dim) without gaps, grouped by owner rank
        spans = sorted((plan.column_start(t), plan.column_start(t) + specs[t].dim, plan.owner[t]) for t in range(64))
        assert spans[0][0] == 0 and spans[-1][1] == plan.total_dim
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert [o for _, _, o in spans] == sorted(o for _, _, o in spans)
    # deterministic
    assert TableWisePlan.balanced(costs, [s.dim for s in specs], 8).owner == \
        TableWisePlan.balanced(costs, [s.dim for s in specs], 8).owner


def test_uniform_tables_split_evenly():
    specs = config4_tables()
    assert len(specs) == 256 and fused_row_bytes(4, 128) == 68
    plan = TableWisePlan.balanced([1.0] * 256, [128] * 256, 8)
    assert [len(plan.tables_of(r)) for r in range(8)] == [32] * 8
    assert specs[0].rows * 68 * 32 < 180e9   # 32 tables of 2.72 GB fit one B200


def test_assemble_columns_single_rank():
    plan = TableWisePlan([0, 0], [3, 2], 1)
    recv = torch.arange(4 * 5, dtype=torch.float32)
    out = assemble_columns(recv, plan, 4)
    assert torch.equal(out, recv.view(4, 5))


def pooled_value(table, bag, col):
    return table * 1000.0 + bag + col / 64.0


def _rank_main(rank, world, port, dims, owner, B, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = TableWisePlan(owner, dims, world)
        # what this rank's lookups would have produced: all bags, its own tables' columns
        cols = []
        for t in plan.tables_of(rank):
            bag = torch.arange(B, dtype=torch.float32).view(B, 1)
            col = torch.arange(dims[t], dtype=torch.float32).view(1, -1)
            cols.append(pooled_value(t, bag, col))
        local_out = torch.cat(cols, dim=1) if cols else torch.zeros((B, 0))
        out = exchange_pooled(local_out.contiguous(), plan, rank)
        rows = B // world
        want = torch.empty((rows, plan.total_dim))
        for t in range(len(dims)):
            c0 = plan.column_start(t)
            bag = torch.arange(rank * rows, (rank + 1) * rows, dtype=torch.float32).view(rows, 1)
            col = torch.arange(dims[t], dtype=torch.float32).view(1, -1)
            want[:, c0:c0 + dims[t]] = pooled_value(t, bag, col)
        q.put((rank, bool(torch.equal(out, want)), tuple(out.shape)))
    finally:
        dist.destroy_process_group()


def test_batchwise_redistribution_two_gloo_ranks():
    dims = [4, 8, 2, 6, 4]
    owner = [1, 0, 1, 0, 1]     # uneven: rank 0 owns 14 columns, rank 1 owns 10
    world, B = 2, 12
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, dims, owner, B, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True, (6, 24)), (1, True, (6, 24))]


def _rank_that_may_leave(rank, world, port, leaver, q):
    """Rank `leaver` raises before the redistribution (a failure made on the
    host); the others must see their exchange fail within the process group's
    short timeout instead of waiting for ever."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    plan = TableWisePlan([0, 1], [4, 4], world)
    local_out = torch.full((8, 4), float(rank))
    t0 = time.monotonic()
    try:
        if rank == leaver:
            raise RuntimeError("this rank's lookup failed")       # never joins the exchange
        exchange_pooled(local_out, plan, rank)
        q.put((rank, "completed", time.monotonic() - t0))
    except RuntimeError as e:
        kind = "left" if "lookup failed" in str(e) else "exchange failed"
        q.put((rank, kind, time.monotonic() - t0))
    # no destroy_process_group: the survivor's group is broken, the leaver just exits


def test_a_rank_that_leaves_is_detected_by_the_others():
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_that_may_leave, args=(r, world, port, 1, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict((r, (kind, dt)) for r, kind, dt in (q.get(timeout=120) for _ in procs))
    for p in procs:
        p.join(timeout=60)
    assert results[1][0] == "left"
    assert results[0][0] == "exchange failed", results      # detected, not hung
    assert results[0][1] < 60


def _rank_with_padded_buffer(rank, world, port, dims, owner, B, q):
    """As ShardedLookup.exchange does it: the local buffer has at least one
    column even on a rank that owns no table; only the rank's own columns are
    sent."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = TableWisePlan(owner, dims, world)
        local = torch.full((B, max(plan.local_dim(rank), 1)), -1.0)
        col0 = 0
        for t in plan.tables_of(rank):
            bag = torch.arange(B, dtype=torch.float32).view(B, 1)
            col = torch.arange(dims[t], dtype=torch.float32).view(1, -1)
            local[:, col0:col0 + dims[t]] = pooled_value(t, bag, col)
            col0 += dims[t]
        out = exchange_pooled(local[:, :plan.local_dim(rank)].contiguous(), plan, rank)
        rows = B // world
        want = torch.empty((rows, plan.total_dim))
        for t in range(len(dims)):
            c0 = plan.column_start(t)
            bag = torch.arange(rank * rows, (rank + 1) * rows, dtype=torch.float32).view(rows, 1)
            col = torch.arange(dims[t], dtype=torch.float32).view(1, -1)
            want[:, c0:c0 + dims[t]] = pooled_value(t, bag, col)
        q.put((rank, bool(torch.equal(out, want)), tuple(out.shape)))
    finally:
        dist.destroy_process_group()


def test_more_ranks_than_tables():
    """Rank 1 owns nothing: it sends zero columns and still receives its slice of everyone else's."""
    dims, owner, world, B = [4, 6], [2, 0], 3, 12
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_with_padded_buffer, args=(r, world, port, dims, owner, B, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(r, True, (4, 10)) for r in range(3)]

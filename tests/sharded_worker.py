"""One rank of the multi-GPU sharded-lookup check (run by test_sharded_gpu.py
through torch.distributed.run).  Each rank owns some tables, pools the global
batch for them in both redistribution modes, and checks its slice of the
batch-wise output against the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    from fbgemm_b200 import embedding as E
    from fbgemm_b200.sharding import ShardedLookup, TableWisePlan, expected_cost
    from fbgemm_b200.workloads import Batch, TableSpec
    from oracle.checker import Oracle

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    oracle = Oracle()
    specs = [TableSpec(3000 + 500 * t, (64, 128, 256)[t % 3], (8, 4, 2)[(t // 2) % 3], 100 + t) for t in range(7)]
    B = 96 * world
    plan = TableWisePlan.balanced([expected_cost(s, B, 10) for s in specs], [s.dim for s in specs], world)
    # every rank builds the same batches (same seed), as if the inputs had been distributed already
    batches = {}
    for t, s in enumerate(specs):
        g = torch.Generator().manual_seed(1000 + t)
        lengths = torch.randint(0, 21, (B,), generator=g)
        off = torch.zeros(B + 1, dtype=torch.int32)
        off[1:] = torch.cumsum(lengths, 0).to(torch.int32)
        idx = torch.randint(0, s.rows, (int(off[-1]),), generator=g, dtype=torch.int32)
        batches[t] = Batch(idx.to(dev), off.to(dev), None, B, int(off[-1]), int(off[-1]))
    results = {}
    for mode in ("p2p", "nccl"):
        sl = ShardedLookup(specs, plan, rank, B, dev, torch.float16, mode=mode)
        sl.launch({t: batches[t] for t in sl.local})
        if mode == "nccl":
            sl.exchange()
        sl.barrier()
        for i in range(len(sl.local)):
            ok, info = E.status_read(i, dev.index)
            assert ok, info
        results[mode] = sl.out[0].cpu().numpy()
        tables = {t: sl.tables[t].cpu().numpy() for t in sl.local}
    # the oracle needs every table: gather the ones other ranks own
    all_tables = [None] * world
    dist.all_gather_object(all_tables, tables)
    merged = {}
    for d in all_tables:
        merged.update(d)
    rows = B // world
    want = np.zeros((rows, plan.total_dim), dtype=np.float16)
    for t, s in enumerate(specs):
        off = batches[t].offsets.cpu().numpy()
        idx = batches[t].indices.cpu().numpy()
        lo, hi = rank * rows, (rank + 1) * rows
        ok, ref = oracle.spmdm(s.bit_rate, s.dim, s.rows, merged[t], idx[off[lo]:off[hi]], off[lo:hi + 1], None,
                               False, np.float16)
        assert ok
        c0 = plan.column_start(t)
        want[:, c0:c0 + s.dim] = ref.reshape(rows, s.dim)
    for mode, got in results.items():
        assert (got.view(np.uint16) == want.view(np.uint16)).all(), f"rank {rank} mode {mode} differs from the oracle"
    dist.barrier()

    # Steps ordered on the device only: no host barrier between them, two
    # buffers, new indices every step.  Each rank checks its own slice - rows
    # that peers stored - as soon as its stream is past the "ready" wait.
    def step_inputs(step):
        host = {}
        for t, s in enumerate(specs):
            g = torch.Generator().manual_seed(5000 + 100 * step + t)
            lengths = torch.randint(0, 17, (B,), generator=g)
            off = torch.zeros(B + 1, dtype=torch.int32)
            off[1:] = torch.cumsum(lengths, 0).to(torch.int32)
            idx = torch.randint(0, s.rows, (int(off[-1]),), generator=g, dtype=torch.int32)
            host[t] = (idx.numpy(), off.numpy())
        return host

    def expected(host):
        w = np.zeros((rows, plan.total_dim), dtype=np.float16)
        lo, hi = rank * rows, (rank + 1) * rows
        for t, s in enumerate(specs):
            idx, off = host[t]
            ok, ref = oracle.spmdm(s.bit_rate, s.dim, s.rows, merged[t], idx[off[lo]:off[hi]], off[lo:hi + 1], None,
                                   False, np.float16)
            assert ok
            c0 = plan.column_start(t)
            w[:, c0:c0 + s.dim] = ref.reshape(rows, s.dim)
        return w

    sl = ShardedLookup(specs, plan, rank, B, dev, torch.float16, mode="p2p", num_buffers=2,
                       tables={t: torch.from_numpy(merged[t]).to(dev) for t in plan.tables_of(rank)})
    streams = [torch.cuda.Stream() for _ in range(2)]
    for step in range(6):
        host = step_inputs(step)
        b = {t: Batch(torch.from_numpy(host[t][0]).to(dev), torch.from_numpy(host[t][1]).to(dev), None, B,
                      len(host[t][0]), len(host[t][0])) for t in sl.local}
        buf = step % 2
        n = sl.step(b, buffer=buf, slot_base=100, streams=streams)
        got = sl.out[buf].cpu().numpy()
        sl.release(buf, n)
        for i in range(len(sl.local)):
            ok, info = E.status_read(100 + i, dev.index)
            assert ok, (step, info)
        assert (got.view(np.uint16) == expected(host).view(np.uint16)).all(), f"rank {rank} ordered step {step} differs"
    dist.barrier()

    # The same ordered steps on buffers from the library's own rendezvous (CUDA IPC handles through the process
    # group) instead of torch's symmetric memory.
    sl_ipc = ShardedLookup(specs, plan, rank, B, dev, torch.float16, mode="p2p", num_buffers=2, tables=sl.tables,
                           rendezvous="ipc")
    for step in range(4):
        host = step_inputs(50 + step)
        b = {t: Batch(torch.from_numpy(host[t][0]).to(dev), torch.from_numpy(host[t][1]).to(dev), None, B,
                      len(host[t][0]), len(host[t][0])) for t in sl_ipc.local}
        buf = step % 2
        n = sl_ipc.step(b, buffer=buf, slot_base=150, streams=streams)
        got = sl_ipc.out[buf].cpu().numpy()
        sl_ipc.release(buf, n)
        for i in range(len(sl_ipc.local)):
            ok, info = E.status_read(150 + i, dev.index)
            assert ok, (step, info)
        assert (got.view(np.uint16) == expected(host).view(np.uint16)).all(), f"rank {rank} ipc step {step} differs"
    torch.cuda.synchronize()
    dist.barrier()
    sl_ipc.close()

    # Host arrays in, this rank's slice out, through fbgemm_b200_multi_host_* with the counters.
    sl = ShardedLookup(specs, plan, rank, B, dev, torch.float16, mode="p2p", num_buffers=2, tables=sl.tables)
    calls = [sl.make_host_call(bf, {t: 20 * B for t in sl.local}, slot=200 + bf) for bf in range(2)]
    outs = [torch.zeros((rows, plan.total_dim), dtype=torch.float16).pin_memory().numpy() for _ in range(2)]
    hosts = {}
    for step in range(6):
        bf = step % 2
        if step >= 2:
            ok, info = calls[bf].wait()
            assert ok, (step, info)
            assert (outs[bf].view(np.uint16) == expected(hosts[step - 2]).view(np.uint16)).all(), \
                f"rank {rank} host step {step - 2} differs"
        hosts[step] = step_inputs(100 + step)
        calls[bf].submit([hosts[step][t][0] for t in sl.local], [hosts[step][t][1] for t in sl.local], None, outs[bf])
    for step in (4, 5):
        ok, info = calls[step % 2].wait()
        assert ok, (step, info)
        assert (outs[step % 2].view(np.uint16) == expected(hosts[step]).view(np.uint16)).all()
    dist.barrier()
    if rank == 0:
        print(f"SHARDED_OK world={world} tables={len(specs)} total_dim={plan.total_dim}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Table-wise sharding of a multi-table quantized embedding-bag lookup over the
GPUs of one box, with the pooled rows redistributed batch-wise.

Every table lives wholly on one GPU.  Each GPU pools the WHOLE (global) batch
for the tables it owns; the pooled rows then have to reach the GPU that owns
their slice of the batch: rank g ends up with rows [g*B/G, (g+1)*B/G) of every
table, columns ordered by owner rank and, within a rank, by table - the layout
the reference's multi-table caller produces on one host
(``output + D_start`` with ``output_stride = total_D``,
fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:343-473
of FBGEMM), cut batch-wise.

Two ways to get them there:

* ``mode="p2p"`` (the product): the lookup kernel itself stores each pooled
  row into the destination GPU's output buffer over NVLink
  (``fbgemm_b200_spmdm_launch_sharded``): lookup and all-to-all are one kernel,
  no staging buffer, no collective call.  The output buffers are symmetric
  memory (``torch.distributed._symmetric_memory``), which hands every rank the
  peers' buffer addresses.  Plain peer stores only - no multicast.  When a
  buffer may be read, and when it may be overwritten, is settled on the device
  by counters in the same symmetric memory (``fbgemm_b200_peer_signal`` /
  ``fbgemm_b200_peer_wait``): ``step`` below = wait for the peers' acks of the
  buffer's previous use, look up, publish "ready", wait for the peers' "ready";
  ``release`` publishes the ack once the consumer is done with the rows.
* ``mode="nccl"`` (the baseline): pool into a local ``[B, sum D_local]``
  buffer, then ``all_to_all_single`` over NCCL and a local copy into the
  column blocks.

``TableWisePlan`` and ``assemble_columns`` are plain host logic and are tested
on CPU ranks (gloo).
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import math

import numpy as np
import torch

from . import _capi
from .workloads import TableSpec, fused_row_bytes


@dataclasses.dataclass
class TableWisePlan:
    """Which rank owns which table, and where each table's columns sit in the
    batch-wise output ``[B/G, total_dim]``."""
    owner: list[int]            # owner[t]
    dims: list[int]             # dims[t]
    world_size: int

    @staticmethod
    def balanced(costs: list[float], dims: list[int], world_size: int) -> "TableWisePlan":
        """Greedy longest-processing-time assignment on expected gathered bytes
        (tables differ in row width and pooling factor, so balancing the table
        COUNT would not balance the work)."""
        load = [0.0] * world_size
        owner = [0] * len(costs)
        for t in sorted(range(len(costs)), key=lambda i: (-costs[i], i)):
            r = min(range(world_size), key=lambda i: (load[i], i))
            owner[t] = r
            load[r] += costs[t]
        return TableWisePlan(owner, list(dims), world_size)

    def tables_of(self, rank: int) -> list[int]:
        return [t for t, o in enumerate(self.owner) if o == rank]

    def local_dim(self, rank: int) -> int:
        return sum(self.dims[t] for t in self.tables_of(rank))

    @property
    def total_dim(self) -> int:
        return sum(self.dims)

    def rank_column_start(self, rank: int) -> int:
        return sum(self.local_dim(r) for r in range(rank))

    def column_start(self, table: int) -> int:
        """First column of `table` in the batch-wise output."""
        r = self.owner[table]
        start = self.rank_column_start(r)
        for t in self.tables_of(r):
            if t == table:
                return start
            start += self.dims[t]
        raise ValueError(table)


# Picoseconds per pooled row as (constant, per column), fitted per bit width to the
# times measured on B200 over the nine (bit width, D) classes of the mixed
# configuration (16 384 bags, Poisson(30) lengths, 12 M-row tables): 8-bit rows
# 24.5 / 41.6 / 67.1 ps at D = 64 / 128 / 256, 4-bit 22.3 / 37.2 / 65.3, 2-bit
# 20.1 / 34.6 / 60.6.
_ROW_COST_PS = {8: (10.3, 0.222), 4: (8.0, 0.224), 2: (6.6, 0.211)}
# A larger table costs a little more per row (fewer of its rows stay in L2):
# 2 M against 12 M rows is 1.5 ps on average over the nine classes, i.e. about
# 0.84 ps per e-fold of rows.
_ROW_COST_PS_PER_LOG_ROWS = 0.84
_ROW_COST_ROWS = 12e6


def expected_cost(spec: TableSpec, bags: int, mean_len: float) -> float:
    """Expected time of one table's lookup, in picoseconds.  The lookup is
    bound by the per-column arithmetic, not by the bytes of the row - a pooled
    row costs about 7 + 0.24 * D ps whatever its bit width - so balancing on
    bytes would overload the ranks that own narrow-bit tables.  The per-width
    fit matters at eight ranks: measured shard by shard, the slowest of eight
    shards balanced with one line for all widths took 3.5 % longer than the
    mean, with this fit 2.3 %, with the table-size term 1.5 %."""
    const, per_column = _ROW_COST_PS.get(spec.bit_rate, (7.0, 0.24))
    size_term = _ROW_COST_PS_PER_LOG_ROWS * math.log(max(spec.rows, 1) / _ROW_COST_ROWS)
    return bags * mean_len * (const + per_column * spec.dim + size_term)


def exchange_pooled(local_out: torch.Tensor, plan: TableWisePlan, rank: int, group=None) -> torch.Tensor:
    """The baseline redistribution.  ``local_out`` is ``[B, local_dim(rank)]``
    (all bags, this rank's columns); returns ``[B/G, total_dim]`` (this rank's
    bags, every rank's columns).  Works on any backend (NCCL on GPUs, gloo on
    CPU ranks)."""
    import torch.distributed as dist

    G = plan.world_size
    B = local_out.shape[0]
    assert B % G == 0, "the global batch must divide evenly over the ranks"
    rows = B // G
    in_splits = [rows * plan.local_dim(rank)] * G
    out_splits = [rows * plan.local_dim(r) for r in range(G)]
    recv = torch.empty(sum(out_splits), dtype=local_out.dtype, device=local_out.device)
    dist.all_to_all_single(recv, local_out.reshape(-1), out_splits, in_splits, group=group)
    return assemble_columns(recv, plan, rows)


def assemble_columns(recv: torch.Tensor, plan: TableWisePlan, rows: int) -> torch.Tensor:
    """``recv`` holds, rank after rank, the ``[rows, local_dim(r)]`` block that
    rank r pooled for our bags; lay the blocks side by side."""
    out = torch.empty((rows, plan.total_dim), dtype=recv.dtype, device=recv.device)
    at = 0
    for r in range(plan.world_size):
        d = plan.local_dim(r)
        if d:
            c0 = plan.rank_column_start(r)
            out[:, c0:c0 + d] = recv[at:at + rows * d].view(rows, d)
        at += rows * d
    return out


class ShardedLookup:
    """The tables one rank owns plus the machinery to pool a global batch for
    them and deliver the rows batch-wise.  One instance per process (one
    process per GPU)."""

    def __init__(self, specs: list[TableSpec], plan: TableWisePlan, rank: int, global_batch: int,
                 device: torch.device, out_dtype=torch.float16, mode: str = "p2p", num_buffers: int = 1,
                 tables: dict[int, torch.Tensor] | None = None, group=None, weighted: bool = False,
                 index_dtype=np.int32, offset_dtype=np.int32, route_local: bool | str = False,
                 rendezvous: str = "symmetric_memory"):
        import torch.distributed as dist

        from . import embedding as E
        from .workloads import random_table

        assert mode in ("p2p", "nccl")
        self.specs, self.plan, self.rank, self.device, self.mode = specs, plan, rank, device, mode
        self.world = plan.world_size
        assert global_batch % self.world == 0
        self.B, self.rows = global_batch, global_batch // self.world
        self.out_dtype = out_dtype
        self.local = plan.tables_of(rank)
        self.group = group if group is not None else (dist.group.WORLD if self.world > 1 else None)
        self.tables = {t: (tables[t] if tables and t in tables else
                           random_table(specs[t].rows, specs[t].dim, specs[t].bit_rate, device, specs[t].seed))
                       for t in self.local}
        np_out = np.float16 if out_dtype == torch.float16 else np.float32
        self.kernels = {}
        for t in self.local:
            s = specs[t]
            stride = plan.total_dim if mode == "p2p" else max(plan.local_dim(rank), 1)
            kw = dict(index_dtype=index_dtype, offset_dtype=offset_dtype, out_dtype=np_out, output_stride=stride)
            self.kernels[t] = (E.GenerateEmbeddingSpMDMWithStrides(s.dim, weighted, False, **kw) if s.bit_rate == 8
                               else E.GenerateEmbeddingSpMDMNBitWithStrides(s.bit_rate, s.dim, weighted, False, **kw))
        self.ctx = E.get_context(device.index)
        esize = 2 if out_dtype == torch.float16 else 4
        self.num_buffers = num_buffers
        if mode == "p2p":
            # Output buffers and counters every rank can address: torch's symmetric memory, or (rendezvous="ipc") the
            # library's own peer buffers, their CUDA IPC handles exchanged through the process group.
            # Counters: [ready|ack][buffer][writer rank], 8 bytes each, zero to start with.
            out_shape, flag_shape = (num_buffers, self.rows, plan.total_dim), (2, num_buffers, self.world)
            assert rendezvous in ("symmetric_memory", "ipc")
            if self.world == 1:
                self.out = torch.zeros(out_shape, dtype=out_dtype, device=device)
                self._flags = torch.zeros(flag_shape, dtype=torch.int64, device=device)
                base, self._flag_base = [self.out.data_ptr()], [self._flags.data_ptr()]
            elif rendezvous == "ipc":
                self.out, base = self._ipc_buffer(out_shape, out_dtype)
                self._flags, self._flag_base = self._ipc_buffer(flag_shape, torch.int64)
            else:
                import torch.distributed._symmetric_memory as symm

                self.out = symm.empty(out_shape, dtype=out_dtype, device=device)
                base = [int(p) for p in symm.rendezvous(self.out, self.group).buffer_ptrs]
                self._flags = symm.empty(flag_shape, dtype=torch.int64, device=device)
                self._flags.zero_()
                self._flag_base = [int(p) for p in symm.rendezvous(self._flags, self.group).buffer_ptrs]
            if self.world > 1:
                torch.cuda.synchronize(device)
                dist.barrier(group=self.group)   # nobody signals before everybody's counters are zero
            self.steps = [0] * num_buffers       # steps begun per buffer
            buf_bytes = self.rows * plan.total_dim * esize
            # peer pointer arrays per (buffer, table): column offset folded in
            self._peer_ptrs = {}
            for b in range(num_buffers):
                for t in self.local:
                    col = plan.column_start(t) * esize
                    # route_local (a measuring aid): every slice's rows go to THIS rank's buffer, so the same
                    # kernels run with no store leaving the GPU - or, with route_local="next", to the next
                    # rank's buffer, so that every store crosses NVLink; the buffer's contents are then meaningless
                    if route_local == "next":
                        dest = [base[(self.rank + 1) % self.world]] * self.world
                    else:
                        dest = [base[self.rank if route_local else r] for r in range(self.world)]
                    arr = (C.c_void_p * self.world)(*[d + b * buf_bytes + col for d in dest])
                    self._peer_ptrs[(b, t)] = arr
        else:
            self.local_out = torch.zeros((num_buffers, self.B, max(plan.local_dim(rank), 1)), dtype=out_dtype,
                                         device=device)
            self.out = torch.zeros((num_buffers, self.rows, plan.total_dim), dtype=out_dtype, device=device)

    def _ipc_buffer(self, shape, dtype):
        """A zeroed device tensor of ``shape`` in a buffer the peer processes
        can map (``fbgemm_b200_peer_buffer_*``), and the addresses of every
        rank's copy as seen from this process."""
        import torch.distributed as dist

        lib = _capi.lib()
        nbytes = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        ptr, handle = C.c_void_p(), C.create_string_buffer(_capi.IPC_HANDLE_BYTES)
        _capi.check(lib.fbgemm_b200_peer_buffer_alloc(self.ctx.handle, nbytes, C.byref(ptr), handle), "peer_buffer_alloc")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=self.group)
        base = []
        for r in range(self.world):
            if r == self.rank:
                base.append(int(ptr.value))
            else:
                peer = C.c_void_p()
                _capi.check(lib.fbgemm_b200_peer_buffer_open(self.ctx.handle, handles[r], C.byref(peer)), "peer_buffer_open")
                base.append(int(peer.value))
        self._ipc_keep = getattr(self, "_ipc_keep", []) + [(int(ptr.value), [b for r, b in enumerate(base) if r != self.rank])]

        class _Raw:   # the buffer as torch sees it (__cuda_array_interface__)
            pass

        raw = _Raw()
        typestr = {torch.float16: "<f2", torch.float32: "<f4", torch.int64: "<i8"}[dtype]
        raw.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr.value), False),
                                        "version": 2, "strides": None}
        return torch.as_tensor(raw, device=self.device), base

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (``rendezvous="ipc"``);
        every rank calls it, after a barrier that ends the last step."""
        lib = _capi.lib()
        keep, self._ipc_keep = getattr(self, "_ipc_keep", []), []
        for _, peers in keep:
            for p in peers:
                lib.fbgemm_b200_peer_buffer_close(self.ctx.handle, p)
        if keep and self.world > 1:
            import torch.distributed as dist

            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)   # nobody frees what a peer still has mapped
        for own, _ in keep:
            lib.fbgemm_b200_peer_buffer_free(self.ctx.handle, own)

    def launch(self, batches: dict, buffer: int = 0, slot_base: int = 0, stream=None, streams=None) -> None:
        """Enqueue the lookups of every local table for one global batch
        (``batches[t]`` = workloads.Batch with B bags).  In p2p mode the rows are
        on their way to their final place when the kernels end; in nccl mode
        call ``exchange`` afterwards.  ``streams`` (a list of stream handles)
        spreads the tables round-robin so that their kernels overlap."""
        lib = _capi.lib()
        if stream is None and not streams:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        col = 0
        for i, t in enumerate(self.local):
            b, s, k = batches[t], self.specs[t], self.kernels[t]
            slot = (slot_base + i) % 512
            if streams:
                stream = streams[i % len(streams)]
            if self.mode == "p2p":
                rc = lib.fbgemm_b200_spmdm_launch_sharded(
                    self.ctx.handle, C.byref(k.cfg), b.output_size, b.index_size, s.rows,
                    self.tables[t].data_ptr(), b.indices.data_ptr(), b.offsets.data_ptr(),
                    b.weights.data_ptr() if (k.cfg.has_weight and b.weights is not None) else None,
                    self._peer_ptrs[(buffer, t)], self.world, self.rows, slot, stream)
                _capi.check(rc, "fbgemm_b200_spmdm_launch_sharded")
            else:
                out = self.local_out[buffer].view(-1)[col:]
                k.launch(b.output_size, b.index_size, s.rows, self.tables[t], b.indices, b.offsets,
                         b.weights if k.cfg.has_weight else None, out, slot=slot, stream=stream)
                col += s.dim

    def make_plan(self, batches: dict, buffer: int = 0, slot: int = 0):
        """The same lookups as ``launch`` as a multi-table plan
        (``fbgemm_b200_multi_plan_*``): the local tables grouped by kernel
        variant, one kernel launch per group, for this input set and output
        buffer.  Call ``.launch(stream)`` on the result."""
        from .embedding import MultiTablePlan

        calls, peers, col = [], [], 0
        for t in self.local:
            b, s, k = batches[t], self.specs[t], self.kernels[t]
            out = None
            if self.mode == "p2p":
                peers.append([int(p) for p in self._peer_ptrs[(buffer, t)]])
            else:
                out = self.local_out[buffer].view(-1)[col:]
                col += s.dim
            calls.append((k, b.output_size, b.index_size, s.rows, self.tables[t], b.indices, b.offsets,
                          b.weights if k.cfg.has_weight else None, out, None))
        if self.mode == "p2p":
            return MultiTablePlan(calls, self.device.index, slot, peer_ptrs=peers, bags_per_peer=self.rows)
        return MultiTablePlan(calls, self.device.index, slot)

    def exchange(self, buffer: int = 0) -> torch.Tensor:
        """nccl mode: the all-to-all and the column assembly (on the current stream)."""
        assert self.mode == "nccl"
        if self.world == 1:
            self.out[buffer].copy_(self.local_out[buffer][:, :self.plan.total_dim])
        else:
            # a rank that owns no table sends nothing (its local buffer has one spare column)
            mine = self.local_out[buffer][:, :self.plan.local_dim(self.rank)].contiguous()
            self.out[buffer].copy_(exchange_pooled(mine, self.plan, self.rank, self.group))
        return self.out[buffer]

    # ---- device-side ordering of the peer stores (p2p mode) ------------------------

    READY, ACK = 0, 1

    def _flag_addr(self, kind: int, buffer: int, writer: int, on_rank: int) -> int:
        return self._flag_base[on_rank] + ((kind * self.num_buffers + buffer) * self.world + writer) * 8

    def signal(self, kind: int, buffer: int, value: int, stream=None) -> None:
        """After everything already on ``stream``: write ``value`` to this rank's
        word of counter ``kind`` of ``buffer`` on every rank."""
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        arr = (C.c_void_p * self.world)(*[self._flag_addr(kind, buffer, self.rank, g) for g in range(self.world)])
        _capi.check(_capi.lib().fbgemm_b200_peer_signal(self.ctx.handle, arr, self.world, value, stream), "peer_signal")

    def wait(self, kind: int, buffer: int, value: int, slot: int = 0, stream=None, timeout_us: int = 2_000_000) -> None:
        """Hold ``stream`` until every rank's word of counter ``kind`` of
        ``buffer`` on this rank has reached ``value`` (or record a timeout in
        status slot ``slot``)."""
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        _capi.check(_capi.lib().fbgemm_b200_peer_wait(self.ctx.handle, self._flag_addr(kind, buffer, 0, self.rank),
                                                      self.world, value, timeout_us, slot, stream), "peer_wait")

    def step(self, batches: dict, buffer: int = 0, slot_base: int = 0, streams=None, plan=None,
             timeout_us: int = 2_000_000) -> int:
        """One whole step on the current stream, ordered on the device: wait
        until every peer has released ``buffer``'s previous rows, pool and store
        this rank's tables (``plan``: a multi-table plan made by ``make_plan``
        for this buffer, else one launch per table over ``streams``), publish
        "ready", wait for every peer's "ready".  When the stream gets past the
        last wait, this rank's ``out[buffer]`` holds every table's rows for its
        slice of the batch.  Returns the step number to pass to ``release``."""
        assert self.mode == "p2p"
        self.steps[buffer] += 1
        n = self.steps[buffer]
        cur = torch.cuda.current_stream(self.device)
        self.wait(self.ACK, buffer, n - 1, slot_base, cur.cuda_stream, timeout_us)
        if plan is not None:
            plan.launch(cur.cuda_stream)
        elif streams:
            for s in streams:
                s.wait_stream(cur)
            self.launch(batches, buffer, slot_base, streams=[s.cuda_stream for s in streams])
            for s in streams:
                cur.wait_stream(s)
        else:
            self.launch(batches, buffer, slot_base, stream=cur.cuda_stream)
        self.signal(self.READY, buffer, n, cur.cuda_stream)
        self.wait(self.READY, buffer, n, slot_base, cur.cuda_stream, timeout_us)
        return n

    def release(self, buffer: int, n: int) -> None:
        """The consumer of ``out[buffer]`` is done with step ``n`` (everything
        enqueued so far on the current stream): let the peers overwrite it."""
        self.signal(self.ACK, buffer, n)

    def make_host_call(self, buffer: int, capacities: dict, slot: int = 0, timeout_us: int = 2_000_000):
        """``fbgemm_b200_multi_host_*`` for this rank's tables and ``buffer``:
        host index arrays in, this rank's ``[B/G, total_dim]`` slice out, with
        the counters of ``buffer`` ordering the peers.  ``capacities[t]`` bounds
        the indices a step may bring for table t.  The handle counts its own
        steps: do not mix it with ``step`` on the same buffer."""
        from .embedding import MultiTableHostCall

        assert self.mode == "p2p"
        tables, peers = [], []
        for t in self.local:
            tables.append((self.kernels[t], self.B, self.specs[t].rows, self.tables[t], None, int(capacities[t])))
            peers.append([int(p) for p in self._peer_ptrs[(buffer, t)]])
        G = self.world
        ready = (C.c_void_p * G)(*[self._flag_addr(self.READY, buffer, self.rank, g) for g in range(G)])
        ack = (C.c_void_p * G)(*[self._flag_addr(self.ACK, buffer, self.rank, g) for g in range(G)])
        sync = _capi.PeerSync(G, ready, self._flag_addr(self.READY, buffer, 0, self.rank), ack,
                              self._flag_addr(self.ACK, buffer, 0, self.rank), timeout_us)
        call = MultiTableHostCall(tables, self.out[buffer], self.device.index, slot, peer_ptrs=peers,
                                  bags_per_peer=self.rows, sync=sync)
        call._sync_arrays = (ready, ack)
        return call

    def make_step_call(self, buffer: int, slot: int = 0, timeout_us: int = 2_000_000):
        """The handle of ``make_host_call`` for DEVICE index arrays
        (``MultiTableHostCall.device_args`` / ``step_device``): the whole
        ordered step - ack wait, this rank's lookups over four streams, ready
        signal and wait, release - in one call from the host per global batch."""
        if self.mode == "p2p":
            return self.make_host_call(buffer, {t: 0 for t in self.local}, slot, timeout_us)
        # the all-to-all baseline: the same one call for the lookups, rows into this rank's [B, local_dim] block
        from .embedding import MultiTableHostCall

        tables, col = [], 0
        esize = self.local_out[buffer].element_size()
        for t in self.local:
            tables.append((self.kernels[t], self.B, self.specs[t].rows, self.tables[t],
                           self.local_out[buffer].data_ptr() + col * esize, 0))
            col += self.specs[t].dim
        return MultiTableHostCall(tables, self.local_out[buffer], self.device.index, slot)

    def barrier(self) -> None:
        """All ranks' kernels (and therefore their peer stores) are complete."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier(group=self.group)
            torch.cuda.synchronize(self.device)

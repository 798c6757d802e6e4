"""Table-batched quantized embedding lookup on the GPU: the caller that sits
above the generators in the reference,
``int_nbit_split_embedding_codegen_forward_{unweighted,weighted}_cpu``
(fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:205-520
of FBGEMM).  Same arguments, same result; the tensors live in HBM.

The reference walks the tables on host threads and calls one generated kernel
per table with ``output + D_start``, ``output_stride = total_D`` and the slice
``offsets[t*B : (t+1)*B + 1]`` of the ``T*B + 1`` offsets.  Here every table is
one launch of the same lookup kernel with *absolute* offsets (the kernel is
given the whole index array and the slice of offsets, so nothing has to be
read back to the host to find where a table's indices start), all launches
enqueued without a synchronisation; or, for callers whose input buffers keep
their addresses, one multi-table plan that is built once and replayed.

Rows are INT8 / INT4 / INT2 with fp16 scale and bias *first* (the layout of
table-batched embeddings, ``scale_bias_last = False``), or scale and bias last
(fp32 pair for INT8) when ``scale_bias_last = True``, or FP32 / FP16 / FP8
values without scale and bias; each row padded to ``row_alignment`` bytes.  An
index of -1 is a pruned row (not for FP8, as in the reference).  Output FP32,
FP16 or BF16 of shape ``[B, total_D]``; INT8/INT4 output belongs to the
reference's nobag operator and is refused.
"""
from __future__ import annotations

import enum

import numpy as np
import torch

from . import embedding as E


class SparseType(enum.IntEnum):
    """fbgemm_gpu/include/fbgemm_gpu/embedding_common.h:20-32."""
    FP32 = 0
    FP16 = 1
    INT8 = 2
    INT4 = 3
    INT2 = 4
    BF16 = 5
    FP8 = 6


class PoolingMode(enum.IntEnum):
    """fbgemm_gpu/include/fbgemm_gpu/embedding_common.h:34."""
    SUM = 0
    MEAN = 1
    NONE = 2


_BITS = {SparseType.INT8: 8, SparseType.INT4: 4, SparseType.INT2: 2}
_PLAIN_BYTES = {SparseType.FP32: 4, SparseType.FP16: 2, SparseType.FP8: 1}
_OUT = {SparseType.FP32: torch.float32, SparseType.FP16: torch.float16, SparseType.BF16: torch.bfloat16}


def padded_row_size_in_bytes(dim: int, weight_ty: SparseType, row_alignment: int, scale_bias_bytes: int = 4) -> int:
    """nbit::padded_row_size_in_bytes (embedding_common.h:189-225)."""
    weight_ty = SparseType(weight_ty)
    if weight_ty in _PLAIN_BYTES:
        unpadded = dim * _PLAIN_BYTES[weight_ty]
    else:
        unpadded = dim * _BITS[weight_ty] // 8 + scale_bias_bytes
    return (unpadded + row_alignment - 1) // row_alignment * row_alignment


def _host(x, dtype):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy().astype(dtype)
    return np.asarray(x, dtype=dtype)


class IntNBitTableBatchedEmbeddingBags:
    """The tables of one table-batched operator and what does not change from
    call to call (row sizes, row counts, kernels)."""

    MAX_PLANS = 16  # cached multi-table plans (one per set of buffer addresses and sizes)

    def __init__(self, dev_weights: torch.Tensor, weights_offsets, weights_tys, D_offsets, total_D: int,
                 pooling_mode: int = PoolingMode.SUM, row_alignment: int = 1, output_dtype: int = SparseType.FP16,
                 scale_bias_last: bool = False, weighted: bool = False, index_dtype=torch.int32,
                 fp8_exponent_bits: int = 4, fp8_exponent_bias: int = 7):
        assert dev_weights.is_cuda and dev_weights.dtype == torch.uint8 and dev_weights.is_contiguous()
        self.dev_weights = dev_weights
        self.device = dev_weights.device
        self.weights_offsets = _host(weights_offsets, np.int64)
        self.weights_tys = [SparseType(int(t)) for t in _host(weights_tys, np.int64)]
        self.D_offsets = _host(D_offsets, np.int64)
        self.T = len(self.D_offsets) - 1
        self.total_D = int(total_D)
        if PoolingMode(pooling_mode) == PoolingMode.NONE:
            raise ValueError("PoolingMode.NONE (sequence output) is the reference's nobag operator, not this one")
        self.normalize = PoolingMode(pooling_mode) == PoolingMode.MEAN
        if SparseType(output_dtype) not in _OUT:
            raise ValueError("output_dtype must be FP32, FP16 or BF16 (INT8/INT4 output is the nobag operator's)")
        self.out_dtype = _OUT[SparseType(output_dtype)]
        self.weighted = bool(weighted)
        self.index_dtype = index_dtype
        np_idx = np.int32 if index_dtype == torch.int32 else np.int64
        # num_rows per table from the sorted unique physical offsets, as the reference derives it (:330-342, :369-381)
        physical = sorted(set(int(o) for o in self.weights_offsets))
        self.kernels, self.rows, self.tables = [], [], []
        for t in range(self.T):
            ty = self.weights_tys[t]
            if ty not in _BITS and ty not in _PLAIN_BYTES:
                raise ValueError(f"table {t}: weight type {ty.name} is not a row format of this path")
            D = int(self.D_offsets[t + 1] - self.D_offsets[t])
            sb_bytes = 8 if (ty == SparseType.INT8 and scale_bias_last) else 4
            D_bytes = padded_row_size_in_bytes(D, ty, row_alignment, sb_bytes)
            start = int(self.weights_offsets[t])
            nxt = [o for o in physical if o > start]
            end = nxt[0] if nxt else dev_weights.numel()
            self.rows.append((end - start) // D_bytes)
            self.tables.append(dev_weights[start:end])
            kw = dict(index_dtype=np_idx, offset_dtype=np_idx,
                      out_dtype={torch.float32: np.float32, torch.float16: np.float16,
                                 torch.bfloat16: np.uint16}[self.out_dtype])
            bf16 = self.out_dtype == torch.bfloat16
            if ty == SparseType.INT8:
                k = E.GenerateEmbeddingSpMDMWithStrides(D, self.weighted, self.normalize, 16, False, True, self.total_D,
                                                        D_bytes, scale_bias_last, False, bf16, **kw)
            elif ty in (SparseType.FP32, SparseType.FP16):
                eb = _PLAIN_BYTES[ty]
                k = E.GenerateEmbeddingSpMDMWithStrides(
                    D, self.weighted, self.normalize, 16, False, True, self.total_D, D_bytes // eb, scale_bias_last,
                    False, bf16, in_dtype=np.float32 if ty == SparseType.FP32 else np.float16, **kw)
            elif ty == SparseType.FP8:
                k = E.GenerateEmbeddingSpMDMFP8WithStrides(D, self.normalize, False, True, self.total_D, D_bytes,
                                                           fp8_exponent_bits, fp8_exponent_bias, bf16, **kw)
                k = k._k[self.weighted]
            else:
                k = E.GenerateEmbeddingSpMDMNBitWithStrides(_BITS[ty], D, self.weighted, self.normalize, 16, False, True,
                                                            self.total_D, D_bytes, scale_bias_last, bf16, **kw)
            k.cfg.absolute_offsets = 1
            self.kernels.append(k)
        self._streams = [torch.cuda.Stream(device=self.device) for _ in range(4)]
        self._plans: dict = {}

    def _calls(self, B, indices, offsets, indice_weights, output):
        flat = output.view(-1)
        n = indices.numel()
        calls = []
        for t in range(self.T):
            calls.append((self.kernels[t], B, n, self.rows[t], self.tables[t], indices, offsets[t * B:],
                          indice_weights if self.weighted else None, flat[int(self.D_offsets[t]):], None))
        return calls

    def forward(self, indices: torch.Tensor, offsets: torch.Tensor, indice_weights: torch.Tensor | None = None,
                output: torch.Tensor | None = None, slot: int = 0, use_plan: bool = False) -> torch.Tensor:
        """``offsets`` has ``T*B + 1`` entries, table after table; returns
        ``[B, total_D]``.  Asynchronous on torch's current stream; a bad index
        or offsets shows in status slot ``slot`` (``fbgemm_b200.status_read``)."""
        assert indices.dtype == offsets.dtype == self.index_dtype and indices.is_cuda and offsets.is_cuda
        assert (offsets.numel() - 1) % self.T == 0
        B = (offsets.numel() - 1) // self.T
        if self.weighted:
            assert indice_weights is not None and indice_weights.dtype == torch.float32
        if output is None:
            output = torch.zeros((B, self.total_D), dtype=self.out_dtype, device=self.device)
        if B == 0:
            return output
        calls = self._calls(B, indices, offsets, indice_weights, output)
        if use_plan:
            key = (indices.data_ptr(), offsets.data_ptr(), indice_weights.data_ptr() if self.weighted else 0,
                   output.data_ptr(), B, indices.numel(), slot)
            plan = self._plans.pop(key, None)
            if plan is None:
                plan = E.MultiTablePlan(calls, self.device.index, slot)
                while len(self._plans) >= self.MAX_PLANS:      # least recently used first
                    self._plans.pop(next(iter(self._plans)))
            self._plans[key] = plan
            plan.launch()
            return output
        cur = torch.cuda.current_stream(self.device)
        for s in self._streams:
            s.wait_stream(cur)
        for t, (k, b, n, rows, table, idx, off, w, out, _) in enumerate(calls):
            k.launch(b, n, rows, table, idx, off, w, out, slot=slot,
                     stream=self._streams[t % len(self._streams)].cuda_stream)
        for s in self._streams:
            cur.wait_stream(s)
        return output


def int_nbit_split_embedding_codegen_forward(dev_weights, weights_offsets, weights_tys, D_offsets, total_D, indices,
                                             offsets, pooling_mode, row_alignment, indice_weights=None,
                                             output_dtype=SparseType.FP16, scale_bias_last=False):
    """One call with the reference operator's arguments (the placement, UVM
    and FP8 arguments, which select other storage or other kernels, left out).
    Builds the per-table kernels every time; keep an
    ``IntNBitTableBatchedEmbeddingBags`` to amortise that."""
    op = IntNBitTableBatchedEmbeddingBags(dev_weights, weights_offsets, weights_tys, D_offsets, total_D, pooling_mode,
                                          row_alignment, output_dtype, scale_bias_last, indice_weights is not None,
                                          indices.dtype)
    return op.forward(indices, offsets, indice_weights)


def _index_tensors(indices, offsets):
    assert indices.is_cuda and offsets.is_cuda and indices.dtype == offsets.dtype
    assert indices.dtype in (torch.int32, torch.int64) and indices.is_contiguous() and offsets.is_contiguous()


def _pruned_lookup(fn_name, indices, offsets, mapping, mapping_offsets, slot):
    _index_tensors(indices, offsets)
    assert mapping.is_cuda and mapping.is_contiguous() and mapping.dtype in (torch.int32, torch.int64)
    assert mapping_offsets.is_cuda and mapping_offsets.dtype == torch.int64 and mapping_offsets.is_contiguous()
    T = mapping_offsets.numel() - 1
    assert T > 0 and (offsets.numel() - 1) % T == 0
    B = (offsets.numel() - 1) // T
    if B <= 0:
        raise ValueError("B must be positive")
    ctx = E.get_context(indices.device.index)
    dense = torch.empty_like(indices)
    fn = getattr(E._capi.lib(), fn_name)
    rc = fn(ctx.handle, T, B, E._ptr(indices), E._ptr(offsets), indices.element_size(), indices.numel(),
            E._ptr(mapping), mapping.element_size(), E._ptr(mapping_offsets), E._ptr(dense), slot,
            torch.cuda.current_stream(indices.device).cuda_stream)
    E._capi.check(rc, fn_name)
    return dense


def pruned_hashmap_lookup(indices: torch.Tensor, offsets: torch.Tensor, hash_table: torch.Tensor,
                          hash_table_offsets: torch.Tensor, slot: int = 0) -> torch.Tensor:
    """``torch.ops.fbgemm.pruned_hashmap_lookup`` of the reference
    (embedding_forward_quantized_cpu_template.cpp:524-601) on CUDA tensors:
    the dense index of every index of a table-batched call, -1 for pruned
    rows; tables whose hash table is empty keep their indices.  Asynchronous
    on torch's current stream."""
    assert hash_table.dim() == 2 and hash_table.shape[1] == 2
    return _pruned_lookup("fbgemm_b200_pruned_hashmap_lookup", indices, offsets, hash_table, hash_table_offsets, slot)


def pruned_array_lookup(indices: torch.Tensor, offsets: torch.Tensor, index_remappings: torch.Tensor,
                        index_remappings_offsets: torch.Tensor, slot: int = 0) -> torch.Tensor:
    """``torch.ops.fbgemm.pruned_array_lookup`` (same file, :605-659) on CUDA
    tensors.  An index outside its table's remapping array gives -1 and shows
    in status slot ``slot`` (``fbgemm_b200.status_read``)."""
    assert index_remappings.dim() == 1
    return _pruned_lookup("fbgemm_b200_pruned_array_lookup", indices, offsets, index_remappings,
                          index_remappings_offsets, slot)


def pruned_hashmap_insert(indices: torch.Tensor, dense_indices: torch.Tensor, offsets: torch.Tensor,
                          hash_table: torch.Tensor, hash_table_offsets: torch.Tensor, slot: int = 0) -> bool:
    """``torch.ops.fbgemm.pruned_hashmap_insert`` (same file, :124-204):
    ``hash_table`` is filled in place (start from -1 everywhere).  With host
    tensors the table is built as the reference builds it, one key after the
    other (move it to the GPU afterwards, as the reference's own GPU module
    does).  With CUDA tensors one kernel inserts all keys at once; that table
    can differ byte for byte from the host-built one, the lookups do not.
    Returns False if a table had no free slot left for a key."""
    if hash_table.is_cuda:
        for x in (indices, dense_indices, offsets, hash_table, hash_table_offsets):
            assert x.is_cuda and x.is_contiguous()
        assert indices.dtype == offsets.dtype == dense_indices.dtype and indices.dtype in (torch.int32, torch.int64)
        assert hash_table.dim() == 2 and hash_table.shape[1] == 2 and hash_table.dtype in (torch.int32, torch.int64)
        assert hash_table_offsets.dtype == torch.int64
        T = hash_table_offsets.numel() - 1
        assert T > 0 and (offsets.numel() - 1) % T == 0
        B = (offsets.numel() - 1) // T
        if B <= 0:
            raise ValueError("B must be positive")
        ctx = E.get_context(hash_table.device.index)
        rc = E._capi.lib().fbgemm_b200_pruned_hashmap_insert(
            ctx.handle, T, B, E._ptr(indices), E._ptr(dense_indices), E._ptr(offsets), indices.element_size(),
            indices.numel(), E._ptr(hash_table), hash_table.element_size(), E._ptr(hash_table_offsets), slot,
            torch.cuda.current_stream(hash_table.device).cuda_stream)
        E._capi.check(rc, "fbgemm_b200_pruned_hashmap_insert")
        return E.status_read(slot, hash_table.device.index)[0]
    for x in (indices, dense_indices, offsets, hash_table, hash_table_offsets):
        assert not x.is_cuda and x.is_contiguous()
    assert indices.dtype == offsets.dtype == dense_indices.dtype and indices.dtype in (torch.int32, torch.int64)
    assert hash_table.dim() == 2 and hash_table.shape[1] == 2 and hash_table.dtype in (torch.int32, torch.int64)
    assert hash_table_offsets.dtype == torch.int64
    T = hash_table_offsets.numel() - 1
    assert T > 0 and (offsets.numel() - 1) % T == 0
    B = (offsets.numel() - 1) // T
    if B <= 0:
        raise ValueError("B must be positive")
    rc = E._capi.lib().fbgemm_b200_pruned_hashmap_insert_host(
        T, B, indices.data_ptr(), dense_indices.data_ptr(), offsets.data_ptr(), indices.element_size(),
        hash_table.data_ptr(), hash_table.element_size(), hash_table_offsets.data_ptr())
    return bool(E._capi.check(rc, "fbgemm_b200_pruned_hashmap_insert_host"))


_SEQ_TABLE = np.dtype([("weight_offset", np.int64), ("rows", np.int64), ("row_bytes", np.int32), ("type", np.int32)])
_SEQ_OUT = {SparseType.FP32: (0, torch.float32), SparseType.FP16: (1, torch.float16),
            SparseType.BF16: (2, torch.bfloat16), SparseType.INT8: (3, torch.uint8), SparseType.INT4: (4, torch.uint8)}


class IntNBitSequenceEmbedding:
    """The sequence ("nobag", ``PoolingMode.NONE``) form of the table-batched
    operator, ``int_nbit_split_embedding_nobag_codegen_forward_unweighted_cpu``
    of the reference (embedding_forward_quantized_cpu_template.cpp:206-520):
    one output row per index, all tables of width ``D``.  Holds the table
    descriptors on the device; ``forward`` is one kernel launch."""

    def __init__(self, dev_weights: torch.Tensor, weights_offsets, weights_tys, D: int, row_alignment: int = 1,
                 output_dtype: int = SparseType.FP16, scale_bias_last: bool = False, fp8_exponent_bits: int = 4,
                 fp8_exponent_bias: int = 7):
        assert dev_weights.is_cuda and dev_weights.dtype == torch.uint8 and dev_weights.is_contiguous()
        self.dev_weights = dev_weights
        self.device = dev_weights.device
        self.D = int(D)
        offs = _host(weights_offsets, np.int64)
        tys = [SparseType(int(t)) for t in _host(weights_tys, np.int64)]
        self.T = len(offs)
        out_ty = SparseType(output_dtype)
        if out_ty not in _SEQ_OUT:
            raise ValueError("output_dtype must be FP32, FP16, BF16, INT8 or INT4")
        self.out_code, self.out_dtype = _SEQ_OUT[out_ty]
        # output row: D columns, plus the 4 bytes of fp16 scale and bias for INT8 / INT4 rows (:284-291)
        if out_ty == SparseType.INT8:
            self.out_cols = self.D + 4
        elif out_ty == SparseType.INT4:
            self.out_cols = (self.D + 8 + 1) // 2
        else:
            self.out_cols = self.D
        self.out_row_bytes = self.out_cols * torch.empty((), dtype=self.out_dtype).element_size()
        self.scale_bias_last = bool(scale_bias_last)
        self.fp8 = (int(fp8_exponent_bits), int(fp8_exponent_bias))
        physical = sorted(set(int(o) for o in offs))
        desc = np.zeros(self.T, dtype=_SEQ_TABLE)
        self.rows = []
        for t in range(self.T):
            ty = tys[t]
            if ty not in _BITS and ty not in _PLAIN_BYTES:
                raise ValueError(f"table {t}: weight type {ty.name} is not a row format of this path")
            if out_ty == SparseType.INT8 and ty != SparseType.INT8:
                raise ValueError("int8 output is only supported for int8 weights")
            if out_ty == SparseType.INT4 and ty != SparseType.INT4:
                raise ValueError("int4 output is only supported for int4 weights")
            sb_bytes = 8 if (ty == SparseType.INT8 and scale_bias_last) else 4
            row_bytes = padded_row_size_in_bytes(self.D, ty, row_alignment, sb_bytes)
            if out_ty == SparseType.INT4 and row_bytes != self.out_row_bytes:
                raise ValueError("int4 output needs table rows of (D + 8 + 1) / 2 bytes (row_alignment 1)")
            start = int(offs[t])
            nxt = [o for o in physical if o > start]
            end = nxt[0] if nxt else dev_weights.numel()
            desc[t] = (start, (end - start) // row_bytes, row_bytes, int(ty))
            self.rows.append((end - start) // row_bytes)
        self._desc = torch.from_numpy(desc.view(np.uint8).copy()).to(self.device)

    def forward(self, indices: torch.Tensor, offsets: torch.Tensor, output: torch.Tensor | None = None,
                slot: int = 0) -> torch.Tensor:
        """``offsets`` has ``T*B + 1`` entries; returns ``[indices.numel(),
        D (+ qparams)]``.  Asynchronous on torch's current stream."""
        _index_tensors(indices, offsets)
        assert (offsets.numel() - 1) % self.T == 0
        B = (offsets.numel() - 1) // self.T
        n = indices.numel()
        if output is None:
            output = torch.zeros((n, self.out_cols), dtype=self.out_dtype, device=self.device)
        assert output.is_contiguous() and output.dtype == self.out_dtype and output.numel() == n * self.out_cols
        if B == 0 or n == 0:
            return output
        ctx = E.get_context(self.device.index)
        rc = E._capi.lib().fbgemm_b200_sequence_lookup(
            ctx.handle, self.dev_weights.data_ptr(), self._desc.data_ptr(), self.T, B, self.D, indices.data_ptr(),
            offsets.data_ptr(), indices.element_size(), n, output.data_ptr(), self.out_code, self.out_row_bytes,
            int(self.scale_bias_last), self.fp8[0], self.fp8[1], slot,
            torch.cuda.current_stream(self.device).cuda_stream)
        E._capi.check(rc, "fbgemm_b200_sequence_lookup")
        return output


def int_nbit_split_embedding_nobag_codegen_forward_unweighted(
        dev_weights, weights_offsets, weights_tys, D, indices, offsets, pooling_mode=PoolingMode.NONE,
        row_alignment=1, output_dtype=SparseType.FP16, fp8_exponent_bits=4, fp8_exponent_bias=7,
        scale_bias_last=False):
    """One call with the reference operator's arguments (placement and UVM
    arguments left out; ``pooling_mode`` is accepted and, bags being one row
    long, changes nothing)."""
    op = IntNBitSequenceEmbedding(dev_weights, weights_offsets, weights_tys, D, row_alignment, output_dtype,
                                  scale_bias_last, fp8_exponent_bits, fp8_exponent_bias)
    return op.forward(indices, offsets)


def int_nbit_split_embedding_codegen_lookup_function(
        dev_weights, uvm_weights, weights_placements, weights_offsets, weights_tys, D_offsets, total_D, max_int2_D,
        max_int4_D, max_int8_D, max_float16_D, max_float32_D, indices, offsets, pooling_mode, indice_weights=None,
        output_dtype=SparseType.FP16, lxu_cache_weights=None, lxu_cache_locations=None, row_alignment=None,
        max_float8_D=None, fp8_exponent_bits=None, fp8_exponent_bias=None, scale_bias_last=False):
    """``fbgemm::int_nbit_split_embedding_codegen_lookup_function`` with the
    reference's argument list (embedding_forward_quantized_host_cpu.cpp:84-227):
    ``PoolingMode.NONE`` goes to the sequence operator with ``D`` = the largest
    of the ``max_*_D``, otherwise to the pooled operator, weighted when
    ``indice_weights`` holds anything.  All tables live in ``dev_weights`` on
    the GPU: ``uvm_weights``, ``weights_placements`` and the cache arguments
    are accepted and must describe nothing (placement is not part of this path)."""
    if uvm_weights is not None and uvm_weights.numel() > 0:
        raise ValueError("tables in unified memory are outside this path: put every table in dev_weights")
    if offsets.dtype != indices.dtype:
        offsets = offsets.to(indices.dtype)
    align = 1 if row_alignment is None else int(row_alignment)
    bits = 4 if fp8_exponent_bits is None or fp8_exponent_bits < 0 else int(fp8_exponent_bits)
    bias = 7 if fp8_exponent_bias is None or fp8_exponent_bias < 0 else int(fp8_exponent_bias)
    if PoolingMode(pooling_mode) == PoolingMode.NONE:
        max_D = max(int(max_int2_D), int(max_int4_D), int(max_int8_D), int(max_float8_D or 0), int(max_float16_D),
                    int(max_float32_D))
        return int_nbit_split_embedding_nobag_codegen_forward_unweighted(
            dev_weights, weights_offsets, weights_tys, max_D, indices, offsets, pooling_mode, align, output_dtype,
            bits, bias, scale_bias_last)
    weighted = indice_weights is not None and indice_weights.numel() > 0
    op = IntNBitTableBatchedEmbeddingBags(dev_weights, weights_offsets, weights_tys, D_offsets, total_D, pooling_mode,
                                          align, output_dtype, scale_bias_last, weighted, indices.dtype, bits, bias)
    return op.forward(indices, offsets, indice_weights if weighted else None)

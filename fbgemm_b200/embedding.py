"""Python mirror of the reference's kernel-generator API for the quantized
embedding-bag path, over the C ABI of libfbgemm_b200.so.

The generator functions carry the reference's names and argument meaning
(include/fbgemm/FbgemmEmbedding.h:65-262 of FBGEMM); template parameters become
keyword arguments (``index_dtype``, ``offset_dtype``, ``out_dtype``).  Each
returns a functor with the reference's call signature

    ok = kernel(output_size, index_size, data_size, input, indices,
                offsets_or_lengths, weights, out[, compressed_indices_table])

where the arrays are either CUDA ``torch.Tensor`` s (zero-copy, enqueued on the
current torch stream) or host ``numpy`` arrays (the table is made resident in
HBM on first use; per-call arrays travel through pinned staging buffers).
``ok`` is the reference's bool.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import threading

import numpy as np

from . import _capi
from ._capi import OUT_F16, OUT_F32, SpmdmConfig

_ctx_lock = threading.Lock()
_ctxs: dict[int, "Context"] = {}


class Context:
    """``fbgemm_b200_ctx`` of one device."""

    def __init__(self, device: int):
        self.device = device
        self._h = C.c_void_p()
        _capi.check(_capi.lib().fbgemm_b200_ctx_create(device, C.byref(self._h)), "fbgemm_b200_ctx_create")

    @property
    def handle(self):
        return self._h

    def close(self):
        if self._h:
            _capi.lib().fbgemm_b200_ctx_destroy(self._h)
            self._h = C.c_void_p()

    # -- table registry ------------------------------------------------------
    def register_table(self, host_array: np.ndarray) -> None:
        a = host_array
        assert a.flags["C_CONTIGUOUS"]
        _capi.check(_capi.lib().fbgemm_b200_table_register(self._h, a.ctypes.data, a.nbytes), "table_register")

    def unregister_table(self, host_array: np.ndarray) -> None:
        _capi.lib().fbgemm_b200_table_unregister(self._h, host_array.ctypes.data)

    def table_device_ptr(self, host_array: np.ndarray):
        return _capi.lib().fbgemm_b200_table_device_ptr(self._h, host_array.ctypes.data)


def get_context(device: int | None = None) -> Context:
    """The process-wide context of ``device`` (default: torch's current device)."""
    if device is None:
        import torch

        if not torch.cuda.is_available():
            raise _capi.Fbgemmb200Error("no CUDA device: fbgemm_b200 has no CPU fallback")
        device = torch.cuda.current_device()
    with _ctx_lock:
        ctx = _ctxs.get(device)
        if ctx is None:
            ctx = _ctxs[device] = Context(device)
        return ctx


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(_capi.lib().fbgemm_b200_launch_count())


def _np_itemsize(dt) -> int:
    return np.dtype(dt).itemsize


def _out_code(out_dtype) -> int:
    """OutType of the reference generators: fp32, or fp16 (also as raw uint16)."""
    try:
        name = np.dtype(out_dtype).name
    except TypeError:
        name = str(out_dtype).rsplit(".", 1)[-1]  # torch.float16 -> float16
    if name == "float32":
        return OUT_F32
    if name in ("float16", "uint16"):
        return OUT_F16
    if name == "bfloat16":
        return 2
    if name == "uint8":
        return 3  # no_bag only: byte copies of the indexed rows
    raise ValueError(f"OutType must be float32, float16, bfloat16 or (no_bag) uint8, got {out_dtype}")


def _is_tensor(x) -> bool:
    return hasattr(x, "data_ptr")


def _ptr(x):
    if x is None:
        return None
    if _is_tensor(x):
        assert x.is_contiguous(), "tensors must be contiguous"
        return x.data_ptr()
    assert x.flags["C_CONTIGUOUS"], "arrays must be contiguous"
    return x.ctypes.data


class SpmdmKernel:
    """The functor a generator returns.  Holds only the configuration."""

    def __init__(self, cfg: SpmdmConfig, rowwise_sparse: bool):
        self.cfg = cfg
        self.rowwise_sparse = rowwise_sparse
        _capi.check(_capi.lib().fbgemm_b200_spmdm_check_config(C.byref(cfg)), "generator arguments")

    # -- the reference's functor signature ----------------------------------
    def __call__(self, output_size, index_size, data_size, input, indices, offsets_or_lengths,
                 weights, out, compressed_indices_table=None) -> bool:
        if self.rowwise_sparse and compressed_indices_table is None:
            raise ValueError("row-wise sparse kernels need a compressed_indices_table")
        if not self.rowwise_sparse and compressed_indices_table is not None:
            raise ValueError("this kernel was not generated for row-wise sparse tables")
        self._check_dtypes(indices, offsets_or_lengths)
        lib = _capi.lib()
        if _is_tensor(input):
            import torch

            dev = input.device.index
            ctx = get_context(dev)
            stream = torch.cuda.current_stream(dev).cuda_stream
            rc = lib.fbgemm_b200_spmdm(
                ctx.handle, C.byref(self.cfg), output_size, index_size, data_size, _ptr(input), _ptr(indices),
                _ptr(offsets_or_lengths), _ptr(weights) if self.cfg.has_weight else None, _ptr(out),
                _ptr(compressed_indices_table), stream)
        else:
            ctx = get_context()
            rc = lib.fbgemm_b200_spmdm_host(
                ctx.handle, C.byref(self.cfg), output_size, index_size, data_size, _ptr(input), _ptr(indices),
                _ptr(offsets_or_lengths), _ptr(weights) if self.cfg.has_weight else None, _ptr(out),
                _ptr(compressed_indices_table))
        return bool(_capi.check(rc, "fbgemm_b200 lookup"))

    # -- asynchronous forms (no counterpart in the reference) ------------------
    def launch(self, output_size, index_size, data_size, input, indices, offsets_or_lengths, weights, out,
               compressed_indices_table=None, slot: int = 0, stream=None) -> None:
        """Enqueue on ``stream`` (int handle; default torch's current stream)
        without synchronising; errors land in status slot ``slot``."""
        import torch

        dev = input.device.index
        ctx = get_context(dev)
        if stream is None:
            stream = torch.cuda.current_stream(dev).cuda_stream
        rc = _capi.lib().fbgemm_b200_spmdm_launch(
            ctx.handle, C.byref(self.cfg), output_size, index_size, data_size, _ptr(input), _ptr(indices),
            _ptr(offsets_or_lengths), _ptr(weights) if self.cfg.has_weight else None, _ptr(out),
            _ptr(compressed_indices_table), slot, stream)
        _capi.check(rc, "fbgemm_b200_spmdm_launch")

    def host_submit(self, lane, output_size, index_size, data_size, input, indices, offsets_or_lengths,
                    weights, out, compressed_indices_table=None) -> None:
        ctx = get_context()
        rc = _capi.lib().fbgemm_b200_spmdm_host_submit(
            ctx.handle, lane, C.byref(self.cfg), output_size, index_size, data_size, _ptr(input), _ptr(indices),
            _ptr(offsets_or_lengths), _ptr(weights) if self.cfg.has_weight else None, _ptr(out),
            _ptr(compressed_indices_table))
        _capi.check(rc, "fbgemm_b200_spmdm_host_submit")

    @staticmethod
    def host_wait(lane) -> bool:
        ctx = get_context()
        return bool(_capi.check(_capi.lib().fbgemm_b200_spmdm_host_wait(ctx.handle, lane), "host_wait"))

    def _check_dtypes(self, indices, offsets):
        for arr, want, what in ((indices, self.cfg.index_bytes, "indices"), (offsets, self.cfg.offset_bytes, "offsets")):
            if arr is None:
                continue
            size = arr.element_size() if _is_tensor(arr) else arr.dtype.itemsize
            if size != want:
                raise TypeError(f"{what} have {size}-byte elements, kernel was generated for {want}")


class MultiTablePlan:
    """Several tables pooled by one call (``fbgemm_b200_multi_plan_*``): what the
    reference's multi-table caller does with a loop of functor calls
    (fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:343-473).

    ``calls`` is a list of ``(kernel, output_size, index_size, data_size, input,
    indices, offsets, weights, out, compressed_indices_table)`` with device
    tensors; ``peer_ptrs`` (optional, one list of ``num_peers`` addresses per
    table) redirects the pooled rows as ``fbgemm_b200_spmdm_launch_sharded``
    does.  The plan keeps the tensors alive and is tied to their addresses."""

    def __init__(self, calls, device: int | None = None, slot: int = 0, peer_ptrs=None, bags_per_peer: int = 0):
        self.ctx = get_context(device)
        self.slot = slot
        self._keep = list(calls)
        n = len(calls)
        arr = (_capi.TableCall * n)()
        self._peer_arrays = []
        num_peers = len(peer_ptrs[0]) if peer_ptrs else 0
        for t, (kern, output_size, index_size, data_size, input, indices, offsets, weights, out, cit) in enumerate(calls):
            c = arr[t]
            c.cfg = kern.cfg
            c.output_size, c.index_size, c.data_size = output_size, index_size, data_size
            c.input, c.indices, c.offsets = _ptr(input), _ptr(indices), _ptr(offsets)
            c.weights = _ptr(weights) if kern.cfg.has_weight else None
            c.out = _ptr(out)
            c.compressed_indices_table = _ptr(cit)
            if peer_ptrs:
                pa = (C.c_void_p * num_peers)(*peer_ptrs[t])
                self._peer_arrays.append(pa)
                c.peer_out = pa
        handle = C.c_void_p()
        rc = _capi.lib().fbgemm_b200_multi_plan_create(self.ctx.handle, arr, n, num_peers, bags_per_peer, slot,
                                                       C.byref(handle))
        _capi.check(rc, "fbgemm_b200_multi_plan_create")
        self._handle = handle

    @property
    def num_launches(self) -> int:
        return int(_capi.lib().fbgemm_b200_multi_plan_num_launches(self._handle))

    def launch(self, stream=None) -> None:
        import torch

        if stream is None:
            stream = torch.cuda.current_stream(self.ctx.device).cuda_stream
        _capi.check(_capi.lib().fbgemm_b200_multi_plan_launch(self._handle, stream), "fbgemm_b200_multi_plan_launch")

    def close(self) -> None:
        if self._handle:
            _capi.lib().fbgemm_b200_multi_plan_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MultiTableHostCall:
    """``fbgemm_b200_multi_host_*``: the tables of one operator call pooled from
    HOST index arrays into a host output buffer, the tables resident in HBM -
    what the reference's multi-table caller is given
    (fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:208-280
    of FBGEMM).

    ``tables`` is a list of ``(kernel, output_size, data_size, device_table,
    out, index_capacity)``; ``out`` is the device address the table's pooled
    rows start at, or with ``peer_ptrs`` (one list of ``num_peers`` addresses
    per table) the rows go to the peers as in
    ``fbgemm_b200_spmdm_launch_sharded``.  ``out_dev`` is the device tensor
    whose bytes travel to the host buffer at the end of a step; ``sync`` an
    optional ``_capi.PeerSync``."""

    def __init__(self, tables, out_dev, device: int | None = None, slot: int = 0, peer_ptrs=None,
                 bags_per_peer: int = 0, sync=None):
        self.ctx = get_context(device)
        self._keep = (list(tables), out_dev, sync)
        n = len(tables)
        arr = (_capi.TableCall * n)()
        caps = (C.c_int64 * n)()
        self._peer_arrays = []
        num_peers = len(peer_ptrs[0]) if peer_ptrs else 0
        self.weighted = False
        for t, (kern, output_size, data_size, table, out, cap) in enumerate(tables):
            c = arr[t]
            c.cfg = kern.cfg
            c.output_size, c.index_size, c.data_size = output_size, 0, data_size
            c.input = _ptr(table)
            c.out = out if isinstance(out, int) or out is None else _ptr(out)
            caps[t] = cap
            self.weighted = self.weighted or bool(kern.cfg.has_weight)
            if peer_ptrs:
                pa = (C.c_void_p * num_peers)(*peer_ptrs[t])
                self._peer_arrays.append(pa)
                c.peer_out = pa
        self.n = n
        self.out_bytes = out_dev.numel() * out_dev.element_size()
        handle = C.c_void_p()
        rc = _capi.lib().fbgemm_b200_multi_host_create(
            self.ctx.handle, arr, n, caps, num_peers, bags_per_peer, out_dev.data_ptr(), self.out_bytes,
            C.byref(sync) if sync is not None else None, slot, C.byref(handle))
        _capi.check(rc, "fbgemm_b200_multi_host_create")
        self._handle = handle
        self._idx = (C.c_void_p * n)()
        self._off = (C.c_void_p * n)()
        self._w = (C.c_void_p * n)()
        self._sizes = (C.c_int64 * n)()

    def submit(self, indices, offsets, weights, out_host) -> None:
        """``indices[t]``, ``offsets[t]``, ``weights[t]`` (or None) are host
        arrays (numpy; pinned memory keeps the copies asynchronous);
        ``out_host`` receives ``out_dev``'s bytes."""
        for t in range(self.n):
            self._idx[t] = indices[t].ctypes.data
            self._off[t] = offsets[t].ctypes.data
            self._w[t] = weights[t].ctypes.data if (weights is not None and weights[t] is not None) else None
            self._sizes[t] = indices[t].shape[0]
        rc = _capi.lib().fbgemm_b200_multi_host_submit(self._handle, self._idx, self._off,
                                                       self._w if self.weighted else None, self._sizes,
                                                       out_host.ctypes.data)
        _capi.check(rc, "fbgemm_b200_multi_host_submit")

    def wait(self):
        """(ok, info[4]) once the rows are in the host buffer."""
        info = (C.c_int32 * 4)()
        rc = _capi.check(_capi.lib().fbgemm_b200_multi_host_wait(self._handle, info), "fbgemm_b200_multi_host_wait")
        return bool(rc), list(info)

    def device_args(self, indices, offsets, weights):
        """The pointer arrays ``step_device`` takes, built once per set of device
        tensors (``indices[t]``, ``offsets[t]``, ``weights[t]`` or None); keep the
        tensors alive as long as the result is used."""
        idx, off, w, sizes = (C.c_void_p * self.n)(), (C.c_void_p * self.n)(), (C.c_void_p * self.n)(), (C.c_int64 * self.n)()
        for t in range(self.n):
            idx[t], off[t] = indices[t].data_ptr(), offsets[t].data_ptr()
            w[t] = weights[t].data_ptr() if (weights is not None and weights[t] is not None) else None
            sizes[t] = indices[t].shape[0]
        return idx, off, (w if self.weighted else None), sizes

    def step_device(self, args, release: bool, stream: int) -> int:
        """One step on device arrays (``args`` from ``device_args``), enqueued
        on ``stream`` (a raw CUDA stream); returns the step number."""
        idx, off, w, sizes = args
        n = _capi.lib().fbgemm_b200_multi_host_step_device(self._handle, idx, off, w, sizes, 1 if release else 0, stream)
        if n <= 0:
            _capi.check(int(n), "fbgemm_b200_multi_host_step_device")
        return int(n)

    def release(self, step: int, stream: int) -> None:
        _capi.check(_capi.lib().fbgemm_b200_multi_host_release(self._handle, step, stream),
                    "fbgemm_b200_multi_host_release")

    def last_step_ms(self):
        """Device time (ms) of the last waited step's (uploads, lookups,
        download); the phases of two handles overlap."""
        ms = (C.c_float * 3)()
        _capi.check(_capi.lib().fbgemm_b200_multi_host_last_step_ms(self._handle, ms),
                    "fbgemm_b200_multi_host_last_step_ms")
        return list(ms)

    def close(self) -> None:
        if self._handle:
            _capi.lib().fbgemm_b200_multi_host_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def status_read(slot: int = 0, device: int | None = None, stream=None):
    """(ok, info[4]) of status slot ``slot`` after waiting for ``stream``."""
    import torch

    ctx = get_context(device)
    if stream is None:
        stream = torch.cuda.current_stream(ctx.device).cuda_stream
    info = (C.c_int32 * 4)()
    rc = _capi.check(_capi.lib().fbgemm_b200_status_read(ctx.handle, slot, stream, info), "status_read")
    return bool(rc), list(info)


def _config(bit_rate, block_size, has_weight, normalize_by_lengths, is_weight_positional, use_offsets,
            output_stride, input_stride, index_dtype, offset_dtype, out_dtype, scale_bias_last=True, no_bag=False,
            is_bf16_out=False) -> SpmdmConfig:
    out_code = _out_code(out_dtype)
    if is_bf16_out and out_code == 1:
        out_code = 2  # a 16-bit OutType holds bf16 when is_bf16_out is set
    return SpmdmConfig(
        scale_bias_first=int(not scale_bias_last),
        no_bag=int(bool(no_bag)),
        bit_rate=bit_rate,
        index_bytes=_np_itemsize(index_dtype),
        offset_bytes=_np_itemsize(offset_dtype),
        out_dtype=out_code,
        block_size=block_size,
        output_stride=output_stride,
        input_stride=input_stride,
        has_weight=int(bool(has_weight)),
        normalize_by_lengths=int(bool(normalize_by_lengths)),
        is_weight_positional=int(bool(is_weight_positional)),
        use_offsets=int(bool(use_offsets)),
    )


def _in_code(in_dtype, is_bf16_in) -> tuple[int, int]:
    """(FBGEMM_B200_IN_* code, element bytes) of the generators' InType:
    uint8 = fused 8-bit rows, float32, float16, or uint16 / bfloat16 storage
    (bf16 when is_bf16_in, as convert_to_float_ref reads it)."""
    try:
        name = np.dtype(in_dtype).name
    except TypeError:
        name = str(in_dtype).rsplit(".", 1)[-1]
    if name == "uint8":
        if is_bf16_in:
            raise ValueError("is_bf16_in belongs to 16-bit tables")
        return 0, 1
    if name == "float32":
        return 1, 4
    if name == "bfloat16" or (name == "uint16" and is_bf16_in):
        return 3, 2
    if name in ("float16", "uint16"):
        return 2, 2
    raise ValueError(f"InType must be uint8, float32, float16 or bfloat16, got {in_dtype}")


def GenerateEmbeddingSpMDM(block_size, has_weight, normalize_by_lengths, prefetch=16,
                           is_weight_positional=False, use_offsets=True, is_bf16_out=False, is_bf16_in=False, *,
                           index_dtype=np.int64, offset_dtype=np.int32, out_dtype=np.float32,
                           in_dtype=np.uint8) -> SpmdmKernel:
    """fbgemm::GenerateEmbeddingSpMDM<InType, Index, Offset, Out>
    (include/fbgemm/FbgemmEmbedding.h:65-84): InType uint8_t = 8-bit rows +
    fp32 scale, bias; float / float16 / uint16_t = tables that are not quantized."""
    return GenerateEmbeddingSpMDMWithStrides(
        block_size, has_weight, normalize_by_lengths, prefetch, is_weight_positional, use_offsets, -1, -1, True,
        False, is_bf16_out, is_bf16_in, index_dtype=index_dtype, offset_dtype=offset_dtype, out_dtype=out_dtype,
        in_dtype=in_dtype)


def GenerateEmbeddingSpMDMWithStrides(block_size, has_weight, normalize_by_lengths, prefetch=16,
                                      is_weight_positional=False, use_offsets=True, output_stride=-1,
                                      input_stride=-1, scale_bias_last=True, no_bag=False, is_bf16_out=False,
                                      is_bf16_in=False, *, index_dtype=np.int64, offset_dtype=np.int32,
                                      out_dtype=np.float32, in_dtype=np.uint8) -> SpmdmKernel:
    """fbgemm::GenerateEmbeddingSpMDMWithStrides<InType, ...>
    (include/fbgemm/FbgemmEmbedding.h:94-117).  ``input_stride`` counts
    elements of InType, as the reference's does."""
    code, ebytes = _in_code(in_dtype, is_bf16_in)
    stride_bytes = input_stride if input_stride == -1 else input_stride * ebytes
    cfg = _config(8, block_size, has_weight, normalize_by_lengths, is_weight_positional, use_offsets, output_stride,
                  stride_bytes, index_dtype, offset_dtype, out_dtype, scale_bias_last, no_bag, is_bf16_out)
    cfg.in_dtype = code
    return SpmdmKernel(cfg, False)


class _Fp8Kernel:
    """The functor of GenerateEmbeddingSpMDMFP8WithStrides: whether the rows are
    weighted is decided by the call (weights null or not), not by the generator."""

    def __init__(self, make):
        self._k = {False: make(False), True: make(True)}
        self.cfg = self._k[False].cfg

    def __call__(self, output_size, index_size, data_size, input, indices, offsets_or_lengths, weights, out):
        return self._k[weights is not None](output_size, index_size, data_size, input, indices, offsets_or_lengths,
                                            weights, out)

    def launch(self, output_size, index_size, data_size, input, indices, offsets_or_lengths, weights, out, **kw):
        return self._k[weights is not None].launch(output_size, index_size, data_size, input, indices,
                                                   offsets_or_lengths, weights, out, **kw)


def GenerateEmbeddingSpMDMFP8WithStrides(block_size, normalize_by_lengths, is_weight_positional=False,
                                         use_offsets=True, output_stride=-1, input_stride=-1, exponent_bits=4,
                                         exponent_bias=7, is_bf16_out=False, *, index_dtype=np.int64,
                                         offset_dtype=np.int32, out_dtype=np.float32) -> _Fp8Kernel:
    """fbgemm::GenerateEmbeddingSpMDMFP8WithStrides (include/fbgemm/FbgemmEmbedding.h:185-203):
    rows of FP8 values, no scale or bias."""
    def make(weighted):
        cfg = _config(8, block_size, weighted, normalize_by_lengths, is_weight_positional, use_offsets, output_stride,
                      input_stride, index_dtype, offset_dtype, out_dtype, True, False, is_bf16_out)
        cfg.in_dtype = 4
        cfg.fp8_exponent_bits, cfg.fp8_exponent_bias = exponent_bits, exponent_bias
        return SpmdmKernel(cfg, False)
    return _Fp8Kernel(make)


def GenerateEmbeddingSpMDMNBit(bit_rate, block_size, has_weight, normalize_by_lengths, prefetch=16,
                               is_weight_positional=False, use_offsets=True, *, index_dtype=np.int64,
                               offset_dtype=np.int32, out_dtype=np.float32) -> SpmdmKernel:
    """fbgemm::GenerateEmbeddingSpMDMNBit (include/fbgemm/FbgemmEmbedding.h:124-140):
    4- or 2-bit rows + fp16 scale, bias."""
    return GenerateEmbeddingSpMDMNBitWithStrides(
        bit_rate, block_size, has_weight, normalize_by_lengths, prefetch, is_weight_positional, use_offsets,
        index_dtype=index_dtype, offset_dtype=offset_dtype, out_dtype=out_dtype)


def GenerateEmbeddingSpMDMNBitWithStrides(input_bit_rate, block_size, has_weight, normalize_by_lengths,
                                          prefetch=16, is_weight_positional=False, use_offsets=True,
                                          output_stride=-1, input_stride=-1, scale_bias_last=True,
                                          is_bf16_out=False, no_bag=False, output_bit_rate=-1, *,
                                          index_dtype=np.int64, offset_dtype=np.int32,
                                          out_dtype=np.float32) -> SpmdmKernel:
    """fbgemm::GenerateEmbeddingSpMDMNBitWithStrides
    (include/fbgemm/FbgemmEmbedding.h:149-174)."""
    if input_bit_rate not in (2, 4):
        raise ValueError("bit_rate must be 2 or 4")  # src/EmbeddingSpMDMNBit.cc:999-1001
    if no_bag:
        # the reference's N-bit no_bag is the int4 -> int4 sequence lookup: a byte copy of the rows
        # (src/RefImplementations.cc:1467-1485)
        if input_bit_rate != 4 or output_bit_rate != 4 or _out_code(out_dtype) != 3:
            raise ValueError("no_bag is only supported for int4 to int4 (uint8 OutType, output_bit_rate = 4)")
    elif output_bit_rate not in (-1, 8 * {0: 4, 1: 2, 2: 2, 3: 1}[_out_code(out_dtype)]) or _out_code(out_dtype) == 3:
        raise ValueError("N-bit output is provided for no_bag only")
    return SpmdmKernel(_config(input_bit_rate, block_size, has_weight, normalize_by_lengths, is_weight_positional,
                               use_offsets, output_stride, input_stride, index_dtype, offset_dtype, out_dtype,
                               scale_bias_last, no_bag, is_bf16_out), False)


def GenerateEmbeddingSpMDMRowWiseSparse(block_size, has_weight, normalize_by_lengths, prefetch=16,
                                        is_weight_positional=False, use_offsets=True, *, index_dtype=np.int64,
                                        offset_dtype=np.int32, in_dtype=np.uint8) -> SpmdmKernel:
    """fbgemm::GenerateEmbeddingSpMDMRowWiseSparse<InType, ...>
    (include/fbgemm/FbgemmEmbedding.h:229-243): pruned table of fused 8-bit
    rows (``in_dtype`` uint8), or of float32 / float16 rows."""
    if np.dtype(in_dtype) not in (np.dtype(np.uint8), np.dtype(np.float32), np.dtype(np.float16)):
        raise ValueError("InType must be uint8, float32 or float16")
    cfg = _config(8, block_size, has_weight, normalize_by_lengths, is_weight_positional, use_offsets,
                  -1, -1, index_dtype, offset_dtype, np.float32)
    cfg.in_dtype = _in_code(in_dtype, False)[0]
    return SpmdmKernel(cfg, True)


def GenerateEmbeddingSpMDMNBitRowWiseSparse(bit_rate, block_size, has_weight, normalize_by_lengths, prefetch=16,
                                            is_weight_positional=False, use_offsets=True, *,
                                            index_dtype=np.int64, offset_dtype=np.int32) -> SpmdmKernel:
    """fbgemm::GenerateEmbeddingSpMDMNBitRowWiseSparse
    (include/fbgemm/FbgemmEmbedding.h:250-262): pruned 4-/2-bit table."""
    if bit_rate not in (2, 4):
        raise ValueError("bit_rate must be 2 or 4")
    return SpmdmKernel(_config(bit_rate, block_size, has_weight, normalize_by_lengths, is_weight_positional,
                               use_offsets, -1, -1, index_dtype, offset_dtype, np.float32), True)


# ---- quantizers (device tensors) ---------------------------------------------

def FloatToFused8BitRowwiseQuantizedSBFloat(x, out=None):
    """fbgemm::FloatOrHalfToFused8BitRowwiseQuantizedSBFloat<float>
    (include/fbgemm/QuantUtils.h:312) on a CUDA fp32 tensor [rows, cols] ->
    uint8 [rows, cols + 8]."""
    import torch

    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous()
    rows, cols = x.shape
    if out is None:
        out = torch.empty((rows, cols + 8), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        _capi.check(_capi.lib().fbgemm_b200_float_to_fused_8bit_rowwise(
            x.data_ptr(), rows, cols, out.data_ptr(), stream), "8-bit quantizer")
    return out


def FloatToFusedNBitRowwiseQuantizedSBHalf(bit_rate, x, out=None):
    """fbgemm::FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf<float>
    (include/fbgemm/QuantUtils.h:277) on a CUDA fp32 tensor [rows, cols] ->
    uint8 [rows, cols / (8/bit_rate) + 4]."""
    import torch

    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous()
    rows, cols = x.shape
    epb = 8 // bit_rate
    if cols % epb:
        raise ValueError("Unsupported number of columns")  # src/QuantUtils.cc:624-627
    if out is None:
        out = torch.empty((rows, cols // epb + 4), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        _capi.check(_capi.lib().fbgemm_b200_float_to_fused_nbit_rowwise(
            bit_rate, x.data_ptr(), rows, cols, out.data_ptr(), stream), "N-bit quantizer")
    return out


def compressed_indices_remap(indices, compressed_indices_mapping, offsets, weights=None):
    """fbgemm::compressed_indices_remap (include/fbgemm/FbgemmEmbedding.h:393-401)
    on CUDA tensors: returns ``(ok, out_indices, out_offsets, out_weights)``
    where ``out_offsets[-1]`` entries of ``out_indices`` / ``out_weights`` are
    valid.  ``ok`` is False when an index lay outside the map."""
    import torch

    assert indices.is_cuda and indices.dtype == offsets.dtype and indices.dtype in (torch.int32, torch.int64)
    assert compressed_indices_mapping.dtype == torch.int32
    ctx = get_context(indices.device.index)
    out_indices = torch.empty_like(indices)
    out_offsets = torch.empty_like(offsets)
    out_weights = torch.empty_like(weights) if weights is not None else None
    rc = _capi.lib().fbgemm_b200_compressed_indices_remap(
        ctx.handle, offsets.numel(), _ptr(indices), indices.element_size(), indices.numel(),
        _ptr(compressed_indices_mapping), compressed_indices_mapping.numel(), _ptr(offsets), _ptr(weights),
        _ptr(out_indices), _ptr(out_offsets), _ptr(out_weights), torch.cuda.current_stream(ctx.device).cuda_stream)
    return bool(_capi.check(rc, "fbgemm_b200_compressed_indices_remap")), out_indices, out_offsets, out_weights

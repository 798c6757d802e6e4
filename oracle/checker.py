"""ctypes access to the CPU checkers.  TEST INFRASTRUCTURE - not the product.

Four libraries, all built by the Makefile in this directory:

* ``liboracle.so``            the plain-C restatement (``embedding_oracle.c``)
* ``_ref/libfbgemm_ref.so``   the reference's own scalar and auto-vectorised
                              sources compiled where they lie (``ref_shim.cc``)
* ``_ref/libfbgemm_jit.so``   the reference's asmjit kernels as bundled in
                              ``libtorch_cpu.so`` (``ref_jit_shim.cc``)
* ``_ref/libfbgemm_tbe_ref.so`` the reference's table-batched CPU operator and
                              pruning lookups, rendered from its template and
                              compiled (``render_tbe_template.py``,
                              ``ref_tbe_shim.cc``)

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py``
may import this module.  All arrays are numpy arrays in host memory.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libfbgemm_ref.so")
JIT_SO = os.path.join(HERE, "_ref", "libfbgemm_jit.so")
TBE_SO = os.path.join(HERE, "_ref", "libfbgemm_tbe_ref.so")

_i64 = C.c_int64
_int = C.c_int
_p = C.c_void_p

_LOOKUP_ARGS = [_i64, _i64, _i64, _i64, _p, _p, _int, _p, _int, _p, _int, _p,
                _int, _int, _int, _i64, _i64]
_SPARSE_ARGS = [_int, _i64, _i64, _i64, _i64, _p, _p, _int, _p, _p, _int, _p,
                _int, _p, _int, _int]


def reference_root():
    """Where a checkout of the reference (FBGEMM) lies: the directory named by
    the environment variable FBGEMM_REFERENCE_ROOT, else a directory called
    ``reference`` beside this repository; None when neither holds the sources."""
    cands = [os.environ.get("FBGEMM_REFERENCE_ROOT"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "src")) and os.path.isdir(os.path.join(c, "include", "fbgemm")):
            return c
    return None


def build(targets=("oracle",), ref_root=None) -> None:
    """Run ``make`` for the named targets (oracle, ref, jit, tbe); ``ref`` and
    ``tbe`` need the reference tree."""
    cmd = ["make", "-C", HERE, "-j8", *targets]
    ref_root = ref_root or reference_root()
    if ref_root:
        cmd.append(f"REF_ROOT={ref_root}")
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "checker arrays must be contiguous"
    return a.ctypes.data


def _load(path):
    if not os.path.exists(path):
        return None
    return C.CDLL(path)


class _Lookups:
    """Shared calling code for the three libraries (same argument order)."""

    def __init__(self, lib, prefix, has_8bit_entry=True):
        self.lib = lib
        self.prefix = prefix
        self.has_8bit_entry = has_8bit_entry

    def _fn(self, name, argtypes, restype=_int):
        f = getattr(self.lib, name)
        f.argtypes = argtypes
        f.restype = restype
        return f

    def spmdm(self, bit_rate, block_size, data_size, table, indices, offsets_or_lengths,
              weights=None, normalize_by_lengths=False, out_dtype=np.float32,
              is_weight_positional=False, use_offsets=True, output_stride=-1,
              input_stride=-1, output_size=None, index_size=None, out=None):
        """Pooled lookup; returns (ok, out).  ``out_dtype`` float32 or float16."""
        indices = np.ascontiguousarray(indices)
        offsets_or_lengths = np.ascontiguousarray(offsets_or_lengths)
        if output_size is None:
            output_size = len(offsets_or_lengths) - (1 if use_offsets else 0)
        if index_size is None:
            index_size = len(indices)
        ostride = block_size if output_stride == -1 else output_stride
        half = np.dtype(out_dtype) == np.float16
        if out is None:
            out = np.zeros(max(output_size, 1) * ostride, dtype=np.float16 if half else np.float32)
        common = (block_size, output_size, index_size, data_size, _ptr(table),
                  _ptr(indices), indices.dtype.itemsize, _ptr(offsets_or_lengths),
                  offsets_or_lengths.dtype.itemsize, _ptr(weights),
                  int(normalize_by_lengths), _ptr(out), int(half),
                  int(is_weight_positional), int(use_offsets), output_stride, input_stride)
        if bit_rate == 8 and self.has_8bit_entry:
            ok = self._fn(self.prefix + "_embedding_spmdm_8bit", _LOOKUP_ARGS)(*common)
        elif self.has_8bit_entry:
            ok = self._fn(self.prefix + "_embedding_spmdm_nbit", [_int] + _LOOKUP_ARGS)(bit_rate, *common)
        else:
            ok = self._fn(self.prefix + "_embedding_spmdm", [_int] + _LOOKUP_ARGS)(bit_rate, *common)
        return bool(ok), out

    def spmdm_ex(self, bit_rate, block_size, data_size, table, indices, offsets_or_lengths=None,
                 weights=None, normalize_by_lengths=False, out_kind="f32",
                 is_weight_positional=False, use_offsets=True, output_stride=-1,
                 input_stride=-1, scale_bias_last=True, no_bag=False, output_size=None,
                 index_size=None):
        """The lookup with every generator option: ``out_kind`` "f32", "f16" or
        "bf16" (16-bit results come back as uint16 bit patterns),
        ``scale_bias_last=False`` for rows with fp16 scale, bias first and -1
        as a pruned index, ``no_bag`` for one output row per index."""
        indices = np.ascontiguousarray(indices)
        if index_size is None:
            index_size = len(indices)
        if no_bag:
            offsets_or_lengths = np.zeros(1, dtype=indices.dtype)
            if output_size is None:
                output_size = index_size
        offsets_or_lengths = np.ascontiguousarray(offsets_or_lengths)
        if output_size is None:
            output_size = len(offsets_or_lengths) - (1 if use_offsets else 0)
        ostride = block_size if output_stride == -1 else output_stride
        kind = {"f32": 0, "f16": 1, "bf16": 2}[out_kind]
        out = np.zeros(max(output_size, 1) * ostride, dtype=np.float32 if kind == 0 else np.uint16)
        f = self._fn(self.prefix + "_embedding_spmdm_ex", [_int] + _LOOKUP_ARGS + [_int, _int])
        ok = f(bit_rate, block_size, output_size, index_size, data_size, _ptr(table),
               _ptr(indices), indices.dtype.itemsize, _ptr(offsets_or_lengths),
               offsets_or_lengths.dtype.itemsize, _ptr(weights), int(normalize_by_lengths),
               _ptr(out), kind, int(is_weight_positional), int(use_offsets), output_stride,
               input_stride, int(scale_bias_last), int(no_bag))
        return bool(ok), out

    def spmdm_plain(self, in_kind, block_size, data_size, table, indices, offsets_or_lengths=None,
                    weights=None, normalize_by_lengths=False, out_kind="f32",
                    is_weight_positional=False, use_offsets=True, output_stride=-1,
                    input_stride=-1, scale_bias_last=True, no_bag=False, exponent_bits=4,
                    exponent_bias=7, output_size=None, index_size=None):
        """Lookup on a table that is not row-wise quantized.  ``in_kind`` "f32",
        "f16", "bf16" (``table`` holds uint16 bit patterns) or "fp8" (uint8);
        ``input_stride`` in elements."""
        indices = np.ascontiguousarray(indices)
        if index_size is None:
            index_size = len(indices)
        if no_bag:
            offsets_or_lengths = np.zeros(1, dtype=indices.dtype)
            if output_size is None:
                output_size = index_size
        offsets_or_lengths = np.ascontiguousarray(offsets_or_lengths)
        if output_size is None:
            output_size = len(offsets_or_lengths) - (1 if use_offsets else 0)
        ostride = block_size if output_stride == -1 else output_stride
        kind = {"f32": 0, "f16": 1, "bf16": 2}[out_kind]
        ik = {"f32": 1, "f16": 2, "bf16": 3, "fp8": 4}[in_kind]
        out = np.zeros(max(output_size, 1) * ostride, dtype=np.float32 if kind == 0 else np.uint16)
        f = self._fn(self.prefix + "_embedding_spmdm_plain", [_int] + _LOOKUP_ARGS + [_int, _int, _int, _int])
        ok = f(ik, block_size, output_size, index_size, data_size, _ptr(table), _ptr(indices),
               indices.dtype.itemsize, _ptr(offsets_or_lengths), offsets_or_lengths.dtype.itemsize,
               _ptr(weights), int(normalize_by_lengths), _ptr(out), kind, int(is_weight_positional),
               int(use_offsets), output_stride, input_stride, int(scale_bias_last), int(no_bag),
               exponent_bits, exponent_bias)
        return bool(ok), out

    def rows_copy(self, bit_rate, block_size, data_size, table, indices, output_stride, input_stride):
        """no_bag with 8-bit output: byte copies of the indexed rows.  Returns
        (ok, out[len(indices), pitch]) with pitch = output_stride (8-bit rows) or
        input_stride (4-bit rows)."""
        indices = np.ascontiguousarray(indices)
        pitch = output_stride if bit_rate == 8 else input_stride
        out = np.zeros((max(len(indices), 1), pitch), dtype=np.uint8)
        if self.prefix == "oracle":
            f = self._fn("oracle_embedding_rows_copy", [_int, _i64, _i64, _p, _p, _int, _p, _i64, _i64])
            ok = f(bit_rate, len(indices), data_size, _ptr(table), _ptr(indices), indices.dtype.itemsize, _ptr(out),
                   output_stride, input_stride)
        else:
            f = self._fn("ref_embedding_rows_copy", [_int, _i64, _i64, _i64, _p, _p, _int, _p, _i64, _i64])
            ok = f(bit_rate, block_size, len(indices), data_size, _ptr(table), _ptr(indices), indices.dtype.itemsize,
                   _ptr(out), output_stride, input_stride)
        return bool(ok), out

    def spmdm_rowwise_sparse(self, bit_rate, block_size, uncompressed_data_size, table,
                             indices, compressed_indices_table, offsets_or_lengths,
                             weights=None, normalize_by_lengths=False,
                             is_weight_positional=False, use_offsets=True,
                             output_size=None, index_size=None):
        indices = np.ascontiguousarray(indices)
        offsets_or_lengths = np.ascontiguousarray(offsets_or_lengths)
        if output_size is None:
            output_size = len(offsets_or_lengths) - (1 if use_offsets else 0)
        if index_size is None:
            index_size = len(indices)
        out = np.zeros(max(output_size, 1) * block_size, dtype=np.float32)
        f = self._fn(self.prefix + "_embedding_spmdm_rowwise_sparse", _SPARSE_ARGS)
        ok = f(bit_rate, block_size, output_size, index_size, uncompressed_data_size,
               _ptr(table), _ptr(indices), indices.dtype.itemsize,
               _ptr(compressed_indices_table), _ptr(offsets_or_lengths),
               offsets_or_lengths.dtype.itemsize, _ptr(weights),
               int(normalize_by_lengths), _ptr(out), int(is_weight_positional),
               int(use_offsets))
        return bool(ok), out


    def spmdm_plain_rowwise_sparse(self, in_kind, block_size, uncompressed_data_size, table, indices,
                                   compressed_indices_table, offsets_or_lengths, weights=None,
                                   normalize_by_lengths=False, is_weight_positional=False, use_offsets=True):
        """Pruned lookup over float ("f32") or fp16 ("f16": uint16 bit patterns;
        "u16": the reference's InType uint16_t, read as fp16 too) rows."""
        kind = {"f32": 1, "f16": 2, "u16": 3}[in_kind]
        if self.prefix == "oracle" and kind == 3:
            kind = 2
        indices = np.ascontiguousarray(indices)
        offsets_or_lengths = np.ascontiguousarray(offsets_or_lengths)
        output_size = len(offsets_or_lengths) - (1 if use_offsets else 0)
        out = np.zeros(max(output_size, 1) * block_size, dtype=np.float32)
        f = self._fn(self.prefix + "_embedding_spmdm_plain_rowwise_sparse", _SPARSE_ARGS)
        ok = f(kind, block_size, output_size, len(indices), uncompressed_data_size, _ptr(table), _ptr(indices),
               indices.dtype.itemsize, _ptr(compressed_indices_table), _ptr(offsets_or_lengths),
               offsets_or_lengths.dtype.itemsize, _ptr(weights), int(normalize_by_lengths), _ptr(out),
               int(is_weight_positional), int(use_offsets))
        return bool(ok), out


class Oracle(_Lookups):
    """The plain-C restatement."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build(("oracle",))
        super().__init__(C.CDLL(ORACLE_SO), "oracle")
        self.lib.oracle_float_to_half_rn.argtypes = [C.c_float]
        self.lib.oracle_float_to_half_rn.restype = C.c_uint16
        self.lib.oracle_half_to_float.argtypes = [C.c_uint16]
        self.lib.oracle_half_to_float.restype = C.c_float

    def quantize_8bit(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        out = np.zeros((rows, cols + 8), dtype=np.uint8)
        f = self._fn("oracle_float_to_fused_8bit_rowwise_sbfloat", [_p, _i64, _int, _p], None)
        f(_ptr(x), rows, cols, _ptr(out))
        return out

    def quantize_nbit(self, bit_rate, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        epb = 8 // bit_rate
        out = np.zeros((rows, (cols + epb - 1) // epb + 4), dtype=np.uint8)
        f = self._fn("oracle_float_to_fused_nbit_rowwise_sbhalf", [_int, _p, _i64, _int, _p], None)
        f(bit_rate, _ptr(x), rows, cols, _ptr(out))
        return out

    def remap(self, indices, mapping, offsets, weights=None):
        indices = np.ascontiguousarray(indices)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        out_i = np.zeros_like(indices)
        out_o = np.zeros_like(offsets)
        out_w = np.zeros(len(indices), dtype=np.float32) if weights is not None else None
        f = self._fn("oracle_compressed_indices_remap", [C.c_int32, _p, _int, _p, _p, _p, _p, _p, _p], None)
        f(len(offsets), _ptr(indices), indices.dtype.itemsize, _ptr(mapping), _ptr(offsets),
          _ptr(weights), _ptr(out_i), _ptr(out_o), _ptr(out_w))
        n = int(out_o[-1])
        return out_i[:n], out_o, (out_w[:n] if out_w is not None else None)

    def pruned_hash(self, key, index_bytes):
        f = self._fn("oracle_pruned_hash", [C.c_uint64, _int], C.c_uint64)
        return int(f(int(key) & (2 ** 64 - 1), index_bytes))

    def pruned_hashmap_insert(self, T, B, indices, dense_indices, offsets, hash_table, hash_table_offsets):
        """Inserts in place into ``hash_table`` ([capacity, 2], int32 or int64, -1 = empty)."""
        indices = np.ascontiguousarray(indices)
        dense_indices = np.ascontiguousarray(dense_indices, dtype=indices.dtype)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        hto = np.ascontiguousarray(hash_table_offsets, dtype=np.int64)
        assert hash_table.flags.c_contiguous and hash_table.shape[1] == 2
        f = self._fn("oracle_pruned_hashmap_insert", [_i64, _i64, _p, _p, _p, _int, _p, _int, _p], _int)
        return bool(f(T, B, _ptr(indices), _ptr(dense_indices), _ptr(offsets), indices.dtype.itemsize,
                      _ptr(hash_table), hash_table.dtype.itemsize, _ptr(hto)))

    def pruned_hashmap_lookup(self, T, B, indices, offsets, hash_table, hash_table_offsets):
        indices = np.ascontiguousarray(indices)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        hto = np.ascontiguousarray(hash_table_offsets, dtype=np.int64)
        out = np.full_like(indices, -7)
        f = self._fn("oracle_pruned_hashmap_lookup", [_i64, _i64, _p, _p, _int, _p, _int, _p, _p], None)
        f(T, B, _ptr(indices), _ptr(offsets), indices.dtype.itemsize, _ptr(hash_table), hash_table.dtype.itemsize,
          _ptr(hto), _ptr(out))
        return out

    def pruned_array_lookup(self, T, B, indices, offsets, remappings, remappings_offsets):
        indices = np.ascontiguousarray(indices)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        ro = np.ascontiguousarray(remappings_offsets, dtype=np.int64)
        remappings = np.ascontiguousarray(remappings)
        out = np.full_like(indices, -7)
        f = self._fn("oracle_pruned_array_lookup", [_i64, _i64, _p, _p, _int, _p, _int, _p, _p], _int)
        ok = bool(f(T, B, _ptr(indices), _ptr(offsets), indices.dtype.itemsize, _ptr(remappings),
                    remappings.dtype.itemsize, _ptr(ro), _ptr(out)))
        return ok, out

    def float_to_half(self, f):
        return int(self.lib.oracle_float_to_half_rn(float(f)))

    def half_to_float(self, h):
        return float(self.lib.oracle_half_to_float(int(h)))


class Reference(_Lookups):
    """The reference's own scalar code; None-like (``available`` False) when the
    library was not built (it needs the reference tree at build time)."""

    def __init__(self):
        lib = _load(REF_SO)
        self.available = lib is not None
        super().__init__(lib, "ref")

    def autovec(self, *args, **kw):
        saved = (self.prefix, self.has_8bit_entry)
        self.prefix, self.has_8bit_entry = "ref_autovec", False
        try:
            return self.spmdm(*args, **kw)
        finally:
            self.prefix, self.has_8bit_entry = saved

    def quantize_8bit(self, x, use_ref=True):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        out = np.zeros((rows, cols + 8), dtype=np.uint8)
        f = self._fn("ref_float_to_fused_8bit_rowwise_sbfloat", [_p, _i64, _int, _p, _int], None)
        f(_ptr(x), rows, cols, _ptr(out), int(use_ref))
        return out

    def quantize_nbit(self, bit_rate, x, use_ref=True):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        epb = 8 // bit_rate
        out = np.zeros((rows, (cols + epb - 1) // epb + 4), dtype=np.uint8)
        f = self._fn("ref_float_to_fused_nbit_rowwise_sbhalf", [_int, _p, _i64, _int, _p, _int], None)
        f(bit_rate, _ptr(x), rows, cols, _ptr(out), int(use_ref))
        return out

    def remap(self, indices, mapping, offsets, weights=None):
        indices = np.ascontiguousarray(indices)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        out_i = np.zeros_like(indices)
        out_o = np.zeros_like(offsets)
        out_w = np.zeros(len(indices), dtype=np.float32) if weights is not None else None
        f = self._fn("ref_compressed_indices_remap", [C.c_int32, _p, _int, _p, _p, _p, _p, _p, _p], None)
        f(len(offsets), _ptr(indices), indices.dtype.itemsize, _ptr(mapping), _ptr(offsets),
          _ptr(weights), _ptr(out_i), _ptr(out_o), _ptr(out_w))
        n = int(out_o[-1])
        return out_i[:n], out_o, (out_w[:n] if out_w is not None else None)

    def float_to_half(self, f):
        self.lib.ref_float_to_half_rn.argtypes = [C.c_float]
        self.lib.ref_float_to_half_rn.restype = C.c_uint16
        return int(self.lib.ref_float_to_half_rn(float(f)))

    def half_to_float(self, h):
        self.lib.ref_half_to_float.argtypes = [C.c_uint16]
        self.lib.ref_half_to_float.restype = C.c_float
        return float(self.lib.ref_half_to_float(int(h)))


class ReferenceJit(_Lookups):
    """The reference's asmjit (AVX2/AVX-512) kernels via libtorch_cpu.so."""

    def __init__(self):
        lib = _load(JIT_SO)
        self.available = lib is not None
        super().__init__(lib, "jit", has_8bit_entry=False)

    def batch_parallel(self, bit_rate, block_size, data_size, table, indices, offsets, weights, normalize_by_lengths,
                       out, threads, compressed_indices_table=None):
        """One whole batch split into ``threads`` contiguous bag ranges, one
        OpenMP thread each (how the reference's callers parallelise the
        kernel).  ``out`` is a preallocated float32/float16 array."""
        f = self._fn("jit_embedding_spmdm_batch_parallel",
                     [_int, _i64, _i64, _i64, _p, _p, _int, _p, _int, _p, _int, _p, _int, _p, _int])
        return bool(f(bit_rate, block_size, len(offsets) - 1, data_size, _ptr(table), _ptr(indices),
                      indices.dtype.itemsize, _ptr(offsets), offsets.dtype.itemsize, _ptr(weights),
                      int(normalize_by_lengths), _ptr(out), int(out.dtype == np.float16),
                      _ptr(compressed_indices_table), threads))


class ReferenceTbe:
    """The reference's table-batched CPU operator and its pruning lookups
    (fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp
    of FBGEMM, compiled from its rendered template)."""

    def __init__(self):
        self.lib = None
        if os.path.exists(TBE_SO):
            import torch  # noqa: F401  (libtorch_cpu.so and libc10.so must be loaded first)

            self.lib = C.CDLL(TBE_SO)
            self.lib.ref_tbe_last_error.restype = C.c_char_p
        self.available = self.lib is not None

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.ref_tbe_last_error().decode())

    def pruned_hashmap_insert(self, T, B, indices, dense_indices, offsets, hash_table, hash_table_offsets):
        indices = np.ascontiguousarray(indices)
        dense_indices = np.ascontiguousarray(dense_indices, dtype=indices.dtype)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        hto = np.ascontiguousarray(hash_table_offsets, dtype=np.int64)
        assert hash_table.flags.c_contiguous and hash_table.shape[1] == 2
        f = self.lib.ref_tbe_pruned_hashmap_insert
        f.argtypes = [C.c_int32, C.c_int32, _p, _p, _p, _int, _p, _int, _i64, _p]
        self._check(f(T, B, _ptr(indices), _ptr(dense_indices), _ptr(offsets), indices.dtype.itemsize,
                      _ptr(hash_table), hash_table.dtype.itemsize, hash_table.shape[0], _ptr(hto)))

    def pruned_hashmap_lookup(self, T, B, indices, offsets, hash_table, hash_table_offsets):
        indices = np.ascontiguousarray(indices)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        hto = np.ascontiguousarray(hash_table_offsets, dtype=np.int64)
        out = np.full_like(indices, -7)
        f = self.lib.ref_tbe_pruned_hashmap_lookup
        f.argtypes = [C.c_int32, C.c_int32, _p, _p, _int, _p, _int, _i64, _p, _p]
        self._check(f(T, B, _ptr(indices), _ptr(offsets), indices.dtype.itemsize, _ptr(hash_table),
                      hash_table.dtype.itemsize, hash_table.shape[0], _ptr(hto), _ptr(out)))
        return out

    def pruned_array_lookup(self, T, B, indices, offsets, remappings, remappings_offsets):
        indices = np.ascontiguousarray(indices)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        ro = np.ascontiguousarray(remappings_offsets, dtype=np.int64)
        remappings = np.ascontiguousarray(remappings)
        out = np.full_like(indices, -7)
        f = self.lib.ref_tbe_pruned_array_lookup
        f.argtypes = [C.c_int32, C.c_int32, _p, _p, _int, _p, _int, _i64, _p, _p]
        self._check(f(T, B, _ptr(indices), _ptr(offsets), indices.dtype.itemsize, _ptr(remappings),
                      remappings.dtype.itemsize, len(remappings), _ptr(ro), _ptr(out)))
        return out

    def forward(self, dev_weights, weights_offsets, weights_tys, D_offsets, dim, indices, offsets, B, pooling_mode,
                row_alignment, indice_weights, output_dtype, scale_bias_last, nobag=False, fp8_exponent_bits=-1,
                fp8_exponent_bias=-1, out_shape=None, out_dtype=None):
        """``int_nbit_split_embedding[_nobag]_codegen_forward_{unweighted,weighted}_cpu``;
        ``dim`` is total_D (pooled) or D (nobag).  Returns the output as a
        numpy array of ``out_dtype`` and ``out_shape``."""
        dev_weights = np.ascontiguousarray(dev_weights, dtype=np.uint8)
        w_off = np.ascontiguousarray(weights_offsets, dtype=np.int64)
        tys = np.ascontiguousarray(weights_tys, dtype=np.uint8)
        dims = np.ascontiguousarray(D_offsets, dtype=np.int32) if D_offsets is not None else None
        indices = np.ascontiguousarray(indices)
        offsets = np.ascontiguousarray(offsets, dtype=indices.dtype)
        w = np.ascontiguousarray(indice_weights, dtype=np.float32) if indice_weights is not None else None
        out = np.zeros(out_shape, dtype=out_dtype)
        f = self.lib.ref_tbe_forward
        f.argtypes = [_int, _p, _i64, _p, _p, C.c_int32, _p, _i64, _p, _p, _int, C.c_int32, _i64, _i64, _p, _i64, _i64,
                      _i64, _int, _p, _i64]
        self._check(f(int(nobag), _ptr(dev_weights), dev_weights.size, _ptr(w_off), _ptr(tys), len(w_off), _ptr(dims),
                      dim, _ptr(indices), _ptr(offsets), indices.dtype.itemsize, B, int(pooling_mode), row_alignment,
                      _ptr(w), int(output_dtype), fp8_exponent_bits, fp8_exponent_bias, int(scale_bias_last),
                      _ptr(out), out.nbytes))
        return out

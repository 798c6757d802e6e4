"""ctypes binding of libfbgemm_b200.so (include/fbgemm_b200/embedding_c_api.h).

The library is loaded from the package directory (it is built in-tree by
``fbgemm_b200.build``).  There is no fallback of any kind: if the library is
missing it is built with nvcc, and if that is impossible the import of the
binding raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

STATUS_SLOTS = 1024
HOST_LANES = 16
USER_SLOTS = STATUS_SLOTS - HOST_LANES - 1
STATUS_PEER_TIMEOUT = 5
IPC_HANDLE_BYTES = 64
NOALLOC_MAX_BAGS = 1 << 20
MAX_PEERS = 8
OUT_F32 = 0
OUT_F16 = 1

EINVAL, ECUDA, ENOMEM, EBUSY = -1, -2, -3, -4


class SpmdmConfig(C.Structure):
    """``fbgemm_b200_spmdm_config``."""

    _fields_ = [
        ("bit_rate", C.c_int32),
        ("index_bytes", C.c_int32),
        ("offset_bytes", C.c_int32),
        ("out_dtype", C.c_int32),
        ("block_size", C.c_int64),
        ("output_stride", C.c_int64),
        ("input_stride", C.c_int64),
        ("has_weight", C.c_int32),
        ("normalize_by_lengths", C.c_int32),
        ("is_weight_positional", C.c_int32),
        ("use_offsets", C.c_int32),
        ("scale_bias_first", C.c_int32),
        ("no_bag", C.c_int32),
        ("absolute_offsets", C.c_int32),
        ("in_dtype", C.c_int32),
        ("fp8_exponent_bits", C.c_int32),
        ("fp8_exponent_bias", C.c_int32),
    ]


class TableCall(C.Structure):
    """``fbgemm_b200_table_call``: the arguments of one table's functor call."""

    _fields_ = [
        ("cfg", SpmdmConfig),
        ("output_size", C.c_int64),
        ("index_size", C.c_int64),
        ("data_size", C.c_int64),
        ("input", C.c_void_p),
        ("indices", C.c_void_p),
        ("offsets", C.c_void_p),
        ("weights", C.c_void_p),
        ("out", C.c_void_p),
        ("compressed_indices_table", C.c_void_p),
        ("peer_out", C.POINTER(C.c_void_p)),
    ]


class PeerSync(C.Structure):
    """``fbgemm_b200_peer_sync``."""

    _fields_ = [
        ("num_peers", C.c_int32),
        ("ready_flags", C.POINTER(C.c_void_p)),
        ("ready_local", C.c_void_p),
        ("ack_flags", C.POINTER(C.c_void_p)),
        ("ack_local", C.c_void_p),
        ("timeout_us", C.c_uint64),
    ]


class Fbgemmb200Error(RuntimeError):
    pass


_p = C.c_void_p
_i64 = C.c_int64
_cfgp = C.POINTER(SpmdmConfig)

# name -> (restype, argtypes); exactly the symbols the header declares.
SIGNATURES = {
    "fbgemm_b200_ctx_create": (C.c_int, [C.c_int, C.POINTER(_p)]),
    "fbgemm_b200_ctx_destroy": (None, [_p]),
    "fbgemm_b200_last_error": (C.c_char_p, []),
    "fbgemm_b200_launch_count": (C.c_uint64, []),
    "fbgemm_b200_set_kernel_choice": (C.c_int, [C.c_int]),
    "fbgemm_b200_spmdm_check_config": (C.c_int, [_cfgp]),
    "fbgemm_b200_spmdm_launch": (C.c_int, [_p, _cfgp, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, C.c_int, _p]),
    "fbgemm_b200_spmdm_launch_sharded": (C.c_int, [_p, _cfgp, _i64, _i64, _i64, _p, _p, _p, _p, C.POINTER(_p),
                                                   C.c_int, _i64, C.c_int, _p]),
    "fbgemm_b200_multi_plan_create": (C.c_int, [_p, C.POINTER(TableCall), C.c_int32, C.c_int32, _i64, C.c_int,
                                                C.POINTER(_p)]),
    "fbgemm_b200_multi_plan_launch": (C.c_int, [_p, _p]),
    "fbgemm_b200_multi_plan_num_launches": (C.c_int, [_p]),
    "fbgemm_b200_multi_plan_destroy": (None, [_p]),
    "fbgemm_b200_status_read": (C.c_int, [_p, C.c_int, _p, C.POINTER(C.c_int32)]),
    "fbgemm_b200_spmdm": (C.c_int, [_p, _cfgp, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _p]),
    "fbgemm_b200_spmdm_lengths_noalloc": (C.c_int, [_cfgp, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p, _p]),
    "fbgemm_b200_compressed_indices_remap": (C.c_int, [_p, C.c_int32, _p, C.c_int32, _i64, _p, _i64, _p, _p, _p, _p,
                                                       _p, _p]),
    "fbgemm_b200_pruned_hashmap_lookup": (C.c_int, [_p, C.c_int32, C.c_int32, _p, _p, C.c_int32, _i64, _p, C.c_int32,
                                                    _p, _p, C.c_int32, _p]),
    "fbgemm_b200_pruned_array_lookup": (C.c_int, [_p, C.c_int32, C.c_int32, _p, _p, C.c_int32, _i64, _p, C.c_int32,
                                                  _p, _p, C.c_int32, _p]),
    "fbgemm_b200_sequence_lookup": (C.c_int, [_p, _p, _p, C.c_int32, C.c_int32, C.c_int32, _p, _p, C.c_int32, _i64, _p,
                                              C.c_int32, _i64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _p]),
    "fbgemm_b200_pruned_hashmap_insert": (C.c_int, [_p, C.c_int32, C.c_int32, _p, _p, _p, C.c_int32, _i64, _p, C.c_int32,
                                                    _p, C.c_int32, _p]),
    "fbgemm_b200_pruned_hashmap_insert_host": (C.c_int, [C.c_int32, C.c_int32, _p, _p, _p, C.c_int32, _p, C.c_int32,
                                                         _p]),
    "fbgemm_b200_table_register": (C.c_int, [_p, _p, C.c_size_t]),
    "fbgemm_b200_table_unregister": (C.c_int, [_p, _p]),
    "fbgemm_b200_table_device_ptr": (_p, [_p, _p]),
    "fbgemm_b200_spmdm_host_submit": (C.c_int, [_p, C.c_int, _cfgp, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p]),
    "fbgemm_b200_spmdm_host_wait": (C.c_int, [_p, C.c_int]),
    "fbgemm_b200_spmdm_host": (C.c_int, [_p, _cfgp, _i64, _i64, _i64, _p, _p, _p, _p, _p, _p]),
    "fbgemm_b200_peer_signal": (C.c_int, [_p, C.POINTER(_p), C.c_int, C.c_uint64, _p]),
    "fbgemm_b200_peer_wait": (C.c_int, [_p, _p, C.c_int, C.c_uint64, C.c_uint64, C.c_int, _p]),
    "fbgemm_b200_peer_buffer_alloc": (C.c_int, [_p, C.c_size_t, C.POINTER(_p), C.c_char_p]),
    "fbgemm_b200_peer_buffer_open": (C.c_int, [_p, C.c_char_p, C.POINTER(_p)]),
    "fbgemm_b200_peer_buffer_close": (C.c_int, [_p, _p]),
    "fbgemm_b200_peer_buffer_free": (C.c_int, [_p, _p]),
    "fbgemm_b200_multi_host_create": (C.c_int, [_p, C.POINTER(TableCall), C.c_int32, C.POINTER(_i64), C.c_int32, _i64,
                                                _p, C.c_size_t, C.POINTER(PeerSync), C.c_int, C.POINTER(_p)]),
    "fbgemm_b200_multi_host_submit": (C.c_int, [_p, C.POINTER(_p), C.POINTER(_p), C.POINTER(_p), C.POINTER(_i64), _p]),
    "fbgemm_b200_multi_host_wait": (C.c_int, [_p, C.POINTER(C.c_int32)]),
    "fbgemm_b200_multi_host_last_step_ms": (C.c_int, [_p, C.POINTER(C.c_float)]),
    "fbgemm_b200_multi_host_step_device": (C.c_int64, [_p, C.POINTER(_p), C.POINTER(_p), C.POINTER(_p), C.POINTER(_i64),
                                           C.c_int, _p]),
    "fbgemm_b200_multi_host_release": (C.c_int, [_p, C.c_int64, _p]),
    "fbgemm_b200_multi_host_destroy": (None, [_p]),
    "fbgemm_b200_float_to_fused_8bit_rowwise": (C.c_int, [_p, _i64, C.c_int32, _p, _p]),
    "fbgemm_b200_float_to_fused_nbit_rowwise": (C.c_int, [C.c_int32, _p, _i64, C.c_int32, _p, _p]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library (built first if the sources changed)."""
    global _lib
    if _lib is None:
        path = _build.LIB_PATH
        if _build.needs_build():
            try:
                path = _build.build()
            except Exception as e:  # no nvcc on this box: use the prebuilt file as is
                if not os.path.exists(path):
                    raise Fbgemmb200Error(
                        f"libfbgemm_b200.so is missing and cannot be built: {e}") from e
        handle = C.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().fbgemm_b200_last_error().decode()


def check(rc: int, what: str) -> int:
    """Raise on a negative return code; pass 0/1 through."""
    if rc < 0:
        raise Fbgemmb200Error(f"{what} failed (code {rc}): {last_error()}")
    return rc

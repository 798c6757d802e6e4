"""What can be checked of the C ABI without a GPU: the library builds and
loads, exports every entry point the header declares, validates generator
arguments, and refuses loudly to run without a CUDA device (there is no CPU
path to fall back to)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from fbgemm_b200 import _capi, build
import fbgemm_b200 as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fbgemm_b200", "embedding_c_api.h")


def declared_entry_points():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"FBGEMM_B200_API\s+[\w\s\*]+?\b(fbgemm_b200_\w+)\s*\(", text)


def test_library_is_built_in_tree_for_sm100a():
    lib = _capi.lib()
    assert lib is not None
    assert os.path.dirname(build.LIB_PATH) == os.path.join(ROOT, "fbgemm_b200")
    assert "arch=compute_100a,code=sm_100a" in " ".join(build.NVCC_FLAGS)


def test_every_declared_entry_point_is_exported_and_bound():
    names = declared_entry_points()
    assert len(names) >= 16
    lib = _capi.lib()
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _capi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_capi.SIGNATURES) == set(names)


def test_config_struct_layout_matches_header():
    # 4 x int32, 3 x int64, 10 x int32 with natural alignment
    assert C.sizeof(_capi.SpmdmConfig) == 16 + 24 + 40
    assert _capi.SpmdmConfig.block_size.offset == 16
    assert _capi.SpmdmConfig.has_weight.offset == 40
    assert _capi.SpmdmConfig.no_bag.offset == 60


def cfg(**kw):
    base = dict(bit_rate=8, index_bytes=8, offset_bytes=8, out_dtype=0, block_size=64, output_stride=-1,
                input_stride=-1, has_weight=0, normalize_by_lengths=0, is_weight_positional=0, use_offsets=1)
    base.update(kw)
    return _capi.SpmdmConfig(**base)


@pytest.mark.parametrize("bad", [
    dict(bit_rate=3), dict(bit_rate=16), dict(index_bytes=2), dict(offset_bytes=16), dict(out_dtype=5),
    dict(block_size=0), dict(block_size=-4), dict(block_size=4096), dict(input_stride=10),
    dict(output_stride=8), dict(bit_rate=4, block_size=64, input_stride=35),
    dict(bit_rate=4, no_bag=1), dict(scale_bias_first=1, input_stride=67), dict(out_dtype=3), dict(bit_rate=2, no_bag=1, out_dtype=3), dict(absolute_offsets=1, use_offsets=0), dict(in_dtype=9), dict(in_dtype=4, fp8_exponent_bits=0),
    dict(in_dtype=2, input_stride=127),
])
def test_check_config_rejects(bad):
    assert _capi.lib().fbgemm_b200_spmdm_check_config(C.byref(cfg(**bad))) == _capi.EINVAL
    assert _capi.last_error() != ""


@pytest.mark.parametrize("good", [
    dict(), dict(bit_rate=4, block_size=64, out_dtype=1), dict(bit_rate=2, block_size=1024),
    dict(block_size=1024), dict(block_size=7, input_stride=20, output_stride=9), dict(bit_rate=4, block_size=1),
    dict(scale_bias_first=1, input_stride=68), dict(out_dtype=2, no_bag=1), dict(bit_rate=2, scale_bias_first=1), dict(out_dtype=3, no_bag=1), dict(bit_rate=4, out_dtype=3, no_bag=1), dict(in_dtype=1, bit_rate=0, block_size=4000),
    dict(in_dtype=4, fp8_exponent_bits=4, fp8_exponent_bias=7), dict(in_dtype=3, no_bag=1, input_stride=256),
])
def test_check_config_accepts(good):
    assert _capi.lib().fbgemm_b200_spmdm_check_config(C.byref(cfg(**good))) == 0


def test_generators_mirror_reference_argument_checks():
    with pytest.raises(ValueError):
        F.GenerateEmbeddingSpMDMNBit(3, 64, False, False)          # bit_rate must be 2 or 4
    with pytest.raises(ValueError):   # the reference's N-bit no_bag is int4 -> int4 only
        F.GenerateEmbeddingSpMDMNBitWithStrides(4, 64, False, False, no_bag=True)
    k = F.GenerateEmbeddingSpMDMNBitWithStrides(4, 64, False, False, no_bag=True, output_bit_rate=4, out_dtype=np.uint8)
    assert (k.cfg.no_bag, k.cfg.out_dtype) == (1, 3)
    with pytest.raises(ValueError):   # is_bf16_in belongs to 16-bit tables
        F.GenerateEmbeddingSpMDM(64, False, False, is_bf16_in=True)
    k = F.GenerateEmbeddingSpMDMWithStrides(64, False, False, input_stride=80, in_dtype=np.float16)
    assert (k.cfg.in_dtype, k.cfg.input_stride) == (2, 160)   # the reference counts the stride in elements
    assert F.GenerateEmbeddingSpMDM(64, False, False, is_bf16_in=True, in_dtype=np.uint16).cfg.in_dtype == 3
    assert F.GenerateEmbeddingSpMDMFP8WithStrides(64, False, exponent_bits=5, exponent_bias=15).cfg.fp8_exponent_bits == 5
    # the table-batched row layout, bf16 output and 8-bit no_bag are carried in the config
    k = F.GenerateEmbeddingSpMDMWithStrides(64, False, False, scale_bias_last=False, no_bag=True, is_bf16_out=True,
                                            out_dtype=np.uint16)
    assert (k.cfg.scale_bias_first, k.cfg.no_bag, k.cfg.out_dtype) == (1, 1, 2)
    k = F.GenerateEmbeddingSpMDMNBitWithStrides(2, 64, False, False, scale_bias_last=False, out_dtype=np.float16)
    assert (k.cfg.scale_bias_first, k.cfg.no_bag, k.cfg.out_dtype) == (1, 0, 1)
    with pytest.raises(Exception):
        F.GenerateEmbeddingSpMDM(64, False, False, out_dtype=np.int8)
    k = F.GenerateEmbeddingSpMDMNBit(4, 64, True, False, index_dtype=np.int32, offset_dtype=np.int32,
                                     out_dtype=np.float16)
    assert (k.cfg.bit_rate, k.cfg.index_bytes, k.cfg.offset_bytes, k.cfg.out_dtype, k.cfg.has_weight) == (4, 4, 4, 1, 1)
    with pytest.raises(TypeError):   # indices of the wrong width are refused before any launch
        k(1, 1, 1, np.zeros(36, np.uint8), np.zeros(1, np.int64), np.zeros(2, np.int32), None, np.zeros(64, np.float16))


def test_no_cpu_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is visible here")
    handle = C.c_void_p()
    rc = _capi.lib().fbgemm_b200_ctx_create(0, C.byref(handle))
    assert rc == _capi.ECUDA and not handle
    assert "CUDA" in _capi.last_error()
    with pytest.raises(_capi.Fbgemmb200Error):
        F.get_context()
    k = F.GenerateEmbeddingSpMDM(8, False, False, index_dtype=np.int64, offset_dtype=np.int64)
    with pytest.raises(_capi.Fbgemmb200Error):   # host arrays, no device: must raise, not compute
        k(1, 1, 1, np.zeros(16, np.uint8), np.zeros(1, np.int64), np.array([0, 1], np.int64), None,
          np.zeros(8, np.float32))


def test_product_does_not_import_the_oracle():
    """Nothing under fbgemm_b200/ may import, load or name the CPU checkers."""
    pkg = os.path.join(ROOT, "fbgemm_b200")
    for dirpath, _, files in os.walk(pkg):
        if "build" in dirpath.split(os.sep)[-1:]:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cc", ".h")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text.lower() or f == "__never__", f"{f} mentions the oracle"

"""The CUDA path against the committed fixtures that were generated from the
reference's own code (tests/golden/make_golden.py), through the C ABI.
Bit-exact: fp32 and fp16 pooled rows, quantizer bytes."""
import os

import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from conftest import bits
from test_oracle import KAT_INPUT, KAT_SBFLOAT_8, KAT_SBHALF

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lookup_golden.npz")


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_lookups_match_reference_fixtures(gpu_ctx):
    g = np.load(GOLDEN)
    for i in range(int(g["n_lookup"])):
        k = f"lookup{i}_"
        bit_rate, batch, rows, dim, weighted, positional, normalize, use_offsets = (int(v) for v in g[k + "meta"])
        want, idx, ol = g[k + "out"], g[k + "indices"], g[k + "ol"]
        kw = dict(index_dtype=idx.dtype.type, offset_dtype=ol.dtype.type, out_dtype=want.dtype.type)
        if bit_rate == 8:
            kern = F.GenerateEmbeddingSpMDM(dim, weighted, normalize, 16, positional, use_offsets, **kw)
        else:
            kern = F.GenerateEmbeddingSpMDMNBit(bit_rate, dim, weighted, normalize, 16, positional, use_offsets, **kw)
        out = torch.zeros(batch * dim, dtype=torch.float16 if want.dtype == np.float16 else torch.float32,
                          device="cuda")
        ok = kern(batch, len(idx), rows, dev(g[k + "table"]), dev(idx), dev(ol),
                  dev(g[k + "weights"]) if weighted else None, out)
        assert ok
        np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(want))


def test_pruned_lookups_match_reference_fixtures(gpu_ctx):
    g = np.load(GOLDEN)
    for i in range(int(g["n_sparse"])):
        k = f"sparse{i}_"
        bit_rate, batch, rows, dim, weighted = (int(v) for v in g[k + "meta"])
        kw = dict(index_dtype=np.int64, offset_dtype=np.int32)
        if bit_rate == 8:
            kern = F.GenerateEmbeddingSpMDMRowWiseSparse(dim, weighted, True, **kw)
        else:
            kern = F.GenerateEmbeddingSpMDMNBitRowWiseSparse(bit_rate, dim, weighted, True, **kw)
        out = torch.zeros(batch * dim, device="cuda")
        ok = kern(batch, len(g[k + "indices"]), rows, dev(g[k + "table"]), dev(g[k + "indices"]),
                  dev(g[k + "offsets"]), dev(g[k + "weights"]) if weighted else None, out, dev(g[k + "mapping"]))
        assert ok
        np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(g[k + "out"]))


def test_quantizers_match_reference_fixtures_and_known_answers(gpu_ctx):
    g = np.load(GOLDEN)
    for i in range(int(g["n_quant"])):
        x = dev(g[f"quant{i}_x"])
        np.testing.assert_array_equal(F.FloatToFused8BitRowwiseQuantizedSBFloat(x).cpu().numpy(), g[f"quant{i}_q8"])
        for b in (4, 2):
            np.testing.assert_array_equal(F.FloatToFusedNBitRowwiseQuantizedSBHalf(b, x).cpu().numpy(),
                                          g[f"quant{i}_q{b}"])
    x = dev(KAT_INPUT)
    np.testing.assert_array_equal(F.FloatToFused8BitRowwiseQuantizedSBFloat(x).cpu().numpy(), KAT_SBFLOAT_8)
    for b, want in KAT_SBHALF.items():
        np.testing.assert_array_equal(F.FloatToFusedNBitRowwiseQuantizedSBHalf(b, x).cpu().numpy(), want)


def test_quantizers_match_oracle_on_random_rows(gpu_ctx, oracle):
    rng = np.random.default_rng(31)
    for rows, cols in ((1000, 128), (777, 64), (300, 256), (50, 8), (41, 36), (20, 4), (3, 1024)):
        x = (rng.standard_normal((rows, cols)) * 10.0 ** rng.integers(-4, 4, (rows, 1))).astype(np.float32)
        x[0] = 0.0
        x[1] = -7.125
        x[2, :] = 1e-30
        d = dev(x)
        np.testing.assert_array_equal(F.FloatToFused8BitRowwiseQuantizedSBFloat(d).cpu().numpy(),
                                      oracle.quantize_8bit(x))
        for b in (4, 2):
            np.testing.assert_array_equal(F.FloatToFusedNBitRowwiseQuantizedSBHalf(b, d).cpu().numpy(),
                                          oracle.quantize_nbit(b, x))
    with pytest.raises(ValueError):   # as the reference: cols must fill whole bytes (src/QuantUtils.cc:624-627)
        F.FloatToFusedNBitRowwiseQuantizedSBHalf(4, dev(np.zeros((2, 7), np.float32)))

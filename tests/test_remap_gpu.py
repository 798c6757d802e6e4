"""compressed_indices_remap on the GPU against the reference-made fixture and
the CPU oracle (bit-exact: integer work), and the identity the reference's own
test relies on (test/EmbeddingSpMDMTest.cc:1040-1193 of FBGEMM): remapping and
then running a plain lookup on the compressed table gives what the row-wise
sparse lookup gives."""
import os

import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from conftest import bits
from helpers import lengths_indices_weights, mapping_table, random_fused_table

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lookup_golden.npz")


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check(oracle, indices, mapping, offsets, weights):
    ri, ro, rw = oracle.remap(indices, mapping, offsets, weights)
    ok, gi, go, gw = F.compressed_indices_remap(dev(indices), dev(mapping), dev(offsets), dev(weights))
    assert ok
    n = int(ro[-1])
    np.testing.assert_array_equal(go.cpu().numpy(), ro)
    np.testing.assert_array_equal(gi.cpu().numpy()[:n], ri[:n])
    if weights is not None:
        np.testing.assert_array_equal(bits(gw.cpu().numpy()[:n]), bits(rw[:n]))
    return n


def test_fixture_made_by_the_reference(gpu_ctx):
    g = np.load(GOLDEN)
    ok, gi, go, gw = F.compressed_indices_remap(dev(g["remap_indices"]), dev(g["remap_mapping"]),
                                                dev(g["remap_offsets"]), dev(g["remap_weights"]))
    assert ok
    n = int(g["remap_out_offsets"][-1])
    np.testing.assert_array_equal(go.cpu().numpy(), g["remap_out_offsets"])
    np.testing.assert_array_equal(gi.cpu().numpy()[:n], g["remap_out_indices"][:n])
    np.testing.assert_array_equal(bits(gw.cpu().numpy()[:n]), bits(g["remap_out_weights"][:n]))


@pytest.mark.parametrize("idt", [np.int32, np.int64])
def test_random_cases_against_the_oracle(gpu_ctx, oracle, idt):
    rng = np.random.default_rng(9100 + np.dtype(idt).itemsize)
    for batch, rows, avg_len, sparsity in ((1, 10, 3, 0.5), (50, 400, 20, 0.7), (700, 20000, 30, 0.5),
                                           (3000, 100000, 40, 0.9), (64, 300, 10, 0.0), (64, 300, 10, 1.0)):
        mapping, _ = mapping_table(rng, rows, sparsity)
        _, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, idt)
        check(oracle, indices, mapping, offsets, weights)
        check(oracle, indices, mapping, offsets, None)
    # offsets that do not start at zero: positions are absolute, the first output offset repeats offsets[0]
    mapping, _ = mapping_table(rng, 500, 0.5)
    _, offsets, indices, weights, n = lengths_indices_weights(rng, 40, 500, 12, idt, idt)
    shift = 37
    indices2 = np.concatenate([rng.integers(0, 500, shift).astype(idt), indices])
    weights2 = np.concatenate([np.zeros(shift, np.float32), weights])
    check(oracle, indices2, mapping, (offsets + shift).astype(idt), weights2)
    # empty input
    check(oracle, np.zeros(0, idt), mapping, np.zeros(5, idt), None)


def test_index_outside_the_map_is_reported(gpu_ctx):
    mapping = torch.arange(10, dtype=torch.int32, device="cuda")
    idx = torch.tensor([1, 2, 10, 3], dtype=torch.int64, device="cuda")
    off = torch.tensor([0, 2, 4], dtype=torch.int64, device="cuda")
    ok, gi, go, _ = F.compressed_indices_remap(idx, mapping, off)
    assert not ok
    assert go.cpu().tolist() == [0, 2, 3] and gi.cpu().tolist()[:3] == [1, 2, 3]


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
def test_remap_then_lookup_equals_rowwise_sparse_lookup(gpu_ctx, oracle, bit_rate):
    rng = np.random.default_rng(9200 + bit_rate)
    batch, rows, dim = 200, 5000, 64
    mapping, dense = mapping_table(rng, rows, 0.6)
    table = random_fused_table(rng, dense, dim, bit_rate)
    _, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 25, np.int64, np.int64)
    d_table, d_map = dev(table), dev(mapping)
    sparse = (F.GenerateEmbeddingSpMDMRowWiseSparse(dim, True, False, index_dtype=np.int64, offset_dtype=np.int64)
              if bit_rate == 8 else
              F.GenerateEmbeddingSpMDMNBitRowWiseSparse(bit_rate, dim, True, False, index_dtype=np.int64,
                                                        offset_dtype=np.int64))
    want = torch.zeros(batch * dim, device="cuda")
    assert sparse(batch, n, rows, d_table, dev(indices), dev(offsets), dev(weights), want, d_map)
    ok, ri, ro, rw = F.compressed_indices_remap(dev(indices), d_map, dev(offsets), dev(weights))
    assert ok
    kept = int(ro[-1])
    plain = (F.GenerateEmbeddingSpMDM(dim, True, False, index_dtype=np.int64, offset_dtype=np.int64) if bit_rate == 8
             else F.GenerateEmbeddingSpMDMNBit(bit_rate, dim, True, False, index_dtype=np.int64, offset_dtype=np.int64))
    got = torch.zeros(batch * dim, device="cuda")
    assert plain(batch, kept, dense, d_table, ri[:kept].contiguous(), ro, rw[:kept].contiguous(), got)
    # sum pooling: skipping a pruned row and never seeing it are the same arithmetic
    np.testing.assert_array_equal(bits(got.cpu().numpy()), bits(want.cpu().numpy()))


def test_more_tiles_than_one_chunk_of_the_tile_scan(gpu_ctx, oracle):
    """Over 256 tiles of 2048 positions the scan of the tile counts carries from chunk to chunk."""
    rng = np.random.default_rng(9200)
    mapping, _ = mapping_table(rng, 300000, 0.5)
    _, offsets, indices, weights, n = lengths_indices_weights(rng, 40000, 300000, 20, np.int64, np.int64)
    assert n > 3 * 256 * 2048 // 2
    check(oracle, indices, mapping, offsets, weights)

"""The benchmark configurations at their full sizes.  The CPU oracle cannot
chew through millions of rows per test, so parity is shown two ways:

* sampled bags: for a random sample of bags, the rows they reference are
  copied back, compacted into a small table with remapped indices, and pooled
  by the oracle - bit-exact agreement with the rows the kernel produced;
* size-independent properties: the same result when the batch is split into
  several calls on slices (offsets then do not start at zero), when bags are
  permuted, when run twice, and - for 8-bit fp32 - when the unweighted lookup
  is replaced by a weighted one with all weights 1.
"""
import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from fbgemm_b200 import workloads as W
from conftest import bits

pytestmark = pytest.mark.gpu


def run(w, kern, b, out=None):
    if out is None:
        out = torch.zeros(b.output_size * w.dim, dtype=w.out_dtype, device="cuda")
    assert kern(b.output_size, b.index_size, w.rows, w.table, b.indices, b.offsets, b.weights, out, w.cit)
    return out.view(b.output_size, w.dim)


def oracle_on_sample(oracle, w, b, bags):
    """Pool the sampled bags on the CPU from a compacted copy of their rows."""
    off = b.offsets.cpu().numpy().astype(np.int64)
    idx_all = b.indices.cpu().numpy()
    wts_all = b.weights.cpu().numpy() if b.weights is not None else None
    pieces, lens = [], []
    for m in bags:
        pieces.append(np.arange(off[m], off[m + 1]))
        lens.append(off[m + 1] - off[m])
    pos = np.concatenate(pieces) if pieces else np.zeros(0, np.int64)
    idx = idx_all[pos].astype(np.int64)
    if w.cit is not None:
        dense = w.cit[torch.from_numpy(idx).cuda()].cpu().numpy().astype(np.int64)
    else:
        dense = idx
    uniq, inv = np.unique(dense[dense >= 0], return_inverse=True)
    small = w.table[torch.from_numpy(uniq).cuda()].cpu().numpy() if len(uniq) else np.zeros((1, w.row_bytes), np.uint8)
    new_off = np.concatenate([[0], np.cumsum(lens)]).astype(off.dtype if b.offsets.dtype == torch.int64 else np.int32)
    wts = wts_all[pos] if wts_all is not None else None
    out_dt = np.float16 if w.out_dtype == torch.float16 else np.float32
    if w.cit is not None:
        # compact the mapping too: uncompressed ids 0..n-1 -> -1 or the small-table row
        mapping = np.full(len(idx), -1, dtype=np.int32)
        mapping[dense >= 0] = inv.astype(np.int32)
        ok, ref = oracle.spmdm_rowwise_sparse(w.bit_rate, w.dim, len(idx), small, np.arange(len(idx), dtype=idx_all.dtype),
                                              mapping, new_off, wts, w.normalize_by_lengths)
    else:
        ok, ref = oracle.spmdm(w.bit_rate, w.dim, len(small), small, inv.astype(idx_all.dtype), new_off, wts,
                               w.normalize_by_lengths, out_dt)
    assert ok
    return ref.reshape(len(bags), w.dim)


@pytest.mark.parametrize("config", [0, 1, 2])
def test_full_size_configuration(gpu_ctx, oracle, config):
    w = W.CONFIGS[config]("cuda")
    kern = w.make_kernel()
    b = w.make_batch(0)
    out = run(w, kern, b)
    rng = np.random.default_rng(config)

    # sampled bags against the oracle
    bags = np.sort(rng.choice(b.output_size, 96, replace=False))
    want = oracle_on_sample(oracle, w, b, bags)
    got = out[torch.from_numpy(bags).cuda()].cpu().numpy()
    np.testing.assert_array_equal(bits(got), bits(want))

    # run twice
    again = run(w, kern, b)
    assert torch.equal(out.view(torch.uint8), again.view(torch.uint8))

    # the batch in three calls on slices of the same arrays (offsets not zero-based)
    cuts = [0, b.output_size // 3, b.output_size // 2, b.output_size]
    parts = torch.zeros_like(out)
    off_host = b.offsets.cpu()
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        i0, i1 = int(off_host[lo]), int(off_host[hi])
        ok = kern(hi - lo, i1 - i0, w.rows, w.table, b.indices[i0:i1], b.offsets[lo:hi + 1],
                  b.weights[i0:i1] if b.weights is not None else None, parts[lo:hi].view(-1), w.cit)
        assert ok
    assert torch.equal(out.view(torch.uint8), parts.view(torch.uint8))

    # bags permuted: outputs permute with them
    perm = torch.randperm(b.output_size, generator=torch.Generator().manual_seed(1))[:2048]
    lens = (off_host[1:] - off_host[:-1])[perm]
    new_off = torch.zeros(len(perm) + 1, dtype=torch.int64)
    new_off[1:] = torch.cumsum(lens.to(torch.int64), 0)
    gather = torch.cat([torch.arange(int(off_host[m]), int(off_host[m + 1])) for m in perm.tolist()]).cuda()
    pb = W.Batch(b.indices[gather], new_off.to(b.offsets.dtype).cuda(),
                 b.weights[gather] if b.weights is not None else None, len(perm), int(gather.numel()), 0)
    pout = run(w, kern, pb)
    assert torch.equal(pout.view(torch.uint8), out[perm.cuda()].contiguous().view(torch.uint8))

    # bad inputs at scale: one index out of range anywhere makes the call false
    bad = b.indices.clone()
    bad[int(rng.integers(0, b.index_size))] = w.rows
    scratch = torch.zeros_like(out).view(-1)
    assert kern(b.output_size, b.index_size, w.rows, w.table, bad, b.offsets, b.weights, scratch, w.cit) is False


def test_unit_weights_equal_unweighted_8bit(gpu_ctx):
    w = W.config0("cuda")
    b = w.make_batch(3)
    plain = run(w, w.make_kernel(), b)
    weighted = F.GenerateEmbeddingSpMDM(w.dim, True, False, index_dtype=np.int64, offset_dtype=np.int64)
    ones = torch.ones(b.index_size, device="cuda")
    out = torch.zeros_like(plain).view(-1)
    assert weighted(b.output_size, b.index_size, w.rows, w.table, b.indices, b.offsets, ones, out)
    assert torch.equal(plain.view(torch.uint8), out.view(-1, w.dim).view(torch.uint8))

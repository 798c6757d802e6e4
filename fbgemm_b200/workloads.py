"""Seeded synthetic inputs for the benchmark configurations.

No dataset is involved: the reference's own embedding benchmarks are synthetic
(bench/EmbeddingSpMDM8BitBenchmark.cc:77-135 of FBGEMM) and its TBE benchmarks
draw Zipf indices, wrap them onto the table with ``(z - 1) % E`` and send them
through a seeded row permutation
(fbgemm_gpu/fbgemm_gpu/tbe/utils/requests.py:319-372,
fbgemm_gpu/src/sparse_ops/sparse_zipf.cu:60-81).  The generators below follow
that recipe with the shapes, sizes and distributions of the five benchmark
configurations.  Everything is produced with torch on the requested device
from an explicit seed, so the GPU arm and the CPU arm of a run see identical
inputs (the CPU arm copies them to the host).
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch

SEED = 12345


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def fused_row_bytes(bit_rate: int, dim: int) -> int:
    """Bytes of one fused row: packed payload + scale,bias (fp32 pair for
    8-bit rows, fp16 pair for 4-/2-bit rows)."""
    epb = 8 // bit_rate
    return (dim + epb - 1) // epb + (8 if bit_rate == 8 else 4)


def zipf(n: int, alpha: float, device, seed: int) -> torch.Tensor:
    """n draws of Zipf(alpha) (alpha > 1) as int64, by the rejection scheme of
    the reference's sampler (sparse_zipf.cu:60-81); draws that do not fit a
    signed 64-bit integer are redrawn."""
    assert alpha > 1.0
    g = _gen(device, seed)
    am1 = alpha - 1.0
    b = 2.0 ** am1
    out = torch.empty(n, dtype=torch.int64, device=device)
    filled = 0
    while filled < n:
        m = int((n - filled) * 1.6) + 1024
        u = 1.0 - torch.rand(m, generator=g, device=device, dtype=torch.float64)
        v = torch.rand(m, generator=g, device=device, dtype=torch.float64)
        x = torch.floor(u.pow(-1.0 / am1))
        t = (1.0 + 1.0 / x).pow(am1)
        ok = (x >= 1.0) & (x < 2.0 ** 62) & (v * x * (t - 1.0) / (b - 1.0) <= t / b)
        acc = x[ok].to(torch.int64)
        k = min(acc.numel(), n - filled)
        out[filled:filled + k] = acc[:k]
        filled += k
    return out


def row_permutation(rows: int, device, seed: int) -> torch.Tensor:
    """The seeded permutation that scatters the hot Zipf ranks over the table."""
    return torch.randperm(rows, generator=_gen(device, seed), device=device)


def zipf_indices(n: int, alpha: float, rows: int, device, seed: int, dtype=torch.int64,
                 perm: torch.Tensor | None = None) -> torch.Tensor:
    """perm[(Zipf(alpha) - 1) mod rows]; `perm` is the table's row permutation
    (one per table, drawn from `seed` if not given)."""
    z = (zipf(n, alpha, device, seed) - 1) % rows
    if perm is None:
        perm = row_permutation(rows, device, seed + 1)
    return perm[z].to(dtype)


def offsets_from_lengths(lengths: torch.Tensor, dtype) -> torch.Tensor:
    off = torch.zeros(lengths.numel() + 1, dtype=torch.int64, device=lengths.device)
    off[1:] = torch.cumsum(lengths.to(torch.int64), 0)
    return off.to(dtype)


def random_rows(rows: int, dim: int, device, seed: int, chunk_rows: int = 1 << 20):
    """The seeded N(0,1) fp32 rows of a table, as (first row, chunk) pieces so
    that the fp32 source never has to exist at once."""
    g = _gen(device, seed)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        yield r0, torch.randn((r1 - r0, dim), generator=g, device=device, dtype=torch.float32)


def random_table(rows: int, dim: int, bit_rate: int, device, seed: int) -> torch.Tensor:
    """``random_rows`` quantized row-wise into fused rows on the device."""
    from .embedding import FloatToFused8BitRowwiseQuantizedSBFloat, FloatToFusedNBitRowwiseQuantizedSBHalf

    out = torch.empty((rows, fused_row_bytes(bit_rate, dim)), dtype=torch.uint8, device=device)
    for r0, x in random_rows(rows, dim, device, seed):
        if bit_rate == 8:
            FloatToFused8BitRowwiseQuantizedSBFloat(x, out[r0:r0 + len(x)])
        else:
            FloatToFusedNBitRowwiseQuantizedSBHalf(bit_rate, x, out[r0:r0 + len(x)])
    return out


@dataclasses.dataclass
class Batch:
    """One functor call's per-call arrays."""
    indices: torch.Tensor
    offsets: torch.Tensor
    weights: torch.Tensor | None
    output_size: int
    index_size: int
    valid_rows: int  # gathered (non-pruned) rows: what the roofline counts


@dataclasses.dataclass
class Workload:
    """A single-table benchmark configuration with its resident table."""
    name: str
    bit_rate: int
    dim: int
    rows: int                 # rows an index may address (uncompressed if pruned)
    table: torch.Tensor       # [table_rows, row_bytes] uint8
    cit: torch.Tensor | None  # compressed_indices_table (pruned configs)
    index_dtype: torch.dtype
    offset_dtype: torch.dtype
    out_dtype: torch.dtype
    has_weight: bool
    normalize_by_lengths: bool
    batch_size: int
    make_batch: "callable"    # (seed) -> Batch

    @property
    def row_bytes(self) -> int:
        return fused_row_bytes(self.bit_rate, self.dim)

    def generator_kwargs(self):
        tnp = {torch.int32: np.int32, torch.int64: np.int64, torch.float32: np.float32, torch.float16: np.float16}
        return dict(index_dtype=tnp[self.index_dtype], offset_dtype=tnp[self.offset_dtype])

    def make_kernel(self):
        """The generator call this configuration names."""
        from . import embedding as E

        tnp = {torch.float32: np.float32, torch.float16: np.float16}
        kw = self.generator_kwargs()
        if self.cit is not None:
            if self.bit_rate == 8:
                return E.GenerateEmbeddingSpMDMRowWiseSparse(self.dim, self.has_weight, self.normalize_by_lengths, **kw)
            return E.GenerateEmbeddingSpMDMNBitRowWiseSparse(
                self.bit_rate, self.dim, self.has_weight, self.normalize_by_lengths, **kw)
        if self.bit_rate == 8:
            return E.GenerateEmbeddingSpMDM(self.dim, self.has_weight, self.normalize_by_lengths,
                                            out_dtype=tnp[self.out_dtype], **kw)
        return E.GenerateEmbeddingSpMDMNBit(self.bit_rate, self.dim, self.has_weight, self.normalize_by_lengths,
                                            out_dtype=tnp[self.out_dtype], **kw)


def _scaled(n: int, scale: float, floor: int = 1) -> int:
    return max(floor, int(round(n * scale)))


def config0(device, scale: float = 1.0, seed: int = SEED, table_maker=random_table) -> Workload:
    """8-bit, 1,000,000 x 128, batch 10,000, pooling 20 fixed, uniform int64
    indices, int64 offsets, unweighted sum, fp32 out."""
    rows, dim, B, L = _scaled(1_000_000, scale, 64), 128, _scaled(10_000, scale, 8), 20
    table = table_maker(rows, dim, 8, device, seed)

    def make_batch(s):
        g = _gen(device, seed + 1000 + s)
        idx = torch.randint(0, rows, (B * L,), generator=g, device=device, dtype=torch.int64)
        off = torch.arange(0, B + 1, device=device, dtype=torch.int64) * L
        return Batch(idx, off, None, B, B * L, B * L)

    return Workload("8bit_1Mx128_B10000_L20_uniform", 8, dim, rows, table, None, torch.int64, torch.int64,
                    torch.float32, False, False, B, make_batch)


def config1(device, scale: float = 1.0, seed: int = SEED, table_maker=random_table) -> Workload:
    """4-bit, 10,000,000 x 64, batch 4,096, bag lengths uniform in [0, 64],
    int32 Zipf(1.05) indices over a seeded permutation, per-sample weights
    U(0,1), weighted sum, fp16 out."""
    rows, dim, B = _scaled(10_000_000, scale, 64), 64, _scaled(4_096, scale, 8)
    table = table_maker(rows, dim, 4, device, seed)
    perm = row_permutation(rows, device, seed + 5)

    def make_batch(s):
        g = _gen(device, seed + 1000 + s)
        lengths = torch.randint(0, 65, (B,), generator=g, device=device, dtype=torch.int64)
        off = offsets_from_lengths(lengths, torch.int32)
        n = int(off[-1])
        idx = zipf_indices(n, 1.05, rows, device, seed + 2000 + s, torch.int32, perm)
        w = torch.rand(n, generator=g, device=device, dtype=torch.float32)
        return Batch(idx, off, w, B, n, n)

    return Workload("4bit_10Mx64_B4096_L0-64_zipf1.05_weighted_fp16", 4, dim, rows, table, None, torch.int32,
                    torch.int32, torch.float16, True, False, B, make_batch)


def config2(device, scale: float = 1.0, seed: int = SEED, table_maker=random_table) -> Workload:
    """2-bit pruned, 20,000,000 logical rows x 128 with a random 50 % mapped to
    -1, batch 8,192, bag lengths Poisson(30), int64 Zipf(1.1) indices, mean
    pooling, fp32 out."""
    rows, dim, B = _scaled(20_000_000, scale, 128), 128, _scaled(8_192, scale, 8)
    g0 = _gen(device, seed + 7)
    keep = torch.rand(rows, generator=g0, device=device) >= 0.5
    cit = torch.full((rows,), -1, dtype=torch.int32, device=device)
    n_dense = int(keep.sum())
    cit[keep] = torch.arange(n_dense, dtype=torch.int32, device=device)
    table = table_maker(max(n_dense, 1), dim, 2, device, seed)
    perm = row_permutation(rows, device, seed + 5)

    def make_batch(s):
        g = _gen(device, seed + 1000 + s)
        lam = torch.full((B,), 30.0, device=device)
        lengths = torch.poisson(lam, generator=g).to(torch.int64)
        off = offsets_from_lengths(lengths, torch.int64)
        n = int(off[-1])
        idx = zipf_indices(n, 1.1, rows, device, seed + 2000 + s, torch.int64, perm)
        valid = int((cit[idx] >= 0).sum())
        return Batch(idx, off, None, B, n, valid)

    return Workload("2bit_pruned_20Mx128_B8192_poisson30_zipf1.1_mean", 2, dim, rows, table, cit, torch.int64,
                    torch.int64, torch.float32, False, True, B, make_batch)


CONFIGS = {0: config0, 1: config1, 2: config2}


def algorithmic_bytes(w: Workload, b: Batch) -> int:
    """Gathered-row bytes of one call: non-pruned rows x fused row size."""
    return b.valid_rows * w.row_bytes


def all_bytes(w: Workload, b: Batch) -> int:
    """The reference benchmarks' fuller byte model: gathered rows plus indices,
    offsets, weights, pruning-map reads and the output rows
    (bench/EmbeddingSpMDM8BitBenchmark.cc:157-160,
    bench/EmbeddingSpMDMNBitRowWiseSparseBenchmark.cc:167-181)."""
    esz = {torch.int32: 4, torch.int64: 8, torch.float32: 4, torch.float16: 2}
    n = algorithmic_bytes(w, b)
    n += b.index_size * esz[w.index_dtype]
    n += (b.output_size + 1) * esz[w.offset_dtype]
    if w.has_weight:
        n += b.index_size * 4
    if w.cit is not None:
        n += b.index_size * 4
    n += b.output_size * w.dim * esz[w.out_dtype]
    return n


# ---- multi-table configurations (table-wise sharded) ----------------------------

@dataclasses.dataclass
class TableSpec:
    rows: int
    dim: int
    bit_rate: int
    seed: int

    @property
    def row_bytes(self) -> int:
        return fused_row_bytes(self.bit_rate, self.dim)


def config3_tables(num_tables: int = 64, scale: float = 1.0, seed: int = SEED) -> list[TableSpec]:
    """64 tables: rows log-uniform in [1M, 20M], D from {64,128,256}, bit width
    from {8,4,2}, i.i.d. from the seed."""
    rng = np.random.default_rng(seed)
    specs = []
    for t in range(num_tables):
        rows = int(round(math.exp(rng.uniform(math.log(1e6), math.log(2e7))) * scale))
        dim = int(rng.choice([64, 128, 256]))
        bits = int(rng.choice([8, 4, 2]))
        specs.append(TableSpec(max(rows, 64), dim, bits, seed + 100 + t))
    return specs


def config4_tables(num_tables: int = 256, scale: float = 1.0, seed: int = SEED) -> list[TableSpec]:
    """256 tables of 40,000,000 x 128, 4-bit (68-byte rows)."""
    return [TableSpec(max(int(40_000_000 * scale), 64), 128, 4, seed + 100 + t) for t in range(num_tables)]

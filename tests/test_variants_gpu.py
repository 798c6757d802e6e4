"""The generators' remaining options on the GPU, bit for bit against the
reference-made fixtures (tests/golden/make_golden_ex.py) and the CPU oracle:
rows with fp16 scale, bias FIRST and -1 as a pruned index (scale_bias_last =
false, the layout of table-batched embeddings), bf16 output, rows padded to an
alignment, and no_bag (one output row per index)."""
import os

import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from conftest import bits
from helpers import REFERENCE_SHAPES, lengths_indices_weights, random_fused_table
from test_oracle import KINDS

pytestmark = pytest.mark.gpu
EX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lookup_ex_golden.npz")
TORCH_KIND = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
NP_KIND = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16}


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def out_bits(t):
    return t.cpu().view(torch.int32 if t.dtype == torch.float32 else torch.int16).numpy().view(
        np.uint32 if t.dtype == torch.float32 else np.uint16)


def generate(bit_rate, dim, weighted, normalize, use_offsets, idt, odt, kind, sb_last, no_bag=False, input_stride=-1):
    kw = dict(index_dtype=idt, offset_dtype=odt, out_dtype=NP_KIND[kind])
    if bit_rate == 8:
        return F.GenerateEmbeddingSpMDMWithStrides(dim, weighted, normalize, 16, False, use_offsets, -1, input_stride,
                                                   sb_last, no_bag, kind == "bf16", **kw)
    return F.GenerateEmbeddingSpMDMNBitWithStrides(bit_rate, dim, weighted, normalize, 16, False, use_offsets, -1,
                                                   input_stride, sb_last, kind == "bf16", **kw)


@pytest.mark.parametrize("kernel", ["default", "staged"])
def test_fixtures_made_by_the_reference(gpu_ctx, kernel):
    from fbgemm_b200 import _capi

    _capi.lib().fbgemm_b200_set_kernel_choice(1 if kernel == "staged" else 0)
    try:
        _fixtures_made_by_the_reference()
    finally:
        _capi.lib().fbgemm_b200_set_kernel_choice(0)


def _fixtures_made_by_the_reference():
    ex = np.load(EX)
    for i in range(int(ex["n_ex"])):
        k = f"ex{i}_"
        bit_rate, count, rows, dim, weighted, normalize, sb_last, no_bag, kind = (int(v) for v in ex[k + "meta"])
        kind = KINDS[kind]
        table, idx, off = ex[k + "table"], ex[k + "indices"], ex[k + "offsets"]
        kern = generate(bit_rate, dim, weighted, normalize, True, idx.dtype.type, off.dtype.type, kind, bool(sb_last),
                        bool(no_bag), table.shape[1])
        out = torch.zeros(count * dim, dtype=TORCH_KIND[kind], device="cuda")
        ok = kern(count, len(idx), rows, dev(table), dev(idx), None if no_bag else dev(off),
                  dev(ex[k + "weights"]) if weighted else None, out)
        assert ok, i
        np.testing.assert_array_equal(out_bits(out), bits(ex[k + "out"]), err_msg=f"case {i}")


@pytest.mark.parametrize("bit_rate", [8, 4, 2])
@pytest.mark.parametrize("sb_last", [False, True])
def test_reference_shapes_with_every_output_kind(gpu_ctx, oracle, bit_rate, sb_last):
    rng = np.random.default_rng(5000 + bit_rate + 10 * sb_last)
    for shape_i, (batch, rows, dim, avg_len) in enumerate(REFERENCE_SHAPES):
        idt, odt = ((np.int32, np.int64), (np.int64, np.int32))[shape_i % 2]
        kind = KINDS[shape_i % 3]
        weighted, normalize, use_offsets = shape_i % 2 == 0, shape_i % 3 == 1, shape_i % 4 != 3
        # rows padded to 16 bytes, as table-batched embeddings store them, every other shape
        data_bytes = (dim * bit_rate + 7) // 8
        natural = data_bytes + (8 if bit_rate == 8 and sb_last else 4)
        stride = (natural + 15) // 16 * 16 if shape_i % 2 else natural
        table = random_fused_table(rng, rows, dim, bit_rate, stride, not sb_last)
        for corner in (None, "oob"):
            lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, avg_len, idt, odt, corner)
            if corner is None:
                indices[rng.integers(0, n, max(1, n // 5))] = -1
            ol = offsets if use_offsets else lengths
            ok_ref, ref = oracle.spmdm_ex(bit_rate, dim, rows, table, indices, ol, weights if weighted else None,
                                          normalize, kind, False, use_offsets, -1, stride, sb_last, False,
                                          output_size=batch, index_size=n)
            kern = generate(bit_rate, dim, weighted, normalize, use_offsets, idt, odt, kind, sb_last, False, stride)
            out = torch.ones(batch * dim + 6, dtype=TORCH_KIND[kind], device="cuda")
            ok = kern(batch, n, rows, dev(table), dev(indices), dev(ol), dev(weights) if weighted else None, out)
            # -1 is a pruned row only when scale, bias come first; otherwise it is an index out of range
            assert ok == ok_ref == (corner is None and not sb_last)
            got = out_bits(out)
            assert (out[batch * dim:].float().cpu().numpy() == 1).all(), "wrote past the output"
            if ok:
                np.testing.assert_array_equal(got[:batch * dim], bits(ref[:batch * dim]), err_msg=str(shape_i))


@pytest.mark.parametrize("sb_last", [False, True])
def test_no_bag(gpu_ctx, oracle, sb_last):
    rng = np.random.default_rng(5100 + sb_last)
    for (rows, dim, count), kind, weighted, idt in zip([(300, 128, 1000), (90, 40, 77), (50, 7, 33), (400, 256, 129)],
                                                       ["f32", "f16", "bf16", "f16"], [True, False, True, True],
                                                       [np.int64, np.int32, np.int64, np.int32]):
        table = random_fused_table(rng, rows, dim, 8, None, not sb_last)
        indices = rng.integers(0, rows, count).astype(idt)
        weights = rng.standard_normal(count).astype(np.float32)
        ok_ref, ref = oracle.spmdm_ex(8, dim, rows, table, indices, None, weights if weighted else None, True, kind,
                                      False, True, -1, -1, sb_last, True)
        kern = generate(8, dim, weighted, True, True, idt, idt, kind, sb_last, True)
        out = torch.zeros(count * dim, dtype=TORCH_KIND[kind], device="cuda")
        ok = kern(count, count, rows, dev(table), dev(indices), None, dev(weights) if weighted else None, out)
        assert ok and ok_ref
        np.testing.assert_array_equal(out_bits(out), bits(ref))
        indices[count // 2] = -1  # no_bag has no pruned rows: -1 is out of range in both layouts
        assert not oracle.spmdm_ex(8, dim, rows, table, indices, None, None, False, kind, False, True, -1, -1, sb_last,
                                   True)[0]
        kern = generate(8, dim, False, False, True, idt, idt, kind, sb_last, True)
        assert not kern(count, count, rows, dev(table), dev(indices), None, None, out)


def test_no_bag_with_8bit_output_copies_rows(gpu_ctx, oracle):
    """The reference's sequence lookups with 8-bit output are byte copies of the
    indexed rows (src/RefImplementations.cc:1235-1254, :1467-1485)."""
    rng = np.random.default_rng(5200)
    for bit_rate, dim, ostride, istride, idt in ((8, 64, 72, 72, np.int64), (8, 64, 68, 80, np.int32), (8, 40, 64, 48, np.int64),
                                                 (8, 37, 45, 45, np.int32), (4, 64, 36, 36, np.int64), (4, 128, 68, 80, np.int32)):
        rows, count = 90, 300
        table = random_fused_table(rng, rows, dim, bit_rate, istride)
        indices = rng.integers(0, rows, count).astype(idt)
        ok_ref, ref = oracle.rows_copy(bit_rate, dim, rows, table, indices, ostride, istride)
        if bit_rate == 8:
            kern = F.GenerateEmbeddingSpMDMWithStrides(dim, False, False, 16, False, True, ostride, istride, True, True,
                                                       index_dtype=idt, offset_dtype=idt, out_dtype=np.uint8)
        else:
            kern = F.GenerateEmbeddingSpMDMNBitWithStrides(4, dim, False, False, 16, False, True, ostride, istride, True,
                                                           False, True, 4, index_dtype=idt, offset_dtype=idt,
                                                           out_dtype=np.uint8)
        pitch = ref.shape[1]
        out = torch.zeros(count * pitch + 5, dtype=torch.uint8, device="cuda")
        assert kern(count, count, rows, dev(table), dev(indices), None, None, out) and ok_ref
        got = out.cpu().numpy()
        width = min(ostride, istride) if bit_rate == 8 else istride
        np.testing.assert_array_equal(got[:count * pitch].reshape(count, pitch)[:, :width], ref[:, :width])
        assert (got[count * pitch:] == 0).all()
        indices[7] = rows
        assert not kern(count, count, rows, dev(table), dev(indices), None, None, out)

"""Table-wise sharding on GPUs: the peer-routing of the sharded launch on one
GPU (two "peers" that are both local buffers), and the real thing on two GPUs
when the box has them (p2p stores over NVLink and the NCCL baseline, both
against the oracle)."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fbgemm_b200 as F
from fbgemm_b200 import _capi
from conftest import bits
from helpers import lengths_indices_weights, random_fused_table

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("bit_rate,out_dt", [(8, np.float32), (4, np.float16), (2, np.float16)])
def test_sharded_launch_routes_bags_to_peers(gpu_ctx, oracle, bit_rate, out_dt):
    """Bags [0, 40) go to 'peer' 0, [40, 80) to peer 1, [80, 100) to peer 2, each
    at its own column offset of a wider row, as the batch-wise layout wants."""
    rng = np.random.default_rng(bit_rate)
    rows, dim, batch, per_peer, total_dim, col = 700, 64, 100, 40, 200, 72
    table = random_fused_table(rng, rows, dim, bit_rate)
    lengths, offsets, indices, weights, n = lengths_indices_weights(rng, batch, rows, 12, np.int32, np.int32)
    ok_ref, ref = oracle.spmdm(bit_rate, dim, rows, table, indices, offsets, weights, False, out_dt)
    ref = ref.reshape(batch, dim)
    tdt = torch.float16 if out_dt == np.float16 else torch.float32
    bufs = [torch.full((per_peer, total_dim), 7, dtype=tdt, device="cuda") for _ in range(3)]
    esize = 2 if out_dt == np.float16 else 4
    ptrs = (C.c_void_p * 3)(*[b.data_ptr() + col * esize for b in bufs])
    kw = dict(index_dtype=np.int32, offset_dtype=np.int32, out_dtype=out_dt, output_stride=total_dim)
    kern = (F.GenerateEmbeddingSpMDMWithStrides(dim, True, False, **kw) if bit_rate == 8 else
            F.GenerateEmbeddingSpMDMNBitWithStrides(bit_rate, dim, True, False, **kw))
    d = [torch.from_numpy(a).cuda() for a in (table, indices, offsets, weights)]
    rc = _capi.lib().fbgemm_b200_spmdm_launch_sharded(
        gpu_ctx.handle, C.byref(kern.cfg), batch, n, rows, d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(),
        d[3].data_ptr(), ptrs, 3, per_peer, 9, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _capi.last_error()
    ok, _ = F.status_read(9)
    assert ok and ok_ref
    for peer, buf in enumerate(bufs):
        got = buf.cpu().numpy()
        lo, hi = peer * per_peer, min(batch, (peer + 1) * per_peer)
        np.testing.assert_array_equal(bits(got[:hi - lo, col:col + dim]), bits(ref[lo:hi]))
        assert (got[:, :col] == 7).all() and (got[:, col + dim:] == 7).all()   # other columns untouched
        assert (got[hi - lo:] == 7).all()                                        # rows past the batch untouched


def test_two_gpu_sharded_lookup_matches_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.join(ROOT, "tests", "sharded_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "SHARDED_OK" in res.stdout

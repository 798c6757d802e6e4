"""fbgemm_b200: FBGEMM's fused row-wise quantized embedding-bag path
(8-, 4- and 2-bit dequantize-gather-pool) as hand-written sm_100a CUDA
kernels behind the reference's kernel-generator API.

Layers, bottom up:

* ``csrc/``        CUDA kernels, the C ABI and the C++ generator templates,
                   built in-tree into ``libfbgemm_b200.so`` (``build.py``)
* ``_capi.py``     ctypes binding of the C ABI
* ``embedding.py`` the reference's generator API in Python (host mirror)
* ``tbe.py``       the table-batched operator above the generators (pooled and
                   sequence form, the pruning lookups that run before it)
* ``workloads.py`` seeded synthetic inputs of the benchmark configurations
* ``sharding.py``  table-wise sharding over the GPUs of one box

Importing the package does not need a GPU; creating a context does, and fails
loudly without one.  There is no CPU path.
"""
from .embedding import (  # noqa: F401
    Context,
    FloatToFused8BitRowwiseQuantizedSBFloat,
    FloatToFusedNBitRowwiseQuantizedSBHalf,
    GenerateEmbeddingSpMDM,
    GenerateEmbeddingSpMDMFP8WithStrides,
    GenerateEmbeddingSpMDMNBit,
    GenerateEmbeddingSpMDMNBitRowWiseSparse,
    GenerateEmbeddingSpMDMNBitWithStrides,
    GenerateEmbeddingSpMDMRowWiseSparse,
    GenerateEmbeddingSpMDMWithStrides,
    MultiTableHostCall,
    MultiTablePlan,
    SpmdmKernel,
    compressed_indices_remap,
    get_context,
    launch_count,
    status_read,
)

__version__ = "0.1.0"

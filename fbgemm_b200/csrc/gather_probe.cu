// A measuring stick, not part of the lookup: how fast can this GPU fetch
// random fixed-size rows at all?  The probe reads the rows the lookup would
// read (same table, same pitch, same indices), with the same lane layout and
// as many rows in flight, but does no arithmetic beyond an XOR that keeps the
// loads alive.  Its rate is the practical ceiling for a gather of rows of this
// size: DRAM serves 32-byte sectors out of 64-byte atoms, so unaligned 36- or
// 136-byte rows cannot approach the bandwidth a streaming copy reaches.
#include "internal.h"

namespace fbgemm_b200 {

namespace {

template <int VEC, int LPB, int U>
__global__ void __launch_bounds__(128)
row_gather_probe(const uint8_t* __restrict__ table, uint32_t stride, int chunks, const int32_t* __restrict__ idx,
                 int64_t n, int rows_per_group, unsigned* sink) {
  const int gl = (threadIdx.x & 31) % LPB;
  const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPB;
  const int64_t r0 = group * rows_per_group;
  if (r0 >= n) {
    return;
  }
  const int rows = (int)min((int64_t)rows_per_group, n - r0);
  unsigned acc = 0;
  for (int r = 0; r + U <= rows; r += U) {
    uint32_t v[U][4 * (VEC / 4)];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint8_t* p = table + (uint64_t)(uint32_t)__ldg(idx + r0 + r + u) * stride + gl * VEC;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (gl + c * LPB < chunks) {
          if constexpr (VEC == 8) {
            const uint2 t = __ldg(reinterpret_cast<const uint2*>(p + c * LPB * VEC));
            v[u][2 * c] = t.x;
            v[u][2 * c + 1] = t.y;
          } else {
            v[u][c] = __ldg(reinterpret_cast<const uint32_t*>(p + c * LPB * VEC));
          }
        } else {
#pragma unroll
          for (int k = 0; k < VEC / 4; ++k) {
            v[u][(VEC / 4) * c + k] = 0;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int c = 0; c < 4 * (VEC / 4); ++c) {
        acc ^= v[u][c];
      }
    }
  }
  if (acc == 0x9e3779b9u) {
    *sink = acc;  // practically never; keeps the loads from being optimised away
  }
}

}  // namespace

}  // namespace fbgemm_b200

using namespace fbgemm_b200;

extern "C" int fbgemm_b200_probe_row_gather(
    const void* table,
    int64_t stride,
    int32_t row_bytes,
    const int32_t* indices,
    int64_t n,
    int32_t rows_per_group,
    void* sink,
    void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const uintptr_t base = reinterpret_cast<uintptr_t>(table);
  if (!table || !indices || !sink || n <= 0 || rows_per_group <= 0 || row_bytes <= 0 || stride > 0xffffffffLL ||
      base % 4 || stride % 4 || row_bytes % 4) {
    set_error("probe: rows must be 4-byte aligned and sized");
    return FBGEMM_B200_EINVAL;
  }
  const bool v8 = base % 8 == 0 && stride % 8 == 0 && row_bytes % 8 == 0;
  const int vec = v8 ? 8 : 4;
  const int chunks = row_bytes / vec;
  int lpb = 4;
  while (lpb < 32 && lpb * 4 < chunks) {
    lpb *= 2;
  }
  if (lpb * 4 < chunks) {
    set_error("probe: row wider than 32 lanes x 4 chunks");
    return FBGEMM_B200_EINVAL;
  }
  const int64_t groups = (n + rows_per_group - 1) / rows_per_group;
  const int64_t blocks = (groups * lpb + 127) / 128;
  unsigned* s = static_cast<unsigned*>(sink);
  const uint8_t* t = static_cast<const uint8_t*>(table);
#define PROBE(V, L) \
  row_gather_probe<V, L, 4><<<(unsigned)blocks, 128, 0, stream>>>(t, (uint32_t)stride, chunks, indices, n, rows_per_group, s)
  if (v8) {
    if (lpb == 4) PROBE(8, 4); else if (lpb == 8) PROBE(8, 8); else if (lpb == 16) PROBE(8, 16); else PROBE(8, 32);
  } else {
    if (lpb == 4) PROBE(4, 4); else if (lpb == 8) PROBE(4, 8); else if (lpb == 16) PROBE(4, 16); else PROBE(4, 32);
  }
#undef PROBE
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : fail_cuda(e, "probe launch");
}

// Row-wise quantizers that build the fused rows the lookups read: the step
// before the hot path.  One warp per row: min/max by shuffles, then every lane
// quantizes and packs whole output bytes.  The arithmetic follows the scalar
// reference so that the produced bytes are identical:
//   8-bit + fp32 scale,bias  src/QuantUtils.cc:677-718
//   N-bit + fp16 scale,bias  src/QuantUtils.cc:534-611
// (fp32 subtract, fp32 multiply by the inverse scale, round half to even).
#include <cuda_fp16.h>

#include "internal.h"

namespace fbgemm_b200 {

namespace {

constexpr int kQuantThreads = 256;

__device__ __forceinline__ void warp_min_max(const float* row, int cols, int lane, float* mn, float* mx) {
  float lo = __ldg(row), hi = lo;  // every lane seeds with element 0
  for (int c = lane; c < cols; c += 32) {
    const float v = __ldg(row + c);
    lo = fminf(lo, v);
    hi = fmaxf(hi, v);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, d));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, d));
  }
  *mn = lo;
  *mx = hi;
}

// Rows are only byte-aligned in general: write a 32-bit word byte by byte.
__device__ __forceinline__ void store_u32_bytes(uint8_t* dst, uint32_t v) {
  dst[0] = (uint8_t)(v & 0xffu);
  dst[1] = (uint8_t)((v >> 8) & 0xffu);
  dst[2] = (uint8_t)((v >> 16) & 0xffu);
  dst[3] = (uint8_t)(v >> 24);
}

__global__ void __launch_bounds__(kQuantThreads)
quantize_8bit_kernel(const float* __restrict__ in, int64_t rows, int cols, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) {
    return;
  }
  const float* x = in + row * cols;
  uint8_t* o = out + row * ((int64_t)cols + 8);
  float mn, mx;
  warp_min_max(x, cols, lane, &mn, &mx);
  const float range = __fsub_rn(mx, mn);
  if (lane == 0) {
    store_u32_bytes(o + cols, __float_as_uint(__fdiv_rn(range, 255.0f)));
    store_u32_bytes(o + cols + 4, __float_as_uint(mn));
  }
  const float inv = __fdiv_rn(255.0f, __fadd_rn(range, 1e-8f));
  for (int c = lane; c < cols; c += 32) {
    o[c] = (uint8_t)__float2int_rn(__fmul_rn(__fsub_rn(__ldg(x + c), mn), inv));
  }
}

template <int BITS>
__global__ void __launch_bounds__(kQuantThreads)
quantize_nbit_kernel(const float* __restrict__ in, int64_t rows, int cols, uint8_t* __restrict__ out) {
  constexpr int EPB = 8 / BITS;
  constexpr int QMAX = (1 << BITS) - 1;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) {
    return;
  }
  const int data_bytes = cols / EPB;
  const float* x = in + row * cols;
  uint8_t* o = out + row * ((int64_t)data_bytes + 4);
  float mn, mx;
  warp_min_max(x, cols, lane, &mn, &mx);
  // the bias is stored as fp16: round the minimum first
  const __half mn_h = __float2half_rn(mn);
  mn = __half2float(mn_h);
  const float range = __fsub_rn(mx, mn);
  // The scale is stored as fp16 too; quantize with the value a reader will see.
  __half scale_h = __float2half_rn(range == 0.f ? 1.0f : __fdiv_rn(range, (float)QMAX));
  float scale = __half2float(scale_h);
  if (scale == 0.f) {
    scale = 1.0f;
    scale_h = __ushort_as_half((unsigned short)0x3C00);
  }
  float inv = __fdiv_rn(1.0f, scale);
  if (isinf(inv)) {
    inv = 1.0f;
    scale_h = __ushort_as_half((unsigned short)0x3C00);
  }
  if (lane == 0) {
    const uint32_t scale_bits = __half_as_ushort(scale_h);
    const uint32_t bias_bits = __half_as_ushort(mn_h);
    store_u32_bytes(o + data_bytes, scale_bits | (bias_bits << 16));
  }
  for (int b = lane; b < data_bytes; b += 32) {
    unsigned packed = 0;
#pragma unroll
    for (int e = 0; e < EPB; ++e) {
      int q = __float2int_rn(__fmul_rn(__fsub_rn(__ldg(x + b * EPB + e), mn), inv));
      q = max(0, min(q, QMAX));
      packed |= (unsigned)q << (e * BITS);
    }
    o[b] = (uint8_t)packed;
  }
}

}  // namespace

cudaError_t launch_quantize_8bit(const float* in, int64_t rows, int cols, uint8_t* out, cudaStream_t s) {
  const int64_t blocks = (rows + kQuantThreads / 32 - 1) / (kQuantThreads / 32);
  if (blocks <= 0 || blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  quantize_8bit_kernel<<<(unsigned)blocks, kQuantThreads, 0, s>>>(in, rows, cols, out);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t launch_quantize_nbit(int bit_rate, const float* in, int64_t rows, int cols, uint8_t* out, cudaStream_t s) {
  const int64_t blocks = (rows + kQuantThreads / 32 - 1) / (kQuantThreads / 32);
  if (blocks <= 0 || blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  if (bit_rate == 8) {
    quantize_nbit_kernel<8><<<(unsigned)blocks, kQuantThreads, 0, s>>>(in, rows, cols, out);
  } else if (bit_rate == 4) {
    quantize_nbit_kernel<4><<<(unsigned)blocks, kQuantThreads, 0, s>>>(in, rows, cols, out);
  } else if (bit_rate == 2) {
    quantize_nbit_kernel<2><<<(unsigned)blocks, kQuantThreads, 0, s>>>(in, rows, cols, out);
  } else {
    return cudaErrorInvalidValue;
  }
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

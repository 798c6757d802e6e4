// Pooled lookup on tables that are NOT row-wise quantized: fp32, fp16, bf16 and
// FP8 rows - the other input types of the reference's generators
// (GenerateEmbeddingSpMDM<float | float16 | uint16_t>, include/fbgemm/FbgemmEmbedding.h:65-117;
// GenerateEmbeddingSpMDMFP8WithStrides, :185-203).  Semantics, from the scalar
// reference (src/RefImplementations.cc:1347-1424 and :1543-1615): rows in index
// order, ONE rounding per row and column,
//     buf[j] = fma(w, float(row[j]), buf[j]),
// then the same normalisation and output conversion as the quantized path.
// FP8 -> fp32 is Float8ToFloat_ref (:184-215): the seven low bits shifted into
// fp32's exponent/mantissa position, times 2^(127 - bias), sign OR-ed in.
//
// These rows carry 1, 2 or 4 bytes per column instead of a quarter to one, so
// the lookup is a plain bandwidth-bound gather and the layout is simple: one
// warp per bag, lane l owning 32-bit words l, l+32, ... of a 1 KB tile of the
// row (consecutive lanes read consecutive words), four rows in flight.  Rows
// wider than a tile are covered by blockIdx.y.  Tables whose address, pitch or
// row width is not a multiple of 4 bytes take the element-wise instantiation.
#include <cuda_fp16.h>

#include "internal.h"

namespace fbgemm_b200 {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kUnitsPerLane = 8;                 // 32-bit words (or elements) per lane and tile
constexpr int kTileUnits = 32 * kUnitsPerLane;
constexpr int kRows = 4;                         // rows of a bag in flight

__device__ __forceinline__ int64_t load_int(const void* p, int64_t i, bool is64) {
  return is64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(p) + i)
              : (int64_t)__ldg(reinterpret_cast<const int*>(p) + i);
}

__device__ __noinline__ void report(int32_t* st, int code, int64_t bag, int64_t pos, int64_t val) {
  if (atomicCAS(st, 0, code) == 0) {
    st[1] = (int32_t)bag;
    st[2] = (int32_t)pos;
    st[3] = (int32_t)val;
  }
}

__device__ __forceinline__ uint16_t to_16bit(float v, bool bf16) {
  return bf16 ? (uint16_t)((__float_as_uint(v) + 0x8000u) >> 16) : __half_as_ushort(__float2half_rn(v));
}

// KIND: 1 fp32, 2 fp16, 3 bf16, 4 fp8.
template <int KIND>
struct Elem {
  static constexpr int kBytes = KIND == 1 ? 4 : (KIND == 4 ? 1 : 2);
  static constexpr int kPerWord = 4 / kBytes;
  // column k of a 32-bit word
  __device__ __forceinline__ static float of_word(uint32_t w, int k, float fp8_mult, int fp8_shift) {
    if constexpr (KIND == 1) {
      return __uint_as_float(w);
    } else if constexpr (KIND == 2) {
      return __half2float(__ushort_as_half((unsigned short)(w >> (16 * k))));
    } else if constexpr (KIND == 3) {
      return __uint_as_float((w >> (16 * k)) << 16);
    } else {
      const uint32_t v = (w >> (8 * k)) & 0xffu;
      const float mag = __fmul_rn(__uint_as_float((v & 0x7fu) << fp8_shift), fp8_mult);
      return __uint_as_float(__float_as_uint(mag) | ((v & 0x80u) << 24));
    }
  }
};

// WORD: a lane's unit is a 32-bit word holding kPerWord columns; otherwise a
// unit is one element (any alignment).
template <int KIND, bool WORD>
__global__ void __launch_bounds__(kThreads) plain_rows_kernel(const __grid_constant__ SpmdmParams p) {
  using E = Elem<KIND>;
  constexpr int CPU = WORD ? E::kPerWord : 1;  // columns per unit
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const bool off64 = p.flags & kOff64;
  const bool idx64 = p.flags & kIdx64;
  const bool weighted = p.flags & kWeighted;
  const bool positional = p.flags & kPositional;
  const bool no_bag = p.flags & kNoBag;
  const bool minus_one_skips = (p.flags & (kSbFirst | kNoBag)) == kSbFirst && KIND != 4;
  const float fp8_mult = __uint_as_float((uint32_t)(254 - p.fp8_exponent_bias) << 23);  // 2^(127 - bias)
  const int fp8_shift = 24 - (8 - p.fp8_exponent_bits);

  const bool rebase = !(p.flags & (kNoBag | kAbsOffsets));
  const int64_t off_base = rebase ? load_int(p.offsets, 0, off64) : 0;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && rebase) {
    const int64_t total = load_int(p.offsets, p.output_size, off64) - off_base;
    if (total != p.index_size) {
      report(p.status, FBGEMM_B200_STATUS_SIZE_MISMATCH, p.output_size, total, p.index_size);
    }
  }
  const int64_t bag = (int64_t)blockIdx.x * kWarps + warp;
  if (bag >= p.output_size) {
    return;
  }
  const int64_t o0 = no_bag ? bag : load_int(p.offsets, bag, off64);
  const int64_t o1 = no_bag ? bag + 1 : load_int(p.offsets, bag + 1, off64);
  const int64_t start = o0 - off_base;
  const int bag_len = (int)(o1 - o0);
  int len = bag_len < 0 ? 0 : bag_len;
  if (bag_len < 0 || start < 0 || start + len > p.index_size) {
    if (lane == 0 && blockIdx.y == 0) {
      report(p.status, FBGEMM_B200_STATUS_BAG_OVERRUN, bag, start, len);
    }
    len = 0;
  }

  // this lane's units of the row: unit u0 + 32*c, c = 0..7, if below `units`
  const int units = WORD ? (p.block_size * E::kBytes) / 4 : p.block_size;
  const int u0 = blockIdx.y * kTileUnits + lane;
  constexpr int kUnitBytes = WORD ? 4 : E::kBytes;

  float acc[kUnitsPerLane][CPU];
#pragma unroll
  for (int c = 0; c < kUnitsPerLane; ++c) {
#pragma unroll
    for (int k = 0; k < CPU; ++k) {
      acc[c][k] = 0.f;
    }
  }

  auto load_unit = [&](const uint8_t* row, int u) -> uint32_t {
    const uint8_t* a = row + (size_t)u * kUnitBytes;
    if constexpr (kUnitBytes == 4) {
      return __ldg(reinterpret_cast<const uint32_t*>(a));
    } else if constexpr (kUnitBytes == 2) {
      return __ldg(reinterpret_cast<const unsigned short*>(a));
    } else {
      return __ldg(a);
    }
  };

  for (int r0 = 0; r0 < len; r0 += kRows) {
    int64_t row_of[kRows];
    float w[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      row_of[r] = -1;
      w[r] = 1.f;
      if (r0 + r < len) {
        const int64_t pos = start + r0 + r;
        const int64_t idx = load_int(p.indices, pos, idx64);
        if (idx < 0 || idx >= p.data_size) {
          if (!(minus_one_skips && idx == -1) && lane == 0 && blockIdx.y == 0) {
            report(p.status, FBGEMM_B200_STATUS_BAD_INDEX, bag, pos, idx);
          }
        } else {
          // a pruning map turns the index into a row of the compressed table, or -1: pruned, slot still consumed
          row_of[r] = p.cit ? (int64_t)__ldg(p.cit + idx) : idx;
        }
        if (weighted) {
          w[r] = __ldg(p.weights + (positional ? (int64_t)(r0 + r) : pos));
        }
      }
    }
    uint32_t x[kRows][kUnitsPerLane];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const uint8_t* row = p.table + (row_of[r] < 0 ? 0 : row_of[r]) * p.input_stride;
#pragma unroll
      for (int c = 0; c < kUnitsPerLane; ++c) {
        const int u = u0 + 32 * c;
        x[r][c] = (row_of[r] >= 0 && u < units) ? load_unit(row, u) : 0u;
      }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      if (row_of[r] >= 0) {  // warp-uniform: every lane looks at the same row
#pragma unroll
        for (int c = 0; c < kUnitsPerLane; ++c) {
#pragma unroll
          for (int k = 0; k < CPU; ++k) {
            acc[c][k] = __fmaf_rn(w[r], E::of_word(x[r][c], k, fp8_mult, fp8_shift), acc[c][k]);
          }
        }
      }
    }
  }

  const bool normalize = (p.flags & kNormalize) && bag_len != 0;
  const float inv = normalize ? __fdiv_rn(1.f, (float)bag_len) : 1.f;
  const bool out16 = p.flags & (kOutHalf | kOutBf16);
  const bool bf16 = p.flags & kOutBf16;
  char* orow = output_row(p, bag, out16 ? 2 : 4);
#pragma unroll
  for (int c = 0; c < kUnitsPerLane; ++c) {
    const int u = u0 + 32 * c;
    if (u < units) {
#pragma unroll
      for (int k = 0; k < CPU; ++k) {
        const int col = u * CPU + k;
        const float v = normalize ? __fmul_rn(acc[c][k], inv) : acc[c][k];
        if (out16) {
          reinterpret_cast<uint16_t*>(orow)[col] = to_16bit(v, bf16);
        } else {
          reinterpret_cast<float*>(orow)[col] = v;
        }
      }
    }
  }
}

// no_bag with 8-bit output: output row m is a byte copy of table row
// indices[m] (src/RefImplementations.cc:1235-1254 for 8-bit rows, :1467-1485
// for 4-bit rows).  One warp per row; 4-byte words when everything is aligned.
__global__ void __launch_bounds__(kThreads) rows_copy_kernel(
    const uint8_t* __restrict__ table,
    const void* __restrict__ indices,
    int idx64,
    int64_t rows_out,
    int64_t data_size,
    int64_t input_stride,
    uint8_t* __restrict__ out,
    int64_t out_pitch,
    int64_t width,
    int wordwise,
    int32_t* status) {
  const int lane = threadIdx.x & 31;
  const int64_t m = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (m >= rows_out) {
    return;
  }
  const int64_t idx = load_int(indices, m, idx64 != 0);
  if (idx < 0 || idx >= data_size) {
    if (lane == 0) {
      report(status, FBGEMM_B200_STATUS_BAD_INDEX, m, m, idx);
    }
    return;
  }
  const uint8_t* src = table + idx * input_stride;
  uint8_t* dst = out + m * out_pitch;
  if (wordwise) {
    for (int64_t i = lane; i < width / 4; i += 32) {
      reinterpret_cast<uint32_t*>(dst)[i] = __ldg(reinterpret_cast<const uint32_t*>(src) + i);
    }
  } else {
    for (int64_t i = lane; i < width; i += 32) {
      dst[i] = __ldg(src + i);
    }
  }
}

using PlainFn = void (*)(const SpmdmParams);

template <bool WORD>
PlainFn pick(int kind) {
  switch (kind) {
    case 1: return plain_rows_kernel<1, WORD>;
    case 2: return plain_rows_kernel<2, WORD>;
    case 3: return plain_rows_kernel<3, WORD>;
    default: return plain_rows_kernel<4, WORD>;
  }
}

}  // namespace

cudaError_t launch_plain_rows(const SpmdmParams& p, cudaStream_t stream) {
  const int ebytes = p.in_kind == 1 ? 4 : (p.in_kind == 4 ? 1 : 2);
  const uintptr_t base = reinterpret_cast<uintptr_t>(p.table);
  const int64_t row_bytes = (int64_t)p.block_size * ebytes;
  const bool word = base % 4 == 0 && p.input_stride % 4 == 0 && row_bytes % 4 == 0;
  const int64_t units = word ? row_bytes / 4 : p.block_size;
  const int64_t tiles = (units + kTileUnits - 1) / kTileUnits;
  const int64_t blocks = (p.output_size + kWarps - 1) / kWarps;
  if (blocks <= 0 || blocks > 0x7fffffffLL || tiles <= 0 || tiles > 65535) {
    return cudaErrorInvalidValue;
  }
  PlainFn fn = word ? pick<true>(p.in_kind) : pick<false>(p.in_kind);
  fn<<<dim3((unsigned)blocks, (unsigned)tiles), kThreads, 0, stream>>>(p);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t launch_rows_copy(
    const uint8_t* table,
    const void* indices,
    int index_bytes,
    int64_t rows_out,
    int64_t data_size,
    int64_t input_stride,
    uint8_t* out,
    int64_t out_pitch,
    int64_t width,
    int32_t* status,
    cudaStream_t stream) {
  const int64_t blocks = (rows_out + kWarps - 1) / kWarps;
  if (blocks <= 0 || blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  const uintptr_t a = reinterpret_cast<uintptr_t>(table), b = reinterpret_cast<uintptr_t>(out);
  const int wordwise = ((a | b | (uintptr_t)input_stride | (uintptr_t)out_pitch | (uintptr_t)width) & 3) == 0;
  rows_copy_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(
      table, indices, index_bytes == 8, rows_out, data_size, input_stride, out, out_pitch, width, wordwise, status);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

// Sequence ("nobag") lookup over the tables of a table-batched operator: one
// output row per index, no pooling - out[k, :] is the dequantized (or copied)
// row indices[k] of the table that position k belongs to.
//
// Reference: int_nbit_split_embedding_nobag_codegen_forward_unweighted_cpu,
// fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:206-520
// of FBGEMM (the `nobag` branch).  Per table it builds offsets of bags of one
// (:391-395) and calls the pooled kernel of the table's row type with
// has_weight = false (:421-473), so a row of a quantized table comes out as
//     out[j] = fma(scale, q[j], 0.0f + bias)      (src/RefImplementations.cc:1290-1346, :1485-1541)
// and a row of an unquantized or FP8 table as fma(1.0f, x[j], 0.0f) (:1347-1424,
// :1543-1615); with INT8 or INT4 output it calls the kernels' no_bag forms,
// which copy row bytes (:1235-1254, :1467-1485).  Output row k sits at
// k * (D + qparams) elements: the tables' outputs follow one another in the
// order of their positions (D_start = offsets[t*B] * elems_D, :351-352).
//
// One launch for all tables, nothing read back to the host.  A warp owns 32
// consecutive positions.  First every lane prepares one of them - its table by
// bisection over the T+1 table starts, the index, the bounds check, the row
// address, scale and bias - so that this chain of dependent loads is paid once
// per 32 positions; then the warp walks the positions (the lane's findings
// broadcast by shuffles): lane l produces columns 4l .. 4l+3 (+128, ...) from one
// load of the 1-16 bytes that hold them and one 8- or 16-byte store, by code
// compiled for the row type and the output type, so that the stores - which
// are most of the traffic, 4 or 2 bytes per column against 1/4 to 4 read - are
// coalesced and wide; widths that are no multiple of 4 and unaligned rows go
// column by column.
#include <cuda_fp16.h>

#include "internal.h"
#include "position_tables.cuh"

namespace fbgemm_b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPerWarp = 32;  // positions a warp walks: one per lane in the prologue

// SparseType of fbgemm_gpu/include/fbgemm_gpu/embedding_common.h:20-32
enum : int { kFP32 = 0, kFP16 = 1, kINT8 = 2, kINT4 = 3, kINT2 = 4, kFP8 = 6 };

struct SeqArgs {
  const uint8_t* weights;
  const SequenceTable* tables;  // [T], device
  const void* indices;
  const void* offsets;
  uint8_t* out;
  int32_t* status;
  int64_t index_size;
  int64_t out_row_bytes;
  int32_t T;
  int32_t B;
  int32_t D;
  int32_t out_kind;  // FBGEMM_B200_OUT_F32/_F16/_BF16/_U8, 4 = packed int4 rows
  int32_t index64;
  int32_t sb_last;
  int32_t fp8_exponent_bits;
  int32_t fp8_exponent_bias;
  int32_t by_fours;  // D % 4 == 0 and output rows aligned for 8- / 16-byte stores
};

__device__ __noinline__ void report(int32_t* st, int code, int64_t table, int64_t pos, int64_t val) {
  if (atomicCAS(st, 0, code) == 0) {
    st[1] = (int32_t)table;
    st[2] = (int32_t)pos;
    st[3] = (int32_t)val;
  }
}

__device__ __forceinline__ uint32_t load_bytes(const uint8_t* p, int n) {
  uint32_t v = 0;
  for (int i = 0; i < n; ++i) {
    v |= (uint32_t)__ldg(p + i) << (8 * i);
  }
  return v;
}

__device__ __forceinline__ uint16_t to_16bit(float v, bool bf16) {
  return bf16 ? (uint16_t)((__float_as_uint(v) + 0x8000u) >> 16) : __half_as_ushort(__float2half_rn(v));
}

// What a lane finds out about its position before the warp walks the 32 positions.
enum : int { kSkip = 0, kZeros = 1, kRow = 2 };

// Output forms the kernel is compiled for.
enum : int { kToF32 = 0, kToF16 = 1, kToBf16 = 2, kCopy = 3 };

// One decoded column, as the pooled kernel of the row type computes a bag of that one row without
// weights: fma(scale, q, 0 + bias) for quantized rows, fma(1, x, 0) otherwise.
__device__ __forceinline__ float from_q(uint32_t q, float scale, float start) {
  return __fmaf_rn(scale, (float)(int)q, start);
}
__device__ __forceinline__ float from_x(float x) {
  return __fmaf_rn(1.f, x, 0.f);
}
__device__ __forceinline__ float from_fp8(uint32_t f, float fp8_mult, int fp8_shift) {
  const float mag = __fmul_rn(__uint_as_float((f & 0x7fu) << fp8_shift), fp8_mult);
  return from_x(__uint_as_float(__float_as_uint(mag) | ((f & 0x80u) << 24)));
}

template <int OUT>
__device__ __forceinline__ void store_column(uint8_t* orow, int j, float v) {
  if constexpr (OUT == kToF32) {
    reinterpret_cast<float*>(orow)[j] = v;
  } else {
    reinterpret_cast<uint16_t*>(orow)[j] = to_16bit(v, OUT == kToBf16);
  }
}

// Four consecutive columns per lane and step: one load of the 1-16 bytes that hold them, one store of
// 8 or 16 bytes.  The caller has checked that D is a multiple of 4 and that loads and stores are aligned.
template <int TYPE, int OUT>
__device__ __forceinline__ void emit_row_by_fours(const uint8_t* data, uint8_t* orow, int D, float scale, float start,
                                                  float fp8_mult, int fp8_shift, int lane) {
  for (int u = lane; u < (D >> 2); u += 32) {
    float v[4];
    if constexpr (TYPE == kINT8) {
      const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(data) + u);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        v[c] = from_q((w >> (8 * c)) & 0xffu, scale, start);
      }
    } else if constexpr (TYPE == kINT4) {
      const uint32_t w = __ldg(reinterpret_cast<const unsigned short*>(data) + u);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        v[c] = from_q((w >> (4 * c)) & 0xfu, scale, start);
      }
    } else if constexpr (TYPE == kINT2) {
      const uint32_t w = __ldg(data + u);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        v[c] = from_q((w >> (2 * c)) & 0x3u, scale, start);
      }
    } else if constexpr (TYPE == kFP32) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(data) + u);
      v[0] = from_x(__uint_as_float(w.x));
      v[1] = from_x(__uint_as_float(w.y));
      v[2] = from_x(__uint_as_float(w.z));
      v[3] = from_x(__uint_as_float(w.w));
    } else if constexpr (TYPE == kFP16) {
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(data) + u);
      v[0] = from_x(__half2float(__ushort_as_half((unsigned short)(w.x & 0xffffu))));
      v[1] = from_x(__half2float(__ushort_as_half((unsigned short)(w.x >> 16))));
      v[2] = from_x(__half2float(__ushort_as_half((unsigned short)(w.y & 0xffffu))));
      v[3] = from_x(__half2float(__ushort_as_half((unsigned short)(w.y >> 16))));
    } else {
      const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(data) + u);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        v[c] = from_fp8((w >> (8 * c)) & 0xffu, fp8_mult, fp8_shift);
      }
    }
    if constexpr (OUT == kToF32) {
      reinterpret_cast<float4*>(orow)[u] = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      constexpr bool bf = OUT == kToBf16;
      reinterpret_cast<uint2*>(orow)[u] = make_uint2((uint32_t)to_16bit(v[0], bf) | ((uint32_t)to_16bit(v[1], bf) << 16),
                                                     (uint32_t)to_16bit(v[2], bf) | ((uint32_t)to_16bit(v[3], bf) << 16));
    }
  }
}

// Any width and alignment: one column per lane and step.
template <int OUT>
__device__ __forceinline__ void emit_row_by_columns(const uint8_t* data, int type, uint8_t* orow, int D, float scale,
                                                    float start, float fp8_mult, int fp8_shift, int lane) {
  if (type == kINT8 || type == kINT4 || type == kINT2) {
    const int bits = type == kINT8 ? 8 : (type == kINT4 ? 4 : 2);
    const int shift_per = bits == 8 ? 0 : (bits == 4 ? 1 : 2);  // log2(columns per byte)
    const uint32_t mask = (1u << bits) - 1u;
    for (int j = lane; j < D; j += 32) {
      const uint32_t byte = __ldg(data + (j >> shift_per));
      store_column<OUT>(orow, j, from_q((byte >> ((j & ((1 << shift_per) - 1)) * bits)) & mask, scale, start));
    }
  } else if (type == kFP32) {
    const bool aligned = (reinterpret_cast<uintptr_t>(data) & 3) == 0;
    for (int j = lane; j < D; j += 32) {
      const uint8_t* e = data + 4 * (int64_t)j;
      store_column<OUT>(orow, j, from_x(__uint_as_float(aligned ? __ldg(reinterpret_cast<const uint32_t*>(e))
                                                                : load_bytes(e, 4))));
    }
  } else if (type == kFP16) {
    const bool aligned = (reinterpret_cast<uintptr_t>(data) & 1) == 0;
    for (int j = lane; j < D; j += 32) {
      const uint8_t* e = data + 2 * (int64_t)j;
      const uint32_t h = aligned ? (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(e)) : load_bytes(e, 2);
      store_column<OUT>(orow, j, from_x(__half2float(__ushort_as_half((unsigned short)h))));
    }
  } else {
    for (int j = lane; j < D; j += 32) {
      store_column<OUT>(orow, j, from_fp8(__ldg(data + j), fp8_mult, fp8_shift));
    }
  }
}

template <int OUT>
__global__ void __launch_bounds__(kThreads) sequence_rows_kernel(const SeqArgs a) {
  __shared__ int64_t starts_s[kSharedStarts];
  const int64_t* starts = stage_table_starts(a, starts_s);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const float fp8_mult = __uint_as_float((uint32_t)(254 - a.fp8_exponent_bias) << 23);  // 2^(127 - bias)
  const int fp8_shift = 24 - (8 - a.fp8_exponent_bits);
  constexpr bool copy = OUT == kCopy;
  const int64_t first = ((int64_t)blockIdx.x * kWarps + warp) * 32;
  if (first >= a.index_size) {
    return;
  }

  // Prologue, one position per lane: table, index, bounds, row address, scale and bias.  The chain of
  // dependent loads (offsets -> index -> descriptor -> scale, bias) is paid once per 32 positions.
  int my_state = kSkip, my_type = 0, my_row_bytes = 0;
  bool my_fours = false;
  const uint8_t* my_row = nullptr;
  float my_scale = 0.f, my_start = 0.f;
  {
    const int64_t k = first + lane;
    const int t = k < a.index_size ? table_of(a, starts, k) : -1;
    if (t >= 0) {
      const int64_t idx = load_position_int(a.indices, k, a.index64);
      const SequenceTable tab = a.tables[t];
      my_type = tab.type;
      my_row_bytes = tab.row_bytes;
      // Scale and bias first makes -1 a pruned row of the pooled kernels (not for FP8 rows): the bag of
      // one pools nothing.  The byte copies know no pruned row.
      const bool pruned = !copy && !a.sb_last && idx == -1 && my_type != kFP8;
      if (pruned) {
        my_state = kZeros;
      } else if (idx < 0 || idx >= tab.rows) {
        report(a.status, FBGEMM_B200_STATUS_BAD_INDEX, t, k, idx);
      } else {
        my_state = kRow;
        my_row = a.weights + tab.weight_offset + idx * (int64_t)tab.row_bytes;
        if (!copy) {
          // where the columns start, and whether the four-column path can take this row: the bytes that
          // hold four columns are the alignment it needs
          const bool quantized = my_type == kINT8 || my_type == kINT4 || my_type == kINT2;
          const int unit = my_type == kFP32 ? 16 : (my_type == kFP16 ? 8 : (my_type == kINT4 ? 2 : (my_type == kINT2 ? 1 : 4)));
          const uint8_t* data = my_row + (quantized && !a.sb_last ? 4 : 0);
          my_fours = a.by_fours && (reinterpret_cast<uintptr_t>(data) & (unit - 1)) == 0;
        }
        // Ask for the row now: the warp reaches it up to 31 positions later, and by then it sits in L2.
        for (int b = 0; b < tab.row_bytes; b += 128) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(my_row + b));
        }
        asm volatile("prefetch.global.L2 [%0];" ::"l"(my_row + tab.row_bytes - 1));
        if (!copy && (my_type == kINT8 || my_type == kINT4 || my_type == kINT2)) {
          const int bits = my_type == kINT8 ? 8 : (my_type == kINT4 ? 4 : 2);
          const uint8_t* sb = my_row + (a.sb_last ? (a.D * bits + 7) / 8 : 0);
          float bias;
          if (my_type == kINT8 && a.sb_last) {
            my_scale = __uint_as_float(load_bytes(sb, 4));
            bias = __uint_as_float(load_bytes(sb + 4, 4));
          } else {
            const uint32_t pair = load_bytes(sb, 4);
            my_scale = __half2float(__ushort_as_half((unsigned short)(pair & 0xffffu)));
            bias = __half2float(__ushort_as_half((unsigned short)(pair >> 16)));
          }
          my_start = __fadd_rn(0.f, bias);  // the reference's buf[j] + bias with buf[j] = 0
        }
      }
    }
  }

  // what the warp needs to know first about a position, in one word: state | type << 2 | four-column path << 5
  const int my_code = my_state | (my_type << 2) | ((int)my_fours << 5);
  const int count = (int)(a.index_size - first < 32 ? a.index_size - first : 32);
  uint8_t* orow = a.out + first * a.out_row_bytes;
  for (int i = 0; i < count; ++i, orow += a.out_row_bytes) {
    const int code = __shfl_sync(0xffffffffu, my_code, i);
    const int state = code & 3;
    if (state == kSkip) {
      continue;
    }
    if (state == kZeros) {
      if constexpr (!copy) {
        for (int j = lane; j < a.D; j += 32) {
          store_column<OUT>(orow, j, 0.f);
        }
      }
      continue;
    }
    const uint8_t* row = reinterpret_cast<const uint8_t*>(
        __shfl_sync(0xffffffffu, (unsigned long long)reinterpret_cast<uintptr_t>(my_row), i));
    const int type = (code >> 2) & 7;

    if constexpr (copy) {
      // byte copy of the row: min(output row, table row) bytes (for 4-bit rows the caller makes the two equal)
      const int64_t row_bytes = __shfl_sync(0xffffffffu, my_row_bytes, i);
      const int64_t width = a.out_row_bytes < row_bytes ? a.out_row_bytes : row_bytes;
      if (((reinterpret_cast<uintptr_t>(row) | reinterpret_cast<uintptr_t>(orow)) & 3) == 0) {
        for (int64_t b = lane; b < width / 4; b += 32) {
          reinterpret_cast<uint32_t*>(orow)[b] = __ldg(reinterpret_cast<const uint32_t*>(row) + b);
        }
        for (int64_t b = (width & ~(int64_t)3) + lane; b < width; b += 32) {
          orow[b] = __ldg(row + b);
        }
      } else {
        for (int64_t b = lane; b < width; b += 32) {
          orow[b] = __ldg(row + b);
        }
      }
    } else {
      const bool quantized = type == kINT8 || type == kINT4 || type == kINT2;
      float scale = 0.f, start = 0.f;
      if (quantized) {
        scale = __shfl_sync(0xffffffffu, my_scale, i);
        start = __shfl_sync(0xffffffffu, my_start, i);
      }
      const uint8_t* data = row + (quantized && !a.sb_last ? 4 : 0);
      if (code & 32) {
        switch (type) {
          case kINT8: emit_row_by_fours<kINT8, OUT>(data, orow, a.D, scale, start, fp8_mult, fp8_shift, lane); break;
          case kINT4: emit_row_by_fours<kINT4, OUT>(data, orow, a.D, scale, start, fp8_mult, fp8_shift, lane); break;
          case kINT2: emit_row_by_fours<kINT2, OUT>(data, orow, a.D, scale, start, fp8_mult, fp8_shift, lane); break;
          case kFP32: emit_row_by_fours<kFP32, OUT>(data, orow, a.D, scale, start, fp8_mult, fp8_shift, lane); break;
          case kFP16: emit_row_by_fours<kFP16, OUT>(data, orow, a.D, scale, start, fp8_mult, fp8_shift, lane); break;
          default: emit_row_by_fours<kFP8, OUT>(data, orow, a.D, scale, start, fp8_mult, fp8_shift, lane); break;
        }
      } else {
        emit_row_by_columns<OUT>(data, type, orow, a.D, scale, start, fp8_mult, fp8_shift, lane);
      }
    }
  }
}

}  // namespace

cudaError_t launch_sequence_lookup(
    const uint8_t* weights,
    const SequenceTable* tables,
    int32_t T,
    int32_t B,
    int32_t D,
    const void* indices,
    const void* offsets,
    int index_bytes,
    int64_t index_size,
    void* out,
    int out_kind,
    int64_t out_row_bytes,
    bool scale_bias_last,
    int fp8_exponent_bits,
    int fp8_exponent_bias,
    int32_t* status,
    cudaStream_t stream) {
  if (index_size == 0) {
    return cudaSuccess;
  }
  SeqArgs a{};
  a.weights = weights;
  a.tables = tables;
  a.indices = indices;
  a.offsets = offsets;
  a.out = static_cast<uint8_t*>(out);
  a.status = status;
  a.index_size = index_size;
  a.out_row_bytes = out_row_bytes;
  a.T = T;
  a.B = B;
  a.D = D;
  a.out_kind = out_kind;
  a.index64 = index_bytes == 8;
  a.sb_last = scale_bias_last;
  a.fp8_exponent_bits = fp8_exponent_bits;
  a.fp8_exponent_bias = fp8_exponent_bias;
  const int64_t per_block = (int64_t)kWarps * kPerWarp;
  const int64_t blocks = (index_size + per_block - 1) / per_block;
  if (blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  const int64_t store_bytes = out_kind == FBGEMM_B200_OUT_F32 ? 16 : 8;
  a.by_fours = D % 4 == 0 && reinterpret_cast<uintptr_t>(out) % store_bytes == 0 && out_row_bytes % store_bytes == 0;
  switch (out_kind) {
    case FBGEMM_B200_OUT_F32: sequence_rows_kernel<kToF32><<<(unsigned)blocks, kThreads, 0, stream>>>(a); break;
    case FBGEMM_B200_OUT_F16: sequence_rows_kernel<kToF16><<<(unsigned)blocks, kThreads, 0, stream>>>(a); break;
    case FBGEMM_B200_OUT_BF16: sequence_rows_kernel<kToBf16><<<(unsigned)blocks, kThreads, 0, stream>>>(a); break;
    default: sequence_rows_kernel<kCopy><<<(unsigned)blocks, kThreads, 0, stream>>>(a); break;
  }
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

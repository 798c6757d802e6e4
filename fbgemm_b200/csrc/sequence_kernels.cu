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
// One launch for all tables, nothing read back to the host: a warp owns a
// position, finds its table by bisection over the T+1 table starts, and lane l
// produces columns l, l+32, ... so that the stores - which are most of the
// traffic, 4 or 2 bytes per column against 1/4 to 4 read - are coalesced; the
// row bytes a warp reads sit in one or two cache lines.
#include <cuda_fp16.h>

#include "internal.h"
#include "position_tables.cuh"

namespace fbgemm_b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPerWarp = 4;  // positions a warp walks

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

__global__ void __launch_bounds__(kThreads) sequence_rows_kernel(const SeqArgs a) {
  __shared__ int64_t starts_s[kSharedStarts];
  const int64_t* starts = stage_table_starts(a, starts_s);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const float fp8_mult = __uint_as_float((uint32_t)(254 - a.fp8_exponent_bias) << 23);  // 2^(127 - bias)
  const int fp8_shift = 24 - (8 - a.fp8_exponent_bits);
  const int64_t first = ((int64_t)blockIdx.x * kWarps + warp) * kPerWarp;
  for (int i = 0; i < kPerWarp; ++i) {
    const int64_t k = first + i;
    if (k >= a.index_size) {
      return;
    }
    const int t = table_of(a, starts, k);
    if (t < 0) {
      continue;
    }
    const int64_t idx = load_position_int(a.indices, k, a.index64);
    const SequenceTable tab = a.tables[t];
    const int type = tab.type;
    uint8_t* orow = a.out + k * a.out_row_bytes;
    const bool quantized = type == kINT8 || type == kINT4 || type == kINT2;

    if (a.out_kind >= FBGEMM_B200_OUT_U8) {
      // byte copy of the row: 8-bit rows min(output row, table row) bytes, 4-bit rows the whole table row
      if (idx < 0 || idx >= tab.rows) {
        if (lane == 0) {
          report(a.status, FBGEMM_B200_STATUS_BAD_INDEX, t, k, idx);
        }
        continue;
      }
      const uint8_t* row = a.weights + tab.weight_offset + idx * (int64_t)tab.row_bytes;
      const int64_t width =
          a.out_kind == FBGEMM_B200_OUT_U8 && a.out_row_bytes < tab.row_bytes ? a.out_row_bytes : tab.row_bytes;
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
      continue;
    }

    const bool out16 = a.out_kind != FBGEMM_B200_OUT_F32;
    const bool bf16 = a.out_kind == FBGEMM_B200_OUT_BF16;
    // Scale and bias first makes -1 a pruned row (not for FP8 rows): the bag of one pools nothing.
    const bool pruned = !a.sb_last && idx == -1 && type != kFP8;
    if (!pruned && (idx < 0 || idx >= tab.rows)) {
      if (lane == 0) {
        report(a.status, FBGEMM_B200_STATUS_BAD_INDEX, t, k, idx);
      }
      continue;
    }
    if (pruned) {
      for (int j = lane; j < a.D; j += 32) {
        if (out16) {
          reinterpret_cast<uint16_t*>(orow)[j] = 0;
        } else {
          reinterpret_cast<float*>(orow)[j] = 0.f;
        }
      }
      continue;
    }
    const uint8_t* row = a.weights + tab.weight_offset + idx * (int64_t)tab.row_bytes;
    if (quantized) {
      const int bits = type == kINT8 ? 8 : (type == kINT4 ? 4 : 2);
      const int payload_bytes = (a.D * bits + 7) / 8;
      const uint8_t* payload = row + (a.sb_last ? 0 : 4);
      const uint8_t* sb = row + (a.sb_last ? payload_bytes : 0);
      float scale, bias;
      if (type == kINT8 && a.sb_last) {
        scale = __uint_as_float(load_bytes(sb, 4));
        bias = __uint_as_float(load_bytes(sb + 4, 4));
      } else {
        const uint32_t pair = load_bytes(sb, 4);
        scale = __half2float(__ushort_as_half((unsigned short)(pair & 0xffffu)));
        bias = __half2float(__ushort_as_half((unsigned short)(pair >> 16)));
      }
      const float start = __fadd_rn(0.f, bias);  // the reference's buf[j] + bias with buf[j] = 0
      const int per_byte = 8 / bits;
      const uint32_t mask = (1u << bits) - 1u;
      for (int j = lane; j < a.D; j += 32) {
        const uint32_t byte = __ldg(payload + j / per_byte);
        const float q = (float)(int)((byte >> ((j % per_byte) * bits)) & mask);
        const float v = __fmaf_rn(scale, q, start);
        if (out16) {
          reinterpret_cast<uint16_t*>(orow)[j] = to_16bit(v, bf16);
        } else {
          reinterpret_cast<float*>(orow)[j] = v;
        }
      }
    } else {
      const int elem_bytes = type == kFP32 ? 4 : (type == kFP16 ? 2 : 1);
      const bool aligned = (reinterpret_cast<uintptr_t>(row) & (elem_bytes - 1)) == 0;
      for (int j = lane; j < a.D; j += 32) {
        const uint8_t* e = row + (int64_t)j * elem_bytes;
        float x;
        if (type == kFP32) {
          x = __uint_as_float(aligned ? __ldg(reinterpret_cast<const uint32_t*>(e)) : load_bytes(e, 4));
        } else if (type == kFP16) {
          const uint32_t h = aligned ? (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(e)) : load_bytes(e, 2);
          x = __half2float(__ushort_as_half((unsigned short)h));
        } else {
          const uint32_t f = __ldg(e);
          const float mag = __fmul_rn(__uint_as_float((f & 0x7fu) << fp8_shift), fp8_mult);
          x = __uint_as_float(__float_as_uint(mag) | ((f & 0x80u) << 24));
        }
        const float v = __fmaf_rn(1.f, x, 0.f);
        if (out16) {
          reinterpret_cast<uint16_t*>(orow)[j] = to_16bit(v, bf16);
        } else {
          reinterpret_cast<float*>(orow)[j] = v;
        }
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
  sequence_rows_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(a);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

// Pooled lookup over fused row-wise quantized tables (8-, 4- and 2-bit) for
// sm_100a.  Stands in for the x86 code FBGEMM generates at run time
// (src/EmbeddingSpMDM.cc:161-968, src/EmbeddingSpMDMNBit.cc:149-971) and
// follows the arithmetic of its scalar reference
// (src/RefImplementations.cc:1290-1346, :1485-1541, :1746-1822) operation for
// operation, so that fp32 results are bit-equal:
//
//     acc[j] = fma(w*scale, q[j], acc[j] + w*bias)    rows in index order
//
// This file holds (1) the staged kernel, which takes every shape and option,
// (2) the dispatcher that sends a lookup to one of the register-resident
// direct kernels (spmdm_direct.cuh; dense or compacting) when a variant fits
// the row width, else to the staged kernel, and (3) the multi-table plans that
// put up to 16 tables of the same variant into one launch.
//
// Scheduling of the staged kernel.  A bag is owned by a group of LPB lanes (8,
// 16 or a full warp,
// chosen from the row width), so a warp pools 4, 2 or 1 bags at once and the
// rows of one bag are accumulated strictly in order (no cross-lane reduction:
// that would change the rounding).  What IS parallel inside a bag is the
// memory traffic: a wave of up to `rows_per_wave` rows is copied from HBM/L2
// into the group's shared-memory stage with cp.async, all rows in flight at
// once, every lane of the group issuing a slice of the flat word list.  Only
// then are the staged rows walked in order: each lane owns CPL 4-byte chunks
// of the packed payload (4, 8 or 16 columns each), unpacks them with byte
// permutes into exact fp32 integers and applies the two roundings above.
//
// The kernel is HBM/L2-latency bound (about 2 flop per byte); tensor cores
// have no role here.
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include <algorithm>
#include <vector>

#include "internal.h"
#include "spmdm_direct.cuh"

namespace fbgemm_b200 {

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kThreads = kWarpsPerBlock * 32;

__device__ __forceinline__ int64_t load_int(const void* p, int64_t i, bool is64) {
  return is64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(p) + i)
              : (int64_t)__ldg(reinterpret_cast<const int*>(p) + i);
}

// First error wins; the rest of the record is diagnostics only.
__device__ __noinline__ void report(int32_t* st, int code, int64_t bag, int64_t pos, int64_t val) {
  if (atomicCAS(st, 0, code) == 0) {
    st[1] = (int32_t)bag;
    st[2] = (int32_t)pos;
    st[3] = (int32_t)val;
  }
}

template <int W>
__device__ __forceinline__ void cp_async(uint32_t dst, const void* src) {
  if constexpr (W == 16) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
  } else if constexpr (W == 8) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(src) : "memory");
  } else {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory");
  }
}

__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;\n" ::: "memory");
}

// Copy rows [0, n) of the wave into the stage.  The rows are seen as one flat
// list of W-byte words; lane `gl` of `lpb` takes words gl, gl+lpb, ...
template <int W>
__device__ __forceinline__ void stage_rows(
    const SpmdmParams& p,
    uint8_t* s_rows,
    const long long* s_off,
    int n,
    int gl,
    int lpb) {
  const int wpr = p.row_bytes / W;  // words per row
  const int drow = lpb / wpr;
  const int dw = lpb - drow * wpr;
  int row = gl / wpr;
  int w = gl - row * wpr;
  const uint32_t s_base = (uint32_t)__cvta_generic_to_shared(s_rows);
  while (row < n) {
    const long long off = s_off[row];
    if (off >= 0) {
      cp_async<W>(s_base + row * p.pitch + w * W, p.table + off + w * W);
    }
    w += dw;
    row += drow;
    if (w >= wpr) {
      w -= wpr;
      ++row;
    }
  }
}

// Rows whose address, pitch or width is not a multiple of 4 bytes: plain byte
// loads.  The payload lands at [data_off, data_off + data_bytes), scale,bias
// at sb_off, wherever they sit in the table row.
__device__ __forceinline__ void stage_rows_bytewise(
    const SpmdmParams& p,
    uint8_t* s_rows,
    const long long* s_off,
    int n,
    int gl,
    int lpb) {
  const int total = n * p.row_bytes;
  for (int k = gl; k < total; k += lpb) {
    const int row = k / p.row_bytes;
    const int b = k - row * p.row_bytes;
    const long long off = s_off[row];
    if (off >= 0) {
      const bool payload = b >= p.data_row_off && b < p.data_row_off + p.data_bytes;
      const int dst = payload ? p.data_off + (b - p.data_row_off) : p.sb_off + (b - p.sb_row_off);
      s_rows[row * p.pitch + dst] = __ldg(p.table + off + b);
    }
  }
}

// Byte `i` of x as an exact fp32 integer: the byte is planted in the mantissa
// of 2^23 and 2^23 is subtracted.
template <int I>
__device__ __forceinline__ float byte_to_float(uint32_t x) {
  return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540u | I)) - 8388608.0f;
}

__device__ __forceinline__ float pool(float acc, float q, float scale, float bias) {
  // Two roundings, as in std::fma(scale, q, buf[j] + bias).
  return __fmaf_rn(scale, q, __fadd_rn(acc, bias));
}

template <int BITS>
__device__ __forceinline__ void accumulate(float* acc, uint32_t x, float scale, float bias) {
  if constexpr (BITS == 8) {
    acc[0] = pool(acc[0], byte_to_float<0>(x), scale, bias);
    acc[1] = pool(acc[1], byte_to_float<1>(x), scale, bias);
    acc[2] = pool(acc[2], byte_to_float<2>(x), scale, bias);
    acc[3] = pool(acc[3], byte_to_float<3>(x), scale, bias);
  } else if constexpr (BITS == 4) {
    // element 2k is the low nibble of byte k, element 2k+1 the high nibble
    const uint32_t lo = x & 0x0F0F0F0Fu;
    const uint32_t hi = (x >> 4) & 0x0F0F0F0Fu;
    acc[0] = pool(acc[0], byte_to_float<0>(lo), scale, bias);
    acc[1] = pool(acc[1], byte_to_float<0>(hi), scale, bias);
    acc[2] = pool(acc[2], byte_to_float<1>(lo), scale, bias);
    acc[3] = pool(acc[3], byte_to_float<1>(hi), scale, bias);
    acc[4] = pool(acc[4], byte_to_float<2>(lo), scale, bias);
    acc[5] = pool(acc[5], byte_to_float<2>(hi), scale, bias);
    acc[6] = pool(acc[6], byte_to_float<3>(lo), scale, bias);
    acc[7] = pool(acc[7], byte_to_float<3>(hi), scale, bias);
  } else {
    // element 4k+i sits in bits [2i+1 : 2i] of byte k
    const uint32_t t0 = x & 0x03030303u;
    const uint32_t t1 = (x >> 2) & 0x03030303u;
    const uint32_t t2 = (x >> 4) & 0x03030303u;
    const uint32_t t3 = (x >> 6) & 0x03030303u;
    acc[0] = pool(acc[0], byte_to_float<0>(t0), scale, bias);
    acc[1] = pool(acc[1], byte_to_float<0>(t1), scale, bias);
    acc[2] = pool(acc[2], byte_to_float<0>(t2), scale, bias);
    acc[3] = pool(acc[3], byte_to_float<0>(t3), scale, bias);
    acc[4] = pool(acc[4], byte_to_float<1>(t0), scale, bias);
    acc[5] = pool(acc[5], byte_to_float<1>(t1), scale, bias);
    acc[6] = pool(acc[6], byte_to_float<1>(t2), scale, bias);
    acc[7] = pool(acc[7], byte_to_float<1>(t3), scale, bias);
    acc[8] = pool(acc[8], byte_to_float<2>(t0), scale, bias);
    acc[9] = pool(acc[9], byte_to_float<2>(t1), scale, bias);
    acc[10] = pool(acc[10], byte_to_float<2>(t2), scale, bias);
    acc[11] = pool(acc[11], byte_to_float<2>(t3), scale, bias);
    acc[12] = pool(acc[12], byte_to_float<3>(t0), scale, bias);
    acc[13] = pool(acc[13], byte_to_float<3>(t1), scale, bias);
    acc[14] = pool(acc[14], byte_to_float<3>(t2), scale, bias);
    acc[15] = pool(acc[15], byte_to_float<3>(t3), scale, bias);
  }
}

// fp32 -> fp16 (round to nearest even) or bf16 as the reference rounds it,
// (bits + 0x8000) >> 16 (include/fbgemm/FloatConversion.h:312-315).
__device__ __forceinline__ uint16_t to_16bit(float v, bool bf16) {
  return bf16 ? (uint16_t)((__float_as_uint(v) + 0x8000u) >> 16) : __half_as_ushort(__float2half_rn(v));
}

template <int COLS>
__device__ __forceinline__ void store_chunk(
    const SpmdmParams& p,
    int64_t bag,
    int col0,
    const float* v) {
  const bool full = col0 + COLS <= p.block_size;
  if (p.flags & (kOutHalf | kOutBf16)) {
    const bool bf16 = p.flags & kOutBf16;
    uint16_t* o = reinterpret_cast<uint16_t*>(output_row(p, bag, 2)) + col0;
    if (full && (p.flags & kOutVec)) {
      uint32_t w[COLS / 2];
#pragma unroll
      for (int i = 0; i < COLS / 2; ++i) {
        w[i] = (uint32_t)to_16bit(v[2 * i], bf16) | ((uint32_t)to_16bit(v[2 * i + 1], bf16) << 16);
      }
      if constexpr (COLS == 4) {
        *reinterpret_cast<uint2*>(o) = make_uint2(w[0], w[1]);
      } else {
#pragma unroll
        for (int i = 0; i < COLS / 8; ++i) {
          reinterpret_cast<uint4*>(o)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < COLS; ++i) {
        if (col0 + i < p.block_size) {
          o[i] = to_16bit(v[i], bf16);
        }
      }
    }
  } else {
    float* o = reinterpret_cast<float*>(output_row(p, bag, 4)) + col0;
    if (full && (p.flags & kOutVec)) {
#pragma unroll
      for (int i = 0; i < COLS / 4; ++i) {
        reinterpret_cast<float4*>(o)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < COLS; ++i) {
        if (col0 + i < p.block_size) {
          o[i] = v[i];
        }
      }
    }
  }
}

// BITS: 8, 4, 2.  LPB: lanes per bag.  CPL: 4-byte payload chunks per lane.
template <int BITS, int LPB, int CPL>
__global__ void __launch_bounds__(kThreads)
spmdm_kernel(const __grid_constant__ SpmdmParams p) {
  constexpr int GPW = 32 / LPB;    // bags per warp
  constexpr int COLS = 32 / BITS;  // columns per 4-byte chunk
  extern __shared__ __align__(16) uint8_t smem[];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int grp = lane / LPB;
  const int gl = lane % LPB;
  const unsigned gmask = LPB == 32 ? 0xffffffffu : (((1u << LPB) - 1u) << (grp * LPB));
  const bool idx64 = p.flags & kIdx64;
  const bool off64 = p.flags & kOff64;
  const bool weighted = p.flags & kWeighted;
  const bool positional = p.flags & kPositional;
  const bool pruned = p.flags & kPruned;

  const bool no_bag = p.flags & kNoBag;
  const bool half_sb = BITS != 8 || (p.flags & kSbFirst);
  // rebasing to offsets[0] (the functor's convention) unless the offsets are absolute
  const bool rebase = !(p.flags & (kNoBag | kAbsOffsets));
  const int64_t off_base = rebase ? load_int(p.offsets, 0, off64) : 0;
  if (blockIdx.x == 0 && threadIdx.x == 0 && rebase) {
    // `return current == index_size` of the reference
    const int64_t total = load_int(p.offsets, p.output_size, off64) - off_base;
    if (total != p.index_size) {
      report(p.status, FBGEMM_B200_STATUS_SIZE_MISMATCH, p.output_size, total, p.index_size);
    }
  }

  const int64_t bag = ((int64_t)blockIdx.x * kWarpsPerBlock + warp) * GPW + grp;
  if (bag >= p.output_size) {
    return;
  }

  // no_bag: output row m is the single row indices[m]
  const int64_t o0 = no_bag ? bag : load_int(p.offsets, bag, off64);
  const int64_t o1 = no_bag ? bag + 1 : load_int(p.offsets, bag + 1, off64);
  const int64_t start = o0 - off_base;
  const int bag_len = (int)(o1 - o0);  // the reference narrows to 32 bits too
  int len = bag_len < 0 ? 0 : bag_len;
  // Offsets that step backwards: the reference, which walks the index array
  // with a running position, ends up past index_size and returns false.
  if (bag_len < 0 || start < 0 || start + len > p.index_size) {
    if (gl == 0) {
      report(p.status, FBGEMM_B200_STATUS_BAG_OVERRUN, bag, start, len);
    }
    len = 0;  // never read past the caller's arrays
  }

  const int S = p.rows_per_wave;
  uint8_t* s_rows = smem + (size_t)(warp * GPW + grp) * p.group_smem;
  long long* s_off = reinterpret_cast<long long*>(s_rows + ((S * p.pitch + 15) & ~15));
  float* s_w = reinterpret_cast<float*>(s_off + S);
  const int nchunks = (p.data_bytes + 3) >> 2;

  float acc[CPL][COLS];
#pragma unroll
  for (int ci = 0; ci < CPL; ++ci) {
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      acc[ci][j] = 0.f;
    }
  }

  for (int wave0 = 0; wave0 < len; wave0 += S) {
    const int n = min(S, len - wave0);

    // 1. indices (and the pruning map, and weights) of this wave
    for (int r = gl; r < n; r += LPB) {
      const int64_t pos = start + wave0 + r;
      int64_t idx = load_int(p.indices, pos, idx64);
      long long off = -1;
      if (idx < 0 || idx >= p.data_size) {
        if (!((p.flags & (kSbFirst | kNoBag)) == kSbFirst && idx == -1)) {  // that layout's pruned row: skipped
          report(p.status, FBGEMM_B200_STATUS_BAD_INDEX, bag, pos, idx);
        }
      } else {
        if (pruned) {
          idx = __ldg(p.cit + idx);  // -1: pruned row, contributes nothing
        }
        if (idx >= 0) {
          off = idx * p.input_stride;
        }
      }
      s_off[r] = off;
      if (weighted) {
        s_w[r] = __ldg(p.weights + (positional ? (int64_t)(wave0 + r) : pos));
      }
    }
    __syncwarp(gmask);

    // 2. all rows of the wave in flight at once
    if (p.copy_width == 4) {
      stage_rows<4>(p, s_rows, s_off, n, gl, LPB);
    } else if (p.copy_width == 8) {
      stage_rows<8>(p, s_rows, s_off, n, gl, LPB);
    } else if (p.copy_width == 16) {
      stage_rows<16>(p, s_rows, s_off, n, gl, LPB);
    } else {
      stage_rows_bytewise(p, s_rows, s_off, n, gl, LPB);
    }
    cp_async_wait_all();
    __syncwarp(gmask);

    // 3. pool the staged rows in index order
    for (int r = 0; r < n; ++r) {
      if (s_off[r] < 0) {
        continue;
      }
      const uint8_t* srow = s_rows + r * p.pitch;
      float scale, bias;
      if (!half_sb) {
        scale = *reinterpret_cast<const float*>(srow + p.sb_off);
        bias = *reinterpret_cast<const float*>(srow + p.sb_off + 4);
      } else {
        const uint32_t sb = *reinterpret_cast<const uint32_t*>(srow + p.sb_off);
        scale = __half2float(__ushort_as_half((unsigned short)(sb & 0xffffu)));
        bias = __half2float(__ushort_as_half((unsigned short)(sb >> 16)));
      }
      if (weighted) {
        const float w = s_w[r];
        scale = __fmul_rn(w, scale);
        bias = __fmul_rn(w, bias);
      }
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci) {
        const int c = gl + ci * LPB;
        if (c < nchunks) {
          const uint32_t x = *reinterpret_cast<const uint32_t*>(srow + p.data_off + 4 * c);
          accumulate<BITS>(acc[ci], x, scale, bias);
        }
      }
    }
    __syncwarp(gmask);
  }

  if ((p.flags & kNormalize) && bag_len != 0) {
    const float inv = __fdiv_rn(1.f, (float)bag_len);
#pragma unroll
    for (int ci = 0; ci < CPL; ++ci) {
#pragma unroll
      for (int j = 0; j < COLS; ++j) {
        acc[ci][j] = __fmul_rn(acc[ci][j], inv);
      }
    }
  }

#pragma unroll
  for (int ci = 0; ci < CPL; ++ci) {
    const int c = gl + ci * LPB;
    if (c < nchunks) {
      store_chunk<COLS>(p, bag, c * COLS, acc[ci]);
    }
  }
}

using KernelFn = void (*)(const SpmdmParams);

struct Variant {
  KernelFn fn;
  int lpb;
  int cpl;
};

template <int BITS>
const Variant* variants(int* count) {
  if constexpr (BITS == 8) {
    static const Variant v[] = {
        {spmdm_kernel<8, 8, 1>, 8, 1},   {spmdm_kernel<8, 16, 1>, 16, 1}, {spmdm_kernel<8, 32, 1>, 32, 1},
        {spmdm_kernel<8, 8, 2>, 8, 2},   {spmdm_kernel<8, 16, 2>, 16, 2}, {spmdm_kernel<8, 32, 2>, 32, 2},
        {spmdm_kernel<8, 8, 4>, 8, 4},   {spmdm_kernel<8, 16, 4>, 16, 4}, {spmdm_kernel<8, 32, 4>, 32, 4},
        {spmdm_kernel<8, 32, 8>, 32, 8},
    };
    *count = sizeof(v) / sizeof(v[0]);
    return v;
  } else if constexpr (BITS == 4) {
    static const Variant v[] = {
        {spmdm_kernel<4, 8, 1>, 8, 1}, {spmdm_kernel<4, 16, 1>, 16, 1}, {spmdm_kernel<4, 32, 1>, 32, 1},
        {spmdm_kernel<4, 8, 2>, 8, 2}, {spmdm_kernel<4, 16, 2>, 16, 2}, {spmdm_kernel<4, 32, 2>, 32, 2},
        {spmdm_kernel<4, 8, 4>, 8, 4}, {spmdm_kernel<4, 16, 4>, 16, 4}, {spmdm_kernel<4, 32, 4>, 32, 4},
    };
    *count = sizeof(v) / sizeof(v[0]);
    return v;
  } else {
    static const Variant v[] = {
        {spmdm_kernel<2, 8, 1>, 8, 1}, {spmdm_kernel<2, 16, 1>, 16, 1}, {spmdm_kernel<2, 32, 1>, 32, 1},
        {spmdm_kernel<2, 8, 2>, 8, 2}, {spmdm_kernel<2, 16, 2>, 16, 2}, {spmdm_kernel<2, 32, 2>, 32, 2},
    };
    *count = sizeof(v) / sizeof(v[0]);
    return v;
  }
}

// Overrides of the variant choice exist only in tuning builds
// (-DFBGEMM_B200_TUNING, which also instantiates variants the dispatcher never
// picks); the product's launch path reads no environment variable.
#ifdef FBGEMM_B200_TUNING
int env_int(const char* name, int dflt) {
  const char* s = std::getenv(name);
  return (s && *s) ? std::atoi(s) : dflt;
}
#else
constexpr int env_int(const char*, int dflt) {
  return dflt;
}
#endif

}  // namespace

std::atomic<uint64_t> g_launch_count{0};
std::atomic<int> g_kernel_choice{FBGEMM_B200_KERNEL_AUTO};

int max_chunks_per_bag(int bit_rate) {
  return 32 * (bit_rate == 8 ? 8 : bit_rate == 4 ? 4 : 2);
}

// The variant of the direct kernel (spmdm_direct.cuh) for this call, or null
// when the rows do not allow 4- or 8-byte vector loads.
static const direct::Variant* pick_direct(const SpmdmParams& p, int bit_rate) {
  if (p.in_kind != 0) {
    return nullptr;  // not a quantized row format
  }
  const uintptr_t base = reinterpret_cast<uintptr_t>(p.table);
  auto divides = [&](int v) {
    return base % 4 == 0 && (base + p.data_row_off) % v == 0 && p.input_stride % v == 0 && p.data_bytes % v == 0;
  };
  // Row ids travel between lanes as 32-bit values and skipped rows read row 0.
  if (!divides(4) || p.data_bytes == 0 || p.data_size == 0 || p.data_size > 0xfffffffeLL ||
      p.input_stride > 0xffffffffLL) {
    return nullptr;
  }
  int vec = divides(8) ? 8 : 4;
  const int env_vec = env_int("FBGEMM_B200_VEC", 0);
  if (env_vec == 4) {
    vec = 4;
  }
  int count = 0;
  const direct::Variant* v = bit_rate == 8 ? direct_variants_8(&count)
      : bit_rate == 4                      ? direct_variants_4(&count)
                                           : direct_variants_2(&count);
  const int cpc = vec * 8 / bit_rate;      // columns per chunk
  const int nchunks = p.data_bytes / vec;
  int cpl_max = 0;
  for (int i = 0; i < count; ++i) {
    if (v[i].vec == vec && v[i].cpl > cpl_max) {
      cpl_max = v[i].cpl;
    }
  }
  // Columns per lane: narrow lane groups amortise the per-row work that does
  // not scale with D, wide ones keep registers (and so resident warps) in
  // check.  Measured best on B200: 32 columns for 8-bit rows, 16 for 4- and
  // 2-bit rows (whose unpacking needs more registers per column).
  // Rows of 256 and more 8-bit columns do better with 16 again (two bags per
  // warp instead of four: 67 against 73 ps per row at D = 256, the ragged bags
  // of a warp wait less for each other).
  const int cols_target = bit_rate == 8 ? (p.data_bytes >= 256 ? 16 : 32) : 16;
  int cpl_target = cols_target / cpc < 1 ? 1 : cols_target / cpc;
  cpl_target = cpl_target > cpl_max ? cpl_max : cpl_target;
  // At least 4 lanes per bag: with 2 (sixteen bags per warp) an 8-bit D=64
  // table measured 32 us per 16384-bag call against 25.5 us with 4.
  int lpb = 4;
  while (lpb < 32 && lpb * cpl_target < nchunks) {
    lpb *= 2;
  }
  int cpl = 1;
  while (lpb * cpl < nchunks) {
    cpl *= 2;
  }
  const int env_lpb = env_int("FBGEMM_B200_LPB", 0);
  const int env_cpl = env_int("FBGEMM_B200_CPL", 0);
  if (env_lpb > 0 && env_cpl > 0 && env_lpb * env_cpl >= nchunks) {
    lpb = env_lpb;
    cpl = env_cpl;
  }
  const direct::Variant* pick = nullptr;
  for (int i = 0; i < count; ++i) {
    if (v[i].vec == vec && v[i].lpb == lpb && v[i].cpl == cpl) {
      pick = &v[i];
    }
  }
  return pick;
}

// 1 when the row's payload is exactly the variant's LPB * CPL chunks.
static int direct_exact(const direct::Variant* v, const SpmdmParams& p) {
  return p.data_bytes == v->vec * v->lpb * v->cpl ? 1 : 0;
}

static int64_t direct_blocks(const direct::Variant* v, int64_t bags) {
  const int64_t bags_per_block = (int64_t)direct::kWarpsPerBlock * (32 / v->lpb);
  return (bags + bags_per_block - 1) / bags_per_block;
}

// One table, one launch; returns cudaErrorNotSupported when the direct kernel
// cannot take the rows.
static cudaError_t launch_direct(const SpmdmParams& p, int bit_rate, cudaStream_t stream) {
  const direct::Variant* pick = pick_direct(p, bit_rate);
  if (!pick) {
    return cudaErrorNotSupported;
  }
  const int64_t blocks = direct_blocks(pick, p.output_size);
  if (blocks <= 0 || blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  // Tables in which an index may name no row (a pruning map, or the layout in
  // which -1 is a pruned index) take the compacting kernel; the plain one has
  // no notion of a skipped row.
  const bool compact = (p.flags & (kPruned | kSbFirst)) || env_int("FBGEMM_B200_COMPACT", 0) == 1;
  const int exact = direct_exact(pick, p);
  (compact ? pick->compact[exact] : pick->fn[exact])<<<(unsigned)blocks, direct::kThreads, 0, stream>>>(p);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

// ---- several tables per launch --------------------------------------------------

MultiPlan::~MultiPlan() {
  for (int i = 0; i < kSideStreams; ++i) {
    if (side[i]) {
      cudaStreamDestroy(side[i]);
    }
    if (join[i]) {
      cudaEventDestroy(join[i]);
    }
  }
  if (fork) {
    cudaEventDestroy(fork);
  }
}

// Tables that share a kernel variant go into one launch (up to kMultiTables of
// them): their parameters travel as the kernel's argument and the grid is the
// sum of their blocks.  Tables the direct kernel cannot take keep a launch of
// their own.
cudaError_t build_multi_plan(const std::vector<SpmdmParams>& tables, const std::vector<int>& bit_rates, MultiPlan* plan) {
  std::vector<const direct::Variant*> variant(tables.size());
  std::vector<size_t> order;
  for (size_t t = 0; t < tables.size(); ++t) {
    variant[t] = tables[t].output_size > 0 ? pick_direct(tables[t], bit_rates[t]) : nullptr;
    if (tables[t].output_size <= 0) {
      continue;  // nothing to pool, nothing to store
    }
    if (variant[t]) {
      order.push_back(t);
    } else {
      plan->singles.push_back({tables[t], bit_rates[t]});
    }
  }
  // what decides a table's kernel besides the variant: 2 = rows may be skipped, 1 = exact-fit addressing
  auto form = [&](size_t t) {
    return ((tables[t].flags & (kPruned | kSbFirst)) != 0 ? 2 : 0) + direct_exact(variant[t], tables[t]);
  };
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
    return variant[a] != variant[b] ? variant[a] < variant[b] : form(a) < form(b);
  });
  for (size_t i = 0; i < order.size();) {
    const direct::Variant* v = variant[order[i]];
    const int f = form(order[i]);
    plan->groups.emplace_back();
    MultiPlan::Launch& g = plan->groups.back();
    g.fn = (f & 2) ? v->compact_multi[f & 1] : v->multi[f & 1];
    g.args = MultiArgs{};
    int64_t blocks = 0;
    for (; i < order.size() && variant[order[i]] == v && form(order[i]) == f && g.args.count < kMultiTables; ++i) {
      const int64_t b = direct_blocks(v, tables[order[i]].output_size);
      if (blocks + b > 0x7fffffffLL) {
        break;  // the rest of this variant's tables start a new launch
      }
      g.args.first_block[g.args.count] = (int32_t)blocks;
      g.args.t[g.args.count] = tables[order[i]];
      blocks += b;
      ++g.args.count;
    }
    if (g.args.count == 0) {
      return cudaErrorInvalidValue;  // a single table with more than 2^31 blocks
    }
    g.args.first_block[g.args.count] = (int32_t)blocks;
    g.blocks = (unsigned)blocks;
  }
  // largest grid first: the short launches fill the tail of the long ones
  std::stable_sort(plan->groups.begin(), plan->groups.end(),
                   [](const MultiPlan::Launch& a, const MultiPlan::Launch& b) { return a.blocks > b.blocks; });
  if (plan->groups.size() + plan->singles.size() > 1) {
    cudaError_t e = cudaEventCreateWithFlags(&plan->fork, cudaEventDisableTiming);
    for (int i = 0; i < MultiPlan::kSideStreams && e == cudaSuccess; ++i) {
      e = cudaStreamCreateWithFlags(&plan->side[i], cudaStreamNonBlocking);
      if (e == cudaSuccess) {
        e = cudaEventCreateWithFlags(&plan->join[i], cudaEventDisableTiming);
      }
    }
    if (e != cudaSuccess) {
      return e;
    }
  }
  return cudaSuccess;
}

cudaError_t launch_multi_plan(const MultiPlan& plan, cudaStream_t stream) {
  const size_t launches = plan.groups.size() + plan.singles.size();
  const bool spread = launches > 1 && plan.fork;
  cudaError_t e = cudaSuccess;
  if (spread) {
    e = cudaEventRecord(plan.fork, stream);
    for (int i = 0; i < MultiPlan::kSideStreams && e == cudaSuccess; ++i) {
      e = cudaStreamWaitEvent(plan.side[i], plan.fork, 0);
    }
    if (e != cudaSuccess) {
      return e;
    }
  }
  size_t n = 0;  // launch n goes to the caller's stream (n % 4 == 0) or to side stream n % 4 - 1
  auto stream_of = [&](size_t i) {
    const size_t k = i % (MultiPlan::kSideStreams + 1);
    return (!spread || k == 0) ? stream : plan.side[k - 1];
  };
  for (const MultiPlan::Launch& g : plan.groups) {
    g.fn<<<g.blocks, direct::kThreads, 0, stream_of(n++)>>>(g.args);
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
      return e;
    }
  }
  for (const auto& single : plan.singles) {
    e = launch_spmdm(single.first, single.second, stream_of(n++));
    if (e != cudaSuccess) {
      return e;
    }
  }
  if (spread) {
    for (int i = 0; i < MultiPlan::kSideStreams && e == cudaSuccess; ++i) {
      e = cudaEventRecord(plan.join[i], plan.side[i]);
      if (e == cudaSuccess) {
        e = cudaStreamWaitEvent(stream, plan.join[i], 0);
      }
    }
  }
  return e;
}

cudaError_t launch_spmdm(const SpmdmParams& p_in, int bit_rate, cudaStream_t stream) {
  if (p_in.in_kind != 0) {
    return launch_plain_rows(p_in, stream);
  }
  const bool staged_only = g_kernel_choice.load(std::memory_order_relaxed) == FBGEMM_B200_KERNEL_GENERIC;
  if (!staged_only) {
    const cudaError_t e = launch_direct(p_in, bit_rate, stream);
    if (e != cudaErrorNotSupported) {
      return e;
    }
  }
  SpmdmParams p = p_in;
  int count = 0;
  const Variant* v = bit_rate == 8 ? variants<8>(&count) : bit_rate == 4 ? variants<4>(&count) : variants<2>(&count);
  const int nchunks = (p.data_bytes + 3) / 4;

  // Smallest lane group that covers the payload with one chunk per lane; wide
  // rows take a full warp and several chunks per lane.
  int want_lpb = nchunks <= 8 ? 8 : nchunks <= 16 ? 16 : 32;
  int want_cpl = 1;
  while (want_lpb * want_cpl < nchunks) {
    want_cpl *= 2;
  }
  const int env_lpb = env_int("FBGEMM_B200_LPB", 0);
  const int env_cpl = env_int("FBGEMM_B200_CPL", 0);
  if (env_lpb > 0 && env_cpl > 0 && env_lpb * env_cpl >= nchunks) {
    want_lpb = env_lpb;
    want_cpl = env_cpl;
  }
  const Variant* pick = nullptr;
  for (int i = 0; i < count; ++i) {
    if (v[i].lpb == want_lpb && v[i].cpl == want_cpl) {
      pick = &v[i];
    }
  }
  if (!pick) {
    return cudaErrorInvalidValue;
  }

  // Shared-memory stage: per bag slot `rows_per_wave` rows, their byte offsets
  // (8 B) and weights (4 B).
  const int gpw = 32 / pick->lpb;
  const int warp_budget = env_int("FBGEMM_B200_SMEM_PER_WARP", 6144);
  const int max_rows = env_int("FBGEMM_B200_WAVE_ROWS", 64);
  int rows = (warp_budget / gpw) / (p.pitch + 12);
  rows = rows < 1 ? 1 : rows > max_rows ? max_rows : rows;
  p.rows_per_wave = rows;
  p.group_smem = ((((rows * p.pitch + 15) & ~15) + rows * 12) + 15) & ~15;
  const size_t smem = (size_t)p.group_smem * gpw * kWarpsPerBlock;
  if (smem > 200 * 1024) {
    return cudaErrorInvalidValue;
  }
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(pick->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      return e;
    }
  }
  const int64_t bags_per_block = (int64_t)kWarpsPerBlock * gpw;
  const int64_t blocks = (p.output_size + bags_per_block - 1) / bags_per_block;
  if (blocks <= 0 || blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  pick->fn<<<(unsigned)blocks, kThreads, smem, stream>>>(p);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

// The fast lookup kernel: rows go from HBM/L2 straight into registers.
//
// Same arithmetic as the staged kernel in spmdm_kernels.cu (and therefore as
// the scalar reference, src/RefImplementations.cc:1290-1346, :1485-1541,
// :1746-1822): per output column, rows strictly in index order,
// acc = fma(w*scale, q, acc + w*bias).  What differs is how the work is laid
// out, because the lookup turned out to be bound by instruction issue, not by
// HBM, once enough rows are in flight:
//
//  * A bag belongs to a group of LPB lanes (4..32); each lane owns CPL
//    "chunks" of VEC bytes of the packed payload, i.e. up to 32 columns kept in
//    registers as 16 fp32x2 pairs.  Narrow groups mean the per-row work that
//    does not scale with D (index fetch, bounds check, address, scale/bias,
//    weight) is paid by few lanes while 32/LPB bags advance per warp
//    instruction.
//  * No shared-memory stage.  The work per row that is independent of the
//    column (index fetch, range check, pruning map, weight) is done by one
//    lane of the group per row and broadcast by shuffle; every lane then issues
//    its own VEC loads for U rows back to back, so U rows per bag (U * 32/LPB
//    per warp) are in flight before the first use, and the indices of the next
//    step are fetched before the arithmetic of the current one.
//  * The two roundings per column per row are done two columns at a time with
//    the packed fp32 instructions of sm_100 (add.rn.f32x2, fma.rn.f32x2), which
//    round each half exactly like the scalar instructions.
//  * Integer -> float: each byte / nibble / crumb is planted with one prmt in
//    the mantissa of 2^23 and 2^23 is subtracted (packed as well).
//
// Three kernels share that block-level code:
//   spmdm_direct_kernel          one table per launch, parameters in constant
//                                memory;
//   spmdm_direct_multi_kernel    several tables of one row format per launch,
//                                each block finding its table in an index array;
//   spmdm_direct_compact_kernel  row-wise sparse tables: the rows that survive
//                                the pruning map are first compacted into a
//                                shared-memory queue, so that only rows that
//                                exist reach the arithmetic.
//
// Requirements (checked by the dispatcher): table address, row pitch and
// payload width are multiples of VEC (4 or 8 bytes).  Everything else takes
// the staged kernel.
#pragma once

#include <cuda_fp16.h>

#include "internal.h"

namespace fbgemm_b200 {
namespace direct {

constexpr int kWarpsPerBlock = 4;
constexpr int kThreads = kWarpsPerBlock * 32;

using u64 = unsigned long long;

__device__ __forceinline__ u64 pack2(float lo, float hi) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(u64 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 add2(u64 a, u64 b) {
  u64 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
  u64 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
  u64 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// Bytes I of xa and J of xb as the fp32 pair (2^23 + byte, 2^23 + byte).
template <int I, int J>
__device__ __forceinline__ u64 magic_pair(uint32_t xa, uint32_t xb) {
  return pack2(
      __uint_as_float(__byte_perm(xa, 0x4B000000u, 0x7540u | I)),
      __uint_as_float(__byte_perm(xb, 0x4B000000u, 0x7540u | J)));
}

// acc = fma(scale, q, acc + bias) on a pair of columns; `m` holds 2^23 + q.
__device__ __forceinline__ u64 pool2(u64 acc, u64 m, u64 scale2, u64 bias2, u64 neg_magic2) {
  return fma2(scale2, add2(m, neg_magic2), add2(acc, bias2));
}

// One 32-bit word of packed payload into 32/BITS columns = 16/BITS pairs.
template <int BITS>
__device__ __forceinline__ void accumulate_word(u64* acc, uint32_t x, u64 s2, u64 b2, u64 nm2) {
  if constexpr (BITS == 8) {
    acc[0] = pool2(acc[0], magic_pair<0, 1>(x, x), s2, b2, nm2);
    acc[1] = pool2(acc[1], magic_pair<2, 3>(x, x), s2, b2, nm2);
  } else if constexpr (BITS == 4) {
    // element 2k = low nibble of byte k, element 2k+1 = high nibble
    const uint32_t lo = x & 0x0F0F0F0Fu;
    const uint32_t hi = (x >> 4) & 0x0F0F0F0Fu;
    acc[0] = pool2(acc[0], magic_pair<0, 0>(lo, hi), s2, b2, nm2);
    acc[1] = pool2(acc[1], magic_pair<1, 1>(lo, hi), s2, b2, nm2);
    acc[2] = pool2(acc[2], magic_pair<2, 2>(lo, hi), s2, b2, nm2);
    acc[3] = pool2(acc[3], magic_pair<3, 3>(lo, hi), s2, b2, nm2);
  } else {
    // element 4k+i = bits [2i+1:2i] of byte k
    const uint32_t t0 = x & 0x03030303u;
    const uint32_t t1 = (x >> 2) & 0x03030303u;
    const uint32_t t2 = (x >> 4) & 0x03030303u;
    const uint32_t t3 = (x >> 6) & 0x03030303u;
    acc[0] = pool2(acc[0], magic_pair<0, 0>(t0, t1), s2, b2, nm2);
    acc[1] = pool2(acc[1], magic_pair<0, 0>(t2, t3), s2, b2, nm2);
    acc[2] = pool2(acc[2], magic_pair<1, 1>(t0, t1), s2, b2, nm2);
    acc[3] = pool2(acc[3], magic_pair<1, 1>(t2, t3), s2, b2, nm2);
    acc[4] = pool2(acc[4], magic_pair<2, 2>(t0, t1), s2, b2, nm2);
    acc[5] = pool2(acc[5], magic_pair<2, 2>(t2, t3), s2, b2, nm2);
    acc[6] = pool2(acc[6], magic_pair<3, 3>(t0, t1), s2, b2, nm2);
    acc[7] = pool2(acc[7], magic_pair<3, 3>(t2, t3), s2, b2, nm2);
  }
}

template <int VEC>
struct Vec;
template <>
struct Vec<4> {
  uint32_t w[1];
  __device__ __forceinline__ void load(const uint8_t* p) { w[0] = __ldg(reinterpret_cast<const uint32_t*>(p)); }
};
template <>
struct Vec<8> {
  uint32_t w[2];
  __device__ __forceinline__ void load(const uint8_t* p) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    w[0] = v.x;
    w[1] = v.y;
  }
};

// Raw scale,bias bits of one row: an fp32 pair for 8-bit rows with scale,bias
// last, an fp16 pair otherwise (`half_sb`; always true for 4- and 2-bit rows).
template <int BITS, int VEC>
struct ScaleBias {
  uint32_t raw[BITS == 8 ? 2 : 1];
  __device__ __forceinline__ void load(const uint8_t* p, bool half_sb) {
    if constexpr (BITS != 8) {
      raw[0] = __ldg(reinterpret_cast<const uint32_t*>(p));
    } else {
      if (half_sb) {
        raw[0] = __ldg(reinterpret_cast<const uint32_t*>(p));
        raw[1] = 0;
      } else if constexpr (VEC >= 8) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
        raw[0] = v.x;
        raw[1] = v.y;
      } else {
        raw[0] = __ldg(reinterpret_cast<const uint32_t*>(p));
        raw[1] = __ldg(reinterpret_cast<const uint32_t*>(p + 4));
      }
    }
  }
  __device__ __forceinline__ void get(float& scale, float& bias, bool half_sb) const {
    if (BITS != 8 || half_sb) {
      scale = __half2float(__ushort_as_half((unsigned short)(raw[0] & 0xffffu)));
      bias = __half2float(__ushort_as_half((unsigned short)(raw[0] >> 16)));
    } else {
      scale = __uint_as_float(raw[0]);
      bias = __uint_as_float(raw[BITS == 8 ? 1 : 0]);
    }
  }
};

__device__ __forceinline__ int64_t load_int(const void* p, int64_t i, bool is64) {
  return is64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(p) + i)
              : (int64_t)__ldg(reinterpret_cast<const int*>(p) + i);
}

static __device__ __noinline__ void report(int32_t* st, int code, int64_t bag, int64_t pos, int64_t val) {
  if (atomicCAS(st, 0, code) == 0) {
    st[1] = (int32_t)bag;
    st[2] = (int32_t)pos;
    st[3] = (int32_t)val;
  }
}

// base + row * stride as one 32 x 32 -> 64-bit multiply-add.
__device__ __forceinline__ const uint8_t* row_address(const uint8_t* base, uint32_t row, uint32_t stride) {
  unsigned long long a;
  asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(a) : "r"(row), "r"(stride), "l"(base));
  return reinterpret_cast<const uint8_t*>(a);
}

// The per-row work that does not depend on the column - index fetch, range
// check, weight fetch - is done once per row by ONE lane of the bag's group:
// in a step of U rows, lane gl resolves rows gl, gl+LPB, ...  The results
// reach the other lanes of the group by shuffle in pool_step.  This kernel
// sees dense tables only (tables with a pruning map, or whose layout makes -1
// a pruned index, take direct_block_compact), so every index names a row to
// pool; an index out of range is reported and replaced by row 0 - the call
// returns false and its output is unspecified, as with the reference.
template <int LPB, int U>
__device__ __forceinline__ void fetch_rows(
    const SpmdmParams& p,
    int gl,
    int64_t bag,
    int64_t pos0,
    int r0,
    uint32_t (&id)[(U + LPB - 1) / LPB],
    float (&w)[(U + LPB - 1) / LPB]) {
  constexpr int OWN = (U + LPB - 1) / LPB;
#pragma unroll
  for (int j = 0; j < OWN; ++j) {
    const int u = gl + j * LPB;
    id[j] = 0u;
    w[j] = 0.f;
    if (u < U) {
      const int64_t pos = pos0 + u;
      const int64_t idx = load_int(p.indices, pos, p.flags & kIdx64);
      if ((unsigned long long)idx >= (unsigned long long)p.data_size) {
        report(p.status, FBGEMM_B200_STATUS_BAD_INDEX, bag, pos, idx);
      } else {
        id[j] = (uint32_t)idx;
      }
      if (p.flags & kWeighted) {
        w[j] = __ldg(p.weights + ((p.flags & kPositional) ? (int64_t)(r0 + u) : pos));
      }
    }
  }
}

// One step: U rows of the bag.  All row loads are issued before the first
// use; then the rows are pooled in order.
// Where a lane finds its payload chunks.  EXACT: the row's payload is exactly
// LPB * CPL chunks, so chunk ci of the lane lies ci * LPB * VEC bytes after its
// first one: one address computation per row, the CPL loads differ by
// immediate offsets, and one pointer is kept instead of CPL.  Otherwise lanes
// whose chunk lies beyond the payload (row width not a multiple of LPB * CPL
// chunks) read chunk 0 instead and simply do not store.
template <int VEC, int LPB, int CPL, bool EXACT>
struct LaneChunks {
  const uint8_t* base[EXACT ? 1 : CPL];  // table + payload offset + byte offset of this lane's chunk ci
  __device__ __forceinline__ void init(const uint8_t* data_base, int gl, int nchunks) {
    if constexpr (EXACT) {
      base[0] = data_base + gl * VEC;
    } else {
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci) {
        const int c = gl + ci * LPB;
        base[ci] = data_base + (c < nchunks ? c * VEC : 0);
      }
    }
  }
  // the CPL chunks of row `row` into d[0..CPL)
  __device__ __forceinline__ void load_row(Vec<VEC> (&d)[CPL], uint32_t row, uint32_t stride) const {
    if constexpr (EXACT) {
      const uint8_t* r = row_address(base[0], row, stride);
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci) {
        d[ci].load(r + ci * LPB * VEC);
      }
    } else {
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci) {
        d[ci].load(row_address(base[ci], row, stride));
      }
    }
  }
};

template <int BITS, int VEC, int LPB, int CPL, int U, bool EXACT>
__device__ __forceinline__ void pool_step(
    const LaneChunks<VEC, LPB, CPL, EXACT>& lc,
    const uint8_t* sb_base,                   // table + data_bytes
    uint32_t stride,
    unsigned gmask,
    int lane0,  // first lane of the group
    bool half_sb,
    bool weighted,
    const uint32_t (&id_own)[(U + LPB - 1) / LPB],
    const float (&w_own)[(U + LPB - 1) / LPB],
    u64 (&acc)[CPL][(VEC / 4) * (16 / BITS)]) {
  constexpr int PAIRS_PER_WORD = 16 / BITS;
  uint32_t rid[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    rid[u] = LPB == 1 ? id_own[u] : __shfl_sync(gmask, id_own[u / LPB], lane0 + (u % LPB));
  }
  Vec<VEC> d[U][CPL];
  ScaleBias<BITS, VEC> sb[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    lc.load_row(d[u], rid[u], stride);
    sb[u].load(row_address(sb_base, rid[u], stride), half_sb);
  }
  const u64 nm2 = pack2(-8388608.0f, -8388608.0f);
#pragma unroll
  for (int u = 0; u < U; ++u) {
    float scale, bias;
    sb[u].get(scale, bias, half_sb);
    if (weighted) {
      const float w = LPB == 1 ? w_own[u] : __shfl_sync(gmask, w_own[u / LPB], lane0 + (u % LPB));
      scale = __fmul_rn(w, scale);
      bias = __fmul_rn(w, bias);
    }
    const u64 s2 = pack2(scale, scale);
    const u64 b2 = pack2(bias, bias);
#pragma unroll
    for (int ci = 0; ci < CPL; ++ci) {
#pragma unroll
      for (int wd = 0; wd < VEC / 4; ++wd) {
        accumulate_word<BITS>(&acc[ci][wd * PAIRS_PER_WORD], d[u][ci].w[wd], s2, b2, nm2);
      }
    }
  }
}

// fp32 -> fp16 (round to nearest even, cpu_float2half_rn) or bf16 the way the
// reference does it: (bits + 0x8000) >> 16 (cpu_float2bfloat16,
// include/fbgemm/FloatConversion.h:312-315).
__device__ __forceinline__ uint16_t to_16bit(float v, bool bf16) {
  return bf16 ? (uint16_t)((__float_as_uint(v) + 0x8000u) >> 16) : __half_as_ushort(__float2half_rn(v));
}

// Store CPC consecutive columns starting at col0 of output row `bag`.
template <int CPC>
__device__ __forceinline__ void store_columns(const SpmdmParams& p, int64_t bag, int col0, const u64* pairs) {
  float v[CPC];
#pragma unroll
  for (int i = 0; i < CPC / 2; ++i) {
    unpack2(pairs[i], v[2 * i], v[2 * i + 1]);
  }
  const bool full = col0 + CPC <= p.block_size;
  if (p.flags & (kOutHalf | kOutBf16)) {
    const bool bf16 = p.flags & kOutBf16;
    uint16_t* o = reinterpret_cast<uint16_t*>(output_row(p, bag, 2)) + col0;
    if (full && (p.flags & kOutVec)) {
      uint32_t h[CPC / 2];
#pragma unroll
      for (int i = 0; i < CPC / 2; ++i) {
        h[i] = (uint32_t)to_16bit(v[2 * i], bf16) | ((uint32_t)to_16bit(v[2 * i + 1], bf16) << 16);
      }
      if constexpr (CPC == 4) {
        *(reinterpret_cast<uint2*>(o)) = make_uint2(h[0], h[1]);
      } else {
#pragma unroll
        for (int i = 0; i < CPC / 8; ++i) {
          *(reinterpret_cast<uint4*>(o) + i) = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < CPC; ++i) {
        if (col0 + i < p.block_size) {
          o[i] = to_16bit(v[i], bf16);
        }
      }
    }
  } else {
    float* o = reinterpret_cast<float*>(output_row(p, bag, 4)) + col0;
    if (full && (p.flags & kOutVec)) {
#pragma unroll
      for (int i = 0; i < CPC / 4; ++i) {
        *(reinterpret_cast<float4*>(o) + i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < CPC; ++i) {
        if (col0 + i < p.block_size) {
          o[i] = v[i];
        }
      }
    }
  }
}

// The work of one thread block: block `block` of the launch that covers the
// bags of `p` (32/LPB bags per warp, kWarpsPerBlock warps).
template <int BITS, int VEC, int LPB, int CPL, bool EXACT>
__device__ __forceinline__ void direct_block(const SpmdmParams& p, int64_t block) {
  constexpr int GPW = 32 / LPB;                       // bags per warp
  constexpr int CPC = VEC * 8 / BITS;                 // columns per chunk
  constexpr int PAIRS = (VEC / 4) * (16 / BITS);      // fp32x2 pairs per chunk
  // Rows per step.  Measured on B200: 4 beats 2, 8 and 16 for every row format
  // (more rows per step cost registers, hence resident warps, and that costs
  // more than the extra loads in flight per warp bring).
  constexpr int UMAX = 4;
  constexpr int OWN = (UMAX + LPB - 1) / LPB;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int grp = lane / LPB;
  const int gl = lane % LPB;
  const int lane0 = grp * LPB;
  const unsigned gmask = LPB == 32 ? 0xffffffffu : (((1u << LPB) - 1u) << lane0);
  const bool off64 = p.flags & kOff64;
  const bool weighted = p.flags & kWeighted;

  const bool no_bag = p.flags & kNoBag;
  // rebasing to offsets[0] (the functor's convention) unless the offsets are absolute
  const bool rebase = !(p.flags & (kNoBag | kAbsOffsets));
  const int64_t off_base = rebase ? load_int(p.offsets, 0, off64) : 0;
  if (block == 0 && threadIdx.x == 0 && rebase) {
    // `return current == index_size` of the reference
    const int64_t total = load_int(p.offsets, p.output_size, off64) - off_base;
    if (total != p.index_size) {
      report(p.status, FBGEMM_B200_STATUS_SIZE_MISMATCH, p.output_size, total, p.index_size);
    }
  }
  const int64_t bag = (block * kWarpsPerBlock + warp) * GPW + grp;
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

  // Lanes whose chunk lies beyond the payload (row width not a multiple of
  // LPB*CPL chunks) read chunk 0 instead and simply do not store.
  const int nchunks = p.data_bytes / VEC;
  LaneChunks<VEC, LPB, CPL, EXACT> lc;
  lc.init(p.table + p.data_row_off, gl, nchunks);
  const uint8_t* sb_base = p.table + p.sb_row_off;
  const bool half_sb = BITS != 8 || (p.flags & kSbFirst);
  const uint32_t stride = (uint32_t)p.input_stride;

  u64 acc[CPL][PAIRS];
#pragma unroll
  for (int ci = 0; ci < CPL; ++ci) {
#pragma unroll
    for (int j = 0; j < PAIRS; ++j) {
      acc[ci][j] = 0ull;  // (+0.f, +0.f)
    }
  }

  // Full steps of UMAX rows.  The lane that resolves a row works two steps
  // ahead of the arithmetic so that nothing waits on a load that was only just
  // issued: while step s is pooled, the indices and weights of step s+2 are in
  // flight and those of step s+1 have landed.
  const int nfull = len / UMAX;
  const bool idx64 = p.flags & kIdx64;
  const bool positional = p.flags & kPositional;
  // loads only: raw index and weight of this lane's rows of step s
  auto issue = [&](int s, long long (&raw)[OWN], float (&w)[OWN]) {
#pragma unroll
    for (int j = 0; j < OWN; ++j) {
      const int u = gl + j * LPB;
      raw[j] = 0;
      w[j] = 0.f;
      if (u < UMAX && s < nfull) {
        const int64_t pos = start + (int64_t)s * UMAX + u;
        raw[j] = load_int(p.indices, pos, idx64);
        if (weighted) {
          w[j] = __ldg(p.weights + (positional ? (int64_t)(s * UMAX + u) : pos));
        }
      }
    }
  };
  // range check (an index out of range is reported and row 0 pooled in its place)
  auto resolve = [&](int s, const long long (&raw)[OWN], uint32_t (&id)[OWN]) {
#pragma unroll
    for (int j = 0; j < OWN; ++j) {
      const int u = gl + j * LPB;
      id[j] = 0u;
      if (u < UMAX && s < nfull) {
        if ((unsigned long long)raw[j] >= (unsigned long long)p.data_size) {
          report(p.status, FBGEMM_B200_STATUS_BAD_INDEX, bag, start + (int64_t)s * UMAX + u, raw[j]);
        } else {
          id[j] = (uint32_t)raw[j];
        }
      }
    }
  };
  long long raw_1[OWN], raw_2[OWN];
  uint32_t id_cur[OWN], id_1[OWN];
  float w_cur[OWN], w_1[OWN], w_2[OWN];
  issue(0, raw_1, w_cur);
  issue(1, raw_2, w_1);
  resolve(0, raw_1, id_cur);
#pragma unroll
  for (int j = 0; j < OWN; ++j) {
    raw_1[j] = raw_2[j];
  }
#pragma unroll 1
  for (int s = 0; s < nfull; ++s) {
    issue(s + 2, raw_2, w_2);
    resolve(s + 1, raw_1, id_1);
    pool_step<BITS, VEC, LPB, CPL, UMAX, EXACT>(lc, sb_base, stride, gmask, lane0, half_sb, weighted, id_cur, w_cur, acc);
#pragma unroll
    for (int j = 0; j < OWN; ++j) {
      id_cur[j] = id_1[j];
      w_cur[j] = w_1[j];
      w_1[j] = w_2[j];
      raw_1[j] = raw_2[j];
    }
  }
  // The remaining rows, largest power of two first (each such step is full).
  int r = nfull * UMAX;
  if (len - r >= 2) {
    uint32_t id2[(2 + LPB - 1) / LPB];
    float w2[(2 + LPB - 1) / LPB];
    fetch_rows<LPB, 2>(p, gl, bag, start + r, r, id2, w2);
    pool_step<BITS, VEC, LPB, CPL, 2, EXACT>(lc, sb_base, stride, gmask, lane0, half_sb, weighted, id2, w2, acc);
    r += 2;
  }
  if (len - r >= 1) {
    uint32_t id1[1];
    float w1[1];
    fetch_rows<LPB, 1>(p, gl, bag, start + r, r, id1, w1);
    pool_step<BITS, VEC, LPB, CPL, 1, EXACT>(lc, sb_base, stride, gmask, lane0, half_sb, weighted, id1, w1, acc);
  }

  if ((p.flags & kNormalize) && bag_len != 0) {
    const float inv = __fdiv_rn(1.f, (float)bag_len);
    const u64 inv2 = pack2(inv, inv);
#pragma unroll
    for (int ci = 0; ci < CPL; ++ci) {
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        acc[ci][j] = mul2(acc[ci][j], inv2);
      }
    }
  }
#pragma unroll
  for (int ci = 0; ci < CPL; ++ci) {
    const int c = gl + ci * LPB;
    if (c < nchunks) {
      store_columns<CPC>(p, bag, c * CPC, acc[ci]);
    }
  }
}

// U rows whose ids (none skipped) every lane of the group already holds: the
// registers they occupy while in flight, all row loads issued together, and
// the rows pooled in order with weights given as fp32 bit patterns.
template <int BITS, int VEC, int CPL, int U>
struct KnownRows {
  Vec<VEC> d[U][CPL];
  ScaleBias<BITS, VEC> sb[U];

  template <int LPB, bool EXACT>
  __device__ __forceinline__ void load(const LaneChunks<VEC, LPB, CPL, EXACT>& lc, const uint8_t* sb_base,
                                       uint32_t stride, bool half_sb, const uint2* entry) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      lc.load_row(d[u], entry[u].x, stride);
      sb[u].load(row_address(sb_base, entry[u].x, stride), half_sb);
    }
  }

  __device__ __forceinline__ void pool(bool half_sb, bool weighted, const uint2* entry,
                                       u64 (&acc)[CPL][(VEC / 4) * (16 / BITS)]) const {
    constexpr int PAIRS_PER_WORD = 16 / BITS;
    const u64 nm2 = pack2(-8388608.0f, -8388608.0f);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float scale, bias;
      sb[u].get(scale, bias, half_sb);
      if (weighted) {
        const float w = __uint_as_float(entry[u].y);
        scale = __fmul_rn(w, scale);
        bias = __fmul_rn(w, bias);
      }
      const u64 s2 = pack2(scale, scale);
      const u64 b2 = pack2(bias, bias);
#pragma unroll
      for (int ci = 0; ci < CPL; ++ci) {
#pragma unroll
        for (int wd = 0; wd < VEC / 4; ++wd) {
          accumulate_word<BITS>(&acc[ci][wd * PAIRS_PER_WORD], d[u][ci].w[wd], s2, b2, nm2);
        }
      }
    }
  }
};

// The block's work for tables in which an index may name no row: row-wise
// sparse tables (a pruning map) and the table-batched layout (-1 = pruned).
// Pooling such a row with zeros would cost the arithmetic of a real one,
// because the lanes of a warp move together.  Here a group first
// walks a stretch of its bag's indices (a queue length at a time), resolves them
// through the pruning map and writes the rows that remain, with their weights,
// in order into a small queue in shared memory; then it pools the queue four
// rows at a time.  Only rows that exist reach the arithmetic.
// Queue entries per lane group: 8 KB of shared memory per block whatever the
// group width (fewer, wider groups get longer queues), 128 entries at most.
constexpr int kQueueBytes = 8192;
__host__ __device__ constexpr int queue_entries(int groups_per_warp) {
  const int q = kQueueBytes / (kWarpsPerBlock * groups_per_warp * 8);
  return q > 128 ? 128 : q;
}

template <int BITS, int VEC, int LPB, int CPL, bool EXACT>
__device__ __forceinline__ void direct_block_compact(const SpmdmParams& p, int64_t block) {
  constexpr int GPW = 32 / LPB;
  constexpr int CPC = VEC * 8 / BITS;
  constexpr int PAIRS = (VEC / 4) * (16 / BITS);
  constexpr int kQueue = queue_entries(GPW);
  // rows of the next step in flight during the arithmetic: only where a row is
  // at most two words per lane, or the extra registers cost resident warps
  constexpr bool kPrefetch = CPL * (VEC / 4) <= 2;
  __shared__ uint2 queue_s[kWarpsPerBlock * GPW][kQueue];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int grp = lane / LPB;
  const int gl = lane % LPB;
  const int lane0 = grp * LPB;
  const unsigned gmask = LPB == 32 ? 0xffffffffu : (((1u << LPB) - 1u) << lane0);
  const bool off64 = p.flags & kOff64;
  const bool idx64 = p.flags & kIdx64;
  const bool weighted = p.flags & kWeighted;
  const bool positional = p.flags & kPositional;
  const bool pruned = p.flags & kPruned;
  const bool minus_one_skips = (p.flags & (kSbFirst | kNoBag)) == kSbFirst;
  const bool half_sb = BITS != 8 || (p.flags & kSbFirst);
  uint2* queue = queue_s[warp * GPW + grp];

  const bool rebase = !(p.flags & (kNoBag | kAbsOffsets));
  const int64_t off_base = rebase ? load_int(p.offsets, 0, off64) : 0;
  if (block == 0 && threadIdx.x == 0 && rebase) {
    const int64_t total = load_int(p.offsets, p.output_size, off64) - off_base;
    if (total != p.index_size) {
      report(p.status, FBGEMM_B200_STATUS_SIZE_MISMATCH, p.output_size, total, p.index_size);
    }
  }
  const int64_t bag = (block * kWarpsPerBlock + warp) * GPW + grp;
  if (bag >= p.output_size) {
    return;
  }
  // no_bag: output row m is the single row indices[m] (there are no offsets)
  const bool no_bag = p.flags & kNoBag;
  const int64_t o0 = no_bag ? bag : load_int(p.offsets, bag, off64);
  const int64_t o1 = no_bag ? bag + 1 : load_int(p.offsets, bag + 1, off64);
  const int64_t start = o0 - off_base;
  const int bag_len = (int)(o1 - o0);
  int len = bag_len < 0 ? 0 : bag_len;
  if (bag_len < 0 || start < 0 || start + len > p.index_size) {
    if (gl == 0) {
      report(p.status, FBGEMM_B200_STATUS_BAG_OVERRUN, bag, start, len);
    }
    len = 0;
  }

  const int nchunks = p.data_bytes / VEC;
  LaneChunks<VEC, LPB, CPL, EXACT> lc;
  lc.init(p.table + p.data_row_off, gl, nchunks);
  const uint8_t* sb_base = p.table + p.sb_row_off;
  const uint32_t stride = (uint32_t)p.input_stride;

  u64 acc[CPL][PAIRS];
#pragma unroll
  for (int ci = 0; ci < CPL; ++ci) {
#pragma unroll
    for (int j = 0; j < PAIRS; ++j) {
      acc[ci][j] = 0ull;
    }
  }

  for (int c0 = 0; c0 < len; c0 += kQueue) {
    const int nc = min(kQueue, len - c0);
    // 1. resolve: lane gl takes candidates gl, gl + LPB, ...; the index of
    // round k+2 and the map entry of round k+1 are in flight while round k is
    // compacted into the queue.
    const int rounds = (nc + LPB - 1) / LPB;
    auto fetch_index = [&](int k) -> long long {
      const int c = k * LPB + gl;
      return c < nc ? load_int(p.indices, start + c0 + c, idx64) : -2;
    };
    // row id after the range check and the pruning map; negative = nothing to pool
    auto resolve = [&](int k, long long raw) -> int32_t {
      const int c = k * LPB + gl;
      if (c >= nc) {
        return -1;
      }
      if ((unsigned long long)raw >= (unsigned long long)p.data_size) {
        if (!(minus_one_skips && raw == -1)) {
          report(p.status, FBGEMM_B200_STATUS_BAD_INDEX, bag, start + c0 + c, raw);
        }
        return -1;
      }
      return pruned ? __ldg(p.cit + raw) : (int32_t)raw;
    };
    long long raw_1 = fetch_index(1);
    int32_t id_0 = resolve(0, fetch_index(0));
    int count = 0;
    for (int k = 0; k < rounds; ++k) {
      const long long raw_2 = fetch_index(k + 2);
      const int32_t id_1 = resolve(k + 1, raw_1);
      const int c = k * LPB + gl;
      float w = 0.f;
      if (weighted && c < nc) {
        w = __ldg(p.weights + (positional ? (int64_t)(c0 + c) : start + c0 + c));
      }
      const bool keep = id_0 >= 0;
      const unsigned kept = (__ballot_sync(gmask, keep) >> lane0) & (LPB == 32 ? 0xffffffffu : ((1u << LPB) - 1u));
      if (keep) {
        queue[count + __popc(kept & ((1u << gl) - 1u))] = make_uint2((uint32_t)id_0, __float_as_uint(w));
      }
      count += __popc(kept);
      id_0 = id_1;
      raw_1 = raw_2;
    }
    __syncwarp(gmask);
    // 2. pool the queue in order, four rows at a time.  The ids of every step
    // are known, so (where the registers allow) the rows of the next step are
    // requested before the current ones are pooled.
    const int nfull = count / 4;
    if constexpr (kPrefetch) {
      KnownRows<BITS, VEC, CPL, 4> a, b;
      if (nfull > 0) {
        a.load(lc, sb_base, stride, half_sb, queue);
      }
      for (int s = 0; s < nfull; s += 2) {
        if (s + 1 < nfull) {
          b.load(lc, sb_base, stride, half_sb, queue + 4 * (s + 1));
        }
        a.pool(half_sb, weighted, queue + 4 * s, acc);
        if (s + 1 < nfull) {
          if (s + 2 < nfull) {
            a.load(lc, sb_base, stride, half_sb, queue + 4 * (s + 2));
          }
          b.pool(half_sb, weighted, queue + 4 * (s + 1), acc);
        }
      }
    } else {
      for (int s = 0; s < nfull; ++s) {
        KnownRows<BITS, VEC, CPL, 4> a;
        a.load(lc, sb_base, stride, half_sb, queue + 4 * s);
        a.pool(half_sb, weighted, queue + 4 * s, acc);
      }
    }
    int r = 4 * nfull;
    if (count - r >= 2) {
      KnownRows<BITS, VEC, CPL, 2> t;
      t.load(lc, sb_base, stride, half_sb, queue + r);
      t.pool(half_sb, weighted, queue + r, acc);
      r += 2;
    }
    if (count - r >= 1) {
      KnownRows<BITS, VEC, CPL, 1> t;
      t.load(lc, sb_base, stride, half_sb, queue + r);
      t.pool(half_sb, weighted, queue + r, acc);
    }
    __syncwarp(gmask);  // the queue is rewritten by the next stretch
  }

  if ((p.flags & kNormalize) && bag_len != 0) {
    const float inv = __fdiv_rn(1.f, (float)bag_len);
    const u64 inv2 = pack2(inv, inv);
#pragma unroll
    for (int ci = 0; ci < CPL; ++ci) {
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        acc[ci][j] = mul2(acc[ci][j], inv2);
      }
    }
  }
#pragma unroll
  for (int ci = 0; ci < CPL; ++ci) {
    const int c = gl + ci * LPB;
    if (c < nchunks) {
      store_columns<CPC>(p, bag, c * CPC, acc[ci]);
    }
  }
}

// One table per launch; the parameters travel in constant memory.
template <int BITS, int VEC, int LPB, int CPL, bool EXACT>
__global__ void __launch_bounds__(kThreads)
spmdm_direct_kernel(const __grid_constant__ SpmdmParams p) {
  direct_block<BITS, VEC, LPB, CPL, EXACT>(p, blockIdx.x);
}

// Several tables of the same row format in one launch (the reference's
// multi-table caller loops over tables,
// fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:343-473).
// The tables' parameters arrive by value, i.e. in constant memory as in the
// single-table kernel; a block finds its table by comparing its index with
// the tables' first blocks (at most kMultiTables - 1 uniform comparisons).
template <int BITS, int VEC, int LPB, int CPL, bool EXACT>
__global__ void __launch_bounds__(kThreads)
spmdm_direct_multi_kernel(const __grid_constant__ MultiArgs a) {
  int t = 0;
#pragma unroll
  for (int i = 1; i < kMultiTables; ++i) {
    t += (i < a.count && blockIdx.x >= (unsigned)a.first_block[i]) ? 1 : 0;
  }
  direct_block<BITS, VEC, LPB, CPL, EXACT>(a.t[t], (int64_t)blockIdx.x - a.first_block[t]);
}

// One table per launch, rows compacted before they are pooled (pruned tables).
template <int BITS, int VEC, int LPB, int CPL, bool EXACT>
__global__ void __launch_bounds__(kThreads)
spmdm_direct_compact_kernel(const __grid_constant__ SpmdmParams p) {
  direct_block_compact<BITS, VEC, LPB, CPL, EXACT>(p, blockIdx.x);
}

// Several such tables in one launch (see spmdm_direct_multi_kernel).
template <int BITS, int VEC, int LPB, int CPL, bool EXACT>
__global__ void __launch_bounds__(kThreads)
spmdm_direct_compact_multi_kernel(const __grid_constant__ MultiArgs a) {
  int t = 0;
#pragma unroll
  for (int i = 1; i < kMultiTables; ++i) {
    t += (i < a.count && blockIdx.x >= (unsigned)a.first_block[i]) ? 1 : 0;
  }
  direct_block_compact<BITS, VEC, LPB, CPL, EXACT>(a.t[t], (int64_t)blockIdx.x - a.first_block[t]);
}

using KernelFn = void (*)(const SpmdmParams);
using MultiKernelFn = void (*)(const MultiArgs);

// One (VEC, LPB, CPL) combination; each kernel in two forms, indexed by whether
// the row's payload is exactly LPB * CPL chunks (see LaneChunks).
struct Variant {
  KernelFn fn[2];
  MultiKernelFn multi[2];
  KernelFn compact[2];
  MultiKernelFn compact_multi[2];
  int vec, lpb, cpl;
};

}  // namespace direct

// Tables of instantiated variants, one translation unit per bit rate
// (spmdm_direct_{8,4,2}.cu).
const direct::Variant* direct_variants_8(int* count);
const direct::Variant* direct_variants_4(int* count);
const direct::Variant* direct_variants_2(int* count);

}  // namespace fbgemm_b200

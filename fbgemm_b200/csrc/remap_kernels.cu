// compressed_indices_remap on the GPU: the other way of pruning rows.  Instead
// of handing the pruning map to the lookup, the caller first rewrites
// (indices, offsets, weights) so that pruned rows disappear and the remaining
// indices address the compressed table, then runs a plain lookup.
//
// Reference: compressed_indices_remap_ref, src/RefImplementations.cc:2308-2333
// (the AVX-512 form behind fbgemm::compressed_indices_remap,
// src/EmbeddingSpMDM.cc:1714-1770, computes the same):
//
//   out_offsets[0] = offsets[0];  j = 0
//   for i in 1..offsets_len-1:
//     for k in offsets[i-1] .. offsets[i]-1:
//       if map[indices[k]] != -1: out_indices[j] = map[indices[k]]
//                                 out_weights[j] = weights[k];  ++j
//     out_offsets[i] = j
//
// That is a stream compaction of the positions [offsets[0], offsets[last]) in
// order.  Three passes over tiles of kTile positions: count the kept entries
// per tile, scan the tile counts (one block), then scan inside each tile,
// scatter, and record for every position how many kept entries precede it; a
// last small kernel reads out_offsets from that record.  The quirk of the
// reference is kept: out_offsets[0] repeats offsets[0] while the others count
// from zero.
#include "internal.h"

namespace fbgemm_b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kPerThread = 8;
constexpr int kTile = kThreads * kPerThread;

__device__ __forceinline__ int64_t load_index(const void* p, int64_t i, bool is64) {
  return is64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(p) + i)
              : (int64_t)__ldg(reinterpret_cast<const int*>(p) + i);
}

struct RemapArgs {
  const void* indices;
  const void* offsets;
  const int32_t* mapping;
  const float* weights;
  void* out_indices;
  void* out_offsets;
  float* out_weights;
  int64_t* tile_counts;   // [tiles + 1]
  int64_t* kept_before;   // [index_size + 1]
  int32_t* status;
  int64_t mapping_size;
  int64_t index_size;     // entries the caller's index array holds
  int32_t offsets_len;
  int32_t is64;
};

// Position range [lo, hi) the offsets cover, clamped to the index array.
__device__ __forceinline__ void covered(const RemapArgs& a, int64_t& lo, int64_t& hi) {
  lo = load_index(a.offsets, 0, a.is64);
  hi = load_index(a.offsets, a.offsets_len - 1, a.is64);
  lo = lo < 0 ? 0 : (lo > a.index_size ? a.index_size : lo);
  hi = hi < lo ? lo : (hi > a.index_size ? a.index_size : hi);
}

// The compressed row of position k, or -1 (pruned, or an index the map does
// not cover - reported, never dereferenced).
__device__ __forceinline__ int32_t mapped_row(const RemapArgs& a, int64_t k) {
  const int64_t idx = load_index(a.indices, k, a.is64);
  if (idx < 0 || idx >= a.mapping_size) {
    if (atomicCAS(a.status, 0, FBGEMM_B200_STATUS_BAD_INDEX) == 0) {
      a.status[1] = 0;
      a.status[2] = (int32_t)k;
      a.status[3] = (int32_t)idx;
    }
    return -1;
  }
  return __ldg(a.mapping + idx);
}

__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {
  __shared__ int warp_sums[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) {
      incl += t;
    }
  }
  if (lane == 31) {
    warp_sums[warp] = incl;
  }
  __syncthreads();
  if (warp == 0) {
    const int w = lane < kThreads / 32 ? warp_sums[lane] : 0;
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) {
        wi += t;
      }
    }
    if (lane < kThreads / 32) {
      warp_sums[lane] = wi - w;
    }
    if (lane == 31) {
      *total = wi;
    }
  }
  __syncthreads();
  const int r = warp_sums[warp] + incl - v;
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(kThreads) remap_count(const RemapArgs a) {
  __shared__ int total;
  int64_t lo, hi;
  covered(a, lo, hi);
  const int64_t base = lo + (int64_t)blockIdx.x * kTile + (int64_t)threadIdx.x * kPerThread;
  int kept = 0;
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    if (base + i < hi) {
      kept += mapped_row(a, base + i) != -1;
    }
  }
  block_exclusive_scan(kept, &total);
  if (threadIdx.x == 0) {
    a.tile_counts[blockIdx.x] = total;
  }
}

// One block: tile_counts[0..tiles) -> exclusive prefix, tile_counts[tiles] = total.  A tile holds at
// most kTile kept entries, so a chunk of kThreads counts is scanned in 32 bits and carried in 64.
__global__ void __launch_bounds__(kThreads) remap_scan_tiles(int64_t* tile_counts, int64_t tiles) {
  __shared__ int total;
  int64_t carry = 0;
  for (int64_t b = 0; b < tiles; b += kThreads) {
    const int64_t i = b + threadIdx.x;
    const int v = i < tiles ? (int)tile_counts[i] : 0;
    const int before = block_exclusive_scan(v, &total);
    if (i < tiles) {
      tile_counts[i] = carry + before;
    }
    carry += total;
    __syncthreads();  // `total` is rewritten by the next chunk's scan
  }
  if (threadIdx.x == 0) {
    tile_counts[tiles] = carry;
  }
}

__global__ void __launch_bounds__(kThreads) remap_scatter(const RemapArgs a) {
  __shared__ int total;
  int64_t lo, hi;
  covered(a, lo, hi);
  const int64_t base = lo + (int64_t)blockIdx.x * kTile + (int64_t)threadIdx.x * kPerThread;
  int32_t row[kPerThread];
  int kept = 0;
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    row[i] = base + i < hi ? mapped_row(a, base + i) : -1;
    kept += row[i] != -1;
  }
  int64_t pos = a.tile_counts[blockIdx.x] + block_exclusive_scan(kept, &total);
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    const int64_t k = base + i;
    if (k < hi) {
      a.kept_before[k - lo] = pos;
      if (row[i] != -1) {
        if (a.is64) {
          static_cast<long long*>(a.out_indices)[pos] = row[i];
        } else {
          static_cast<int*>(a.out_indices)[pos] = row[i];
        }
        if (a.weights) {
          a.out_weights[pos] = __ldg(a.weights + k);
        }
        ++pos;
      }
    }
  }
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
    a.kept_before[hi - lo] = a.tile_counts[gridDim.x];
  }
}

__global__ void __launch_bounds__(kThreads) remap_offsets(const RemapArgs a) {
  const int i = blockIdx.x * kThreads + threadIdx.x;
  if (i >= a.offsets_len) {
    return;
  }
  int64_t lo, hi;
  covered(a, lo, hi);
  int64_t v;
  if (i == 0) {
    v = load_index(a.offsets, 0, a.is64);  // as the reference: offsets[0], not 0
  } else {
    int64_t k = load_index(a.offsets, i, a.is64);
    k = k < lo ? lo : (k > hi ? hi : k);
    v = hi > lo ? a.kept_before[k - lo] : 0;
  }
  if (a.is64) {
    static_cast<long long*>(a.out_offsets)[i] = v;
  } else {
    static_cast<int*>(a.out_offsets)[i] = (int)v;
  }
}

}  // namespace

size_t remap_scratch_bytes(int64_t index_size) {
  const int64_t tiles = (index_size + kTile - 1) / kTile + 1;
  return (size_t)(tiles + 1 + index_size + 1) * sizeof(int64_t);
}

cudaError_t launch_compressed_indices_remap(
    int32_t offsets_len,
    const void* indices,
    int index_bytes,
    int64_t index_size,
    const int32_t* mapping,
    int64_t mapping_size,
    const void* offsets,
    const float* weights,
    void* out_indices,
    void* out_offsets,
    float* out_weights,
    int32_t* status,
    void* scratch,
    cudaStream_t stream) {
  RemapArgs a{};
  a.indices = indices;
  a.offsets = offsets;
  a.mapping = mapping;
  a.weights = weights;
  a.out_indices = out_indices;
  a.out_offsets = out_offsets;
  a.out_weights = out_weights;
  a.status = status;
  a.mapping_size = mapping_size;
  a.index_size = index_size;
  a.offsets_len = offsets_len;
  a.is64 = index_bytes == 8;
  const int64_t tiles = (index_size + kTile - 1) / kTile;
  a.tile_counts = static_cast<int64_t*>(scratch);
  a.kept_before = a.tile_counts + tiles + 2;
  if (tiles > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  if (tiles > 0) {
    remap_count<<<(unsigned)tiles, kThreads, 0, stream>>>(a);
    remap_scan_tiles<<<1, kThreads, 0, stream>>>(a.tile_counts, tiles);
    remap_scatter<<<(unsigned)tiles, kThreads, 0, stream>>>(a);
    g_launch_count.fetch_add(3, std::memory_order_relaxed);
  }
  remap_offsets<<<(offsets_len + kThreads - 1) / kThreads, kThreads, 0, stream>>>(a);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

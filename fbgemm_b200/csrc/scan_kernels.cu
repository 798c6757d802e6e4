// Exclusive scan of bag lengths into offsets, for the lengths flavour of the
// lookup (use_offsets = false, the Caffe2 SparseLengthsSum interface of
// include/fbgemm/FbgemmEmbedding.h:55-63).  The reference walks the lengths
// sequentially (`current += len`, src/RefImplementations.cc:1290-1298); on the
// GPU every bag has to know its start up front.
//
// Three small launches: per-tile scan, scan of the tile totals by one block,
// add-back.  Each length is narrowed to 32 bits first, as `int len` does in
// the reference, and a negative length advances nothing.
#include "internal.h"

namespace fbgemm_b200 {

namespace {

constexpr int kScanThreads = 1024;
constexpr int kItemsPerThread = 4;
constexpr int kTile = kScanThreads * kItemsPerThread;

__device__ __forceinline__ int64_t load_len(const void* p, int64_t i, bool is64, int64_t n) {
  if (i >= n) {
    return 0;
  }
  const int v = is64 ? (int)__ldg(reinterpret_cast<const long long*>(p) + i)
                     : __ldg(reinterpret_cast<const int*>(p) + i);
  return v < 0 ? 0 : (int64_t)v;
}

// Exclusive scan of one value per thread across the block; returns the
// exclusive prefix, *total gets the block sum.
__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t* total) {
  __shared__ int64_t warp_sums[32];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  int64_t incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int64_t t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) {
      incl += t;
    }
  }
  if (lane == 31) {
    warp_sums[warp] = incl;
  }
  __syncthreads();
  if (warp == 0) {
    int64_t w = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0;
    int64_t wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int64_t t = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) {
        wi += t;
      }
    }
    warp_sums[lane] = wi - w;  // exclusive prefix of the warp sums
    if (lane == 31) {
      *total = wi;
    }
  }
  __syncthreads();
  const int64_t r = warp_sums[warp] + incl - v;
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(kScanThreads)
scan_tiles(const void* lengths, int is64, int64_t n, int64_t* offsets, int64_t* tile_sums) {
  __shared__ int64_t total;
  const int64_t base = (int64_t)blockIdx.x * kTile + (int64_t)threadIdx.x * kItemsPerThread;
  int64_t v[kItemsPerThread];
  int64_t sum = 0;
#pragma unroll
  for (int i = 0; i < kItemsPerThread; ++i) {
    v[i] = load_len(lengths, base + i, is64 != 0, n);
    sum += v[i];
  }
  int64_t prefix = block_exclusive_scan(sum, &total);
#pragma unroll
  for (int i = 0; i < kItemsPerThread; ++i) {
    if (base + i < n) {
      offsets[base + i] = prefix;
    }
    prefix += v[i];
  }
  if (threadIdx.x == 0) {
    tile_sums[blockIdx.x] = total;
  }
}

// One block turns tile_sums[0..m) into its exclusive scan, in place, and
// writes the grand total to offsets[n].
__global__ void __launch_bounds__(kScanThreads)
scan_tile_sums(int64_t* tile_sums, int64_t m, int64_t* offsets, int64_t n) {
  __shared__ int64_t total;
  int64_t carry = 0;
  for (int64_t base = 0; base < m; base += kScanThreads) {
    const int64_t i = base + threadIdx.x;
    const int64_t v = i < m ? tile_sums[i] : 0;
    const int64_t prefix = block_exclusive_scan(v, &total);
    if (i < m) {
      tile_sums[i] = carry + prefix;
    }
    carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    offsets[n] = carry;
  }
}

__global__ void __launch_bounds__(kScanThreads)
add_tile_prefix(int64_t* offsets, const int64_t* tile_sums, int64_t n) {
  const int64_t add = tile_sums[blockIdx.x];
  const int64_t base = (int64_t)blockIdx.x * kTile + (int64_t)threadIdx.x * kItemsPerThread;
#pragma unroll
  for (int i = 0; i < kItemsPerThread; ++i) {
    if (base + i < n) {
      offsets[base + i] += add;
    }
  }
}

}  // namespace

size_t scan_scratch_elems(int64_t n) {
  return (size_t)((n + kTile - 1) / kTile) + 1;
}

cudaError_t launch_length_scan(
    const void* lengths,
    int length_bytes,
    int64_t n,
    int64_t* offsets,
    int64_t* tile_sums,
    cudaStream_t stream) {
  const int64_t tiles = (n + kTile - 1) / kTile;
  if (tiles <= 0 || tiles > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  scan_tiles<<<(unsigned)tiles, kScanThreads, 0, stream>>>(lengths, length_bytes == 8, n, offsets, tile_sums);
  scan_tile_sums<<<1, kScanThreads, 0, stream>>>(tile_sums, tiles, offsets, n);
  add_tile_prefix<<<(unsigned)tiles, kScanThreads, 0, stream>>>(offsets, tile_sums, n);
  g_launch_count.fetch_add(3, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

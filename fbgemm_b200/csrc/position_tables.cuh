// Which table of a table-batched call does position k of the index array
// belong to?  The call's offsets hold T*B+1 entries, table after table, so the
// tables' positions start at offsets[t*B], t = 0..T.  A kernel whose threads
// (or warps) own positions stages these T+1 starts in shared memory, clamped to
// the index array, and bisects; beyond kSharedStarts-1 tables it bisects in
// global memory instead.  Args needs: offsets, index_size, T, B, index64.
#pragma once

#include <cstdint>

namespace fbgemm_b200 {

constexpr int kSharedStarts = 2048;  // 16 KB of shared memory per block

__device__ __forceinline__ int64_t load_position_int(const void* p, int64_t i, bool is64) {
  return is64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(p) + i)
              : (int64_t)__ldg(reinterpret_cast<const int*>(p) + i);
}

template <typename Args>
__device__ __forceinline__ int64_t table_start(const Args& a, const int64_t* starts, int t) {
  if (starts) {
    return starts[t];
  }
  const int64_t v = load_position_int(a.offsets, (int64_t)t * a.B, a.index64);
  return v < 0 ? 0 : (v > a.index_size ? a.index_size : v);
}

// Call with every thread of the block; `smem` holds kSharedStarts entries.
// Returns what table_start / table_of read: shared memory, or null = global.
template <typename Args>
__device__ __forceinline__ const int64_t* stage_table_starts(const Args& a, int64_t* smem) {
  if (a.T + 1 > kSharedStarts) {
    return nullptr;
  }
  for (int t = threadIdx.x; t <= a.T; t += blockDim.x) {
    smem[t] = table_start(a, static_cast<const int64_t*>(nullptr), t);
  }
  __syncthreads();
  return smem;
}

// The last t in [0, T) with start(t) <= k, provided start(0) <= k < start(T);
// -1 if no table covers k.  With offsets that step backwards the answer is
// some table - never an access outside the arrays.
template <typename Args>
__device__ __forceinline__ int table_of(const Args& a, const int64_t* starts, int64_t k) {
  if (k < table_start(a, starts, 0) || k >= table_start(a, starts, a.T)) {
    return -1;
  }
  int lo = 0, hi = a.T;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (table_start(a, starts, mid) <= k) {
      lo = mid;
    } else {
      hi = mid;
    }
  }
  return lo;
}

}  // namespace fbgemm_b200

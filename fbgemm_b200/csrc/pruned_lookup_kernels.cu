// Index remapping of table-batched pruned tables: sparse index -> dense index
// (or -1 for a pruned row) through a per-table open-addressing hash map or a
// per-table array, run by a table-batched caller before the lookup.
//
// Reference: pruned_hashmap_lookup_{un}weighted_cpu and pruned_array_lookup_cpu,
// fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:524-601,
// :605-659; hash :102-120 (MurmurHash3 finalisers); the reference's CUDA forms
// (embedding_forward_quantized_split_lookup.cu:20-160) give a warp to every
// bag.  Here a thread owns one POSITION of the index array, so the work per
// thread does not depend on how ragged the bags are and index loads and result
// stores are coalesced; the thread finds its table by bisection over the T+1
// table starts offsets[t*B] (staged in shared memory when they fit) and then
// probes alone: at a load factor of 0.8 a hit walks about 3 slots and a miss
// about 13, i.e. one to four neighbouring 32-byte sectors.
//
// The reference's probe loop has no end on a full table that lacks the key;
// here it stops after `capacity` slots with -1, so no launch can spin.
#include "internal.h"
#include "position_tables.cuh"

namespace fbgemm_b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kPerThread = 4;

__device__ __forceinline__ int64_t load_int(const void* p, int64_t i, bool is64) {
  return is64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(p) + i)
              : (int64_t)__ldg(reinterpret_cast<const int*>(p) + i);
}

__device__ __forceinline__ void store_int(void* p, int64_t i, int64_t v, bool is64) {
  if (is64) {
    static_cast<long long*>(p)[i] = v;
  } else {
    static_cast<int*>(p)[i] = (int)v;
  }
}

__device__ __forceinline__ uint32_t hash32(uint32_t h) {
  h ^= h >> 16;
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  h *= 0xc2b2ae35u;
  h ^= h >> 16;
  return h;
}

__device__ __forceinline__ uint64_t hash64(uint64_t k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return k;
}

struct PrunedArgs {
  const void* indices;
  const void* offsets;
  const void* map;            // hash table ([.][2]) or remapping array
  const int64_t* map_offsets; // [T + 1]
  void* dense;
  int32_t* status;
  int64_t index_size;
  int32_t T;
  int32_t B;
  int32_t index64;
  int32_t map64;
};

__device__ __forceinline__ void report(const PrunedArgs& a, int code, int64_t table, int64_t pos, int64_t value) {
  if (atomicCAS(a.status, 0, code) == 0) {
    a.status[1] = (int32_t)table;
    a.status[2] = (int32_t)pos;
    a.status[3] = (int32_t)value;
  }
}

template <bool HASH>
__global__ void __launch_bounds__(kThreads) pruned_lookup_kernel(const PrunedArgs a) {
  __shared__ int64_t starts_s[kSharedStarts];
  const int64_t* starts = stage_table_starts(a, starts_s);
  const int64_t base = ((int64_t)blockIdx.x * kPerThread) * kThreads + threadIdx.x;
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    const int64_t k = base + (int64_t)i * kThreads;
    if (k >= a.index_size) {
      break;
    }
    const int t = table_of(a, starts, k);
    if (t < 0) {
      continue;
    }
    const int64_t idx = load_int(a.indices, k, a.index64);
    const int64_t map_start = __ldg(a.map_offsets + t);
    const int64_t capacity = __ldg(a.map_offsets + t + 1) - map_start;
    int64_t dense = -1;
    if (capacity <= 0) {
      dense = idx;
    } else if (HASH) {
      const uint64_t h = a.index64 ? hash64((uint64_t)idx) : (uint64_t)hash32((uint32_t)idx);
      int64_t slot = (int64_t)(h % (uint64_t)capacity);
      // One slot per step.  Examining four slots per step with their loads in flight together was
      // measured slower (950 against 700 us for 7.9 M positions over 16 tables of 2.5 M slots): the
      // limit is the rate of random 32-byte sectors, not the chain of dependent loads, and a window of
      // four slots straddles sectors that a probe sequence would not have touched.
      for (int64_t probes = 0; probes < capacity; ++probes) {
        int64_t key, value;
        if (a.map64) {
          const longlong2 kv = __ldg(reinterpret_cast<const longlong2*>(a.map) + map_start + slot);
          key = kv.x;
          value = kv.y;
        } else {
          const int2 kv = __ldg(reinterpret_cast<const int2*>(a.map) + map_start + slot);
          key = kv.x;
          value = kv.y;
        }
        if (key == -1) {
          break;
        }
        if (key == idx) {
          dense = value;
          break;
        }
        slot = slot + 1 == capacity ? 0 : slot + 1;
      }
    } else if (idx < 0 || idx >= capacity) {
      report(a, FBGEMM_B200_STATUS_BAD_INDEX, t, k, idx);
    } else {
      dense = load_int(a.map, map_start + idx, a.map64);
    }
    store_int(a.dense, k, dense, a.index64);
  }
}

}  // namespace

cudaError_t launch_pruned_lookup(
    bool hashmap,
    int32_t T,
    int32_t B,
    const void* indices,
    const void* offsets,
    int index_bytes,
    int64_t index_size,
    const void* map,
    int map_bytes,
    const int64_t* map_offsets,
    void* dense_indices,
    int32_t* status,
    cudaStream_t stream) {
  if (index_size == 0) {
    return cudaSuccess;
  }
  PrunedArgs a{};
  a.indices = indices;
  a.offsets = offsets;
  a.map = map;
  a.map_offsets = map_offsets;
  a.dense = dense_indices;
  a.status = status;
  a.index_size = index_size;
  a.T = T;
  a.B = B;
  a.index64 = index_bytes == 8;
  a.map64 = map_bytes == 8;
  const int64_t per_block = (int64_t)kThreads * kPerThread;
  const int64_t blocks = (index_size + per_block - 1) / per_block;
  if (blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  if (hashmap) {
    pruned_lookup_kernel<true><<<(unsigned)blocks, kThreads, 0, stream>>>(a);
  } else {
    pruned_lookup_kernel<false><<<(unsigned)blocks, kThreads, 0, stream>>>(a);
  }
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

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
// probes alone (see pruned_hashmap_kernel for how the lanes of a warp are kept
// busy while their probe sequences differ in length).
//
// The reference's probe loop has no end on a full table that lacks the key;
// here it stops after `capacity` slots with -1, so no launch can spin.
#include "internal.h"
#include "position_tables.cuh"

namespace fbgemm_b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kPerThread = 4;  // positions per thread, array form
constexpr int kHashPer = 2;  // positions per thread, hash-map form

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

// The array form, and tables without a map: one load per position.
__global__ void __launch_bounds__(kThreads) pruned_array_kernel(const PrunedArgs a) {
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
    } else if (idx < 0 || idx >= capacity) {
      report(a, FBGEMM_B200_STATUS_BAD_INDEX, t, k, idx);
    } else {
      dense = load_int(a.map, map_start + idx, a.map64);
    }
    store_int(a.dense, k, dense, a.index64);
  }
}

template <bool MAP64>
__device__ __forceinline__ void load_slot(const void* slots, int64_t at, int64_t& key, int64_t& value) {
  if constexpr (MAP64) {
    const longlong2 kv = __ldg(reinterpret_cast<const longlong2*>(slots) + at);
    key = kv.x;
    value = kv.y;
  } else {
    const int2 kv = __ldg(reinterpret_cast<const int2*>(slots) + at);
    key = kv.x;
    value = kv.y;
  }
}

// The hash-map form.  A thread owns kHashPer positions and the work is split in two.  First, all
// lanes together: table, index, hash and first slot of every position (the expensive part, a modulo
// included), kept in registers.  Then one loop with 32-bit slot arithmetic in which each lane walks its
// positions' probe sequences back to back - a lane that finishes one starts its next at once.
// Measured on 7.9 M positions over 16 tables of 2.5 M slots at a load factor of 0.8 (a hit walks 3
// slots on average, a miss 13, some of them dozens), half of the keys present: 498 us with 2 positions
// per thread, 520 with 4, 563 with 8, 732 with 16; 700 us for the first form (a thread looping over 4
// positions one after the other with 64-bit slot arithmetic, 6 of 32 threads active per instruction),
// 950 us with four slots examined per step.
template <bool MAP64>
__global__ void __launch_bounds__(kThreads) pruned_hashmap_kernel(const PrunedArgs a) {
  __shared__ int64_t starts_s[kSharedStarts];
  const int64_t* starts = stage_table_starts(a, starts_s);
  const int64_t base = ((int64_t)blockIdx.x * kHashPer) * kThreads + threadIdx.x;
  uint32_t first_slot[kHashPer];
  int table[kHashPer];
  uint32_t todo = 0;  // bit i: position i has a probe sequence to walk
#pragma unroll
  for (int i = 0; i < kHashPer; ++i) {
    first_slot[i] = 0;
    table[i] = 0;
    const int64_t k = base + (int64_t)i * kThreads;
    const int t = k < a.index_size ? table_of(a, starts, k) : -1;
    if (t >= 0) {
      const int64_t idx = load_int(a.indices, k, a.index64);
      const int64_t map_start = __ldg(a.map_offsets + t);
      const int64_t capacity = __ldg(a.map_offsets + t + 1) - map_start;
      if (capacity <= 0) {
        store_int(a.dense, k, idx, a.index64);  // a table without a map keeps its indices
      } else {
        const uint64_t h = a.index64 ? hash64((uint64_t)idx) : (uint64_t)hash32((uint32_t)idx);
        if (capacity <= 0x7fffffffLL) {
          first_slot[i] = (h >> 32) == 0 ? (uint32_t)h % (uint32_t)capacity : (uint32_t)(h % (uint64_t)capacity);
          table[i] = t;
          todo |= 1u << i;
        } else {
          // a table of 2^31 slots or more: walked here, with 64-bit slot arithmetic
          int64_t slot = (int64_t)(h % (uint64_t)capacity), dense = -1;
          for (int64_t probes = 0; probes < capacity; ++probes) {
            int64_t key, value;
            load_slot<MAP64>(a.map, map_start + slot, key, value);
            if (key == -1) {
              break;
            }
            if (key == idx) {
              dense = value;
              break;
            }
            slot = slot + 1 == capacity ? 0 : slot + 1;
          }
          store_int(a.dense, k, dense, a.index64);
        }
      }
    }
  }

  bool walking = false;
  int64_t k = 0, idx = 0;
  const void* slots = nullptr;
  uint32_t slot = 0, capacity = 0, probes = 0;
  while (true) {
    if (!walking) {
      if (todo == 0) {
        break;
      }
      const int i = __ffs(todo) - 1;
      todo &= todo - 1;
      int t = 0;
#pragma unroll
      for (int q = 0; q < kHashPer; ++q) {
        if (q == i) {
          slot = first_slot[q];
          t = table[q];
        }
      }
      k = base + (int64_t)i * kThreads;
      idx = load_int(a.indices, k, a.index64);
      const int64_t map_start = __ldg(a.map_offsets + t);
      capacity = (uint32_t)(__ldg(a.map_offsets + t + 1) - map_start);
      slots = static_cast<const char*>(a.map) + map_start * (MAP64 ? 16 : 8);
      probes = 0;
      walking = true;
    }
    int64_t key, value;
    load_slot<MAP64>(slots, slot, key, value);
    if (key == -1 || key == idx) {
      store_int(a.dense, k, key == -1 ? -1 : value, a.index64);
      walking = false;
    } else {
      slot = slot + 1 == capacity ? 0 : slot + 1;
      if (++probes >= capacity) {  // a full table without the key
        store_int(a.dense, k, -1, a.index64);
        walking = false;
      }
    }
  }
}

// Filling the hash map on the device.  The reference only inserts on the host, one key after the
// other; here every position claims the first free slot of its probe sequence with a compare-and-swap
// on the key, so the slots a cluster's keys end up in depend on the order the threads arrive in - the
// table differs from the host-built one byte for byte but every lookup gives the same answer (a key
// sits within its probe sequence, before the first empty slot).  Positions whose dense index is -1
// are not inserted, as in the reference; a table without a free slot is reported.
template <bool MAP64>
__global__ void __launch_bounds__(kThreads) pruned_hashmap_insert_kernel(const PrunedArgs a, const void* dense_indices) {
  __shared__ int64_t starts_s[kSharedStarts];
  const int64_t* starts = stage_table_starts(a, starts_s);
  const int64_t k = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int t = k < a.index_size ? table_of(a, starts, k) : -1;
  if (t < 0) {
    return;
  }
  const int64_t dense = load_int(dense_indices, k, a.index64);
  const int64_t map_start = __ldg(a.map_offsets + t);
  const int64_t capacity = __ldg(a.map_offsets + t + 1) - map_start;
  if (dense == -1 || capacity <= 0) {
    return;
  }
  const int64_t idx = load_int(a.indices, k, a.index64);
  const uint64_t h = a.index64 ? hash64((uint64_t)idx) : (uint64_t)hash32((uint32_t)idx);
  int64_t slot = (int64_t)(h % (uint64_t)capacity);
  for (int64_t probes = 0; probes < capacity; ++probes) {
    const int64_t at = 2 * (map_start + slot);
    int64_t seen;
    if constexpr (MAP64) {
      unsigned long long* keys = static_cast<unsigned long long*>(const_cast<void*>(a.map));
      seen = (int64_t)atomicCAS(keys + at, ~0ULL, (unsigned long long)idx);
      if (seen == -1 || seen == idx) {
        reinterpret_cast<long long*>(keys)[at + 1] = dense;
        return;
      }
    } else {
      int* keys = static_cast<int*>(const_cast<void*>(a.map));
      seen = atomicCAS(keys + at, -1, (int)idx);
      if (seen == -1 || seen == (int)idx) {
        keys[at + 1] = (int)dense;
        return;
      }
    }
    slot = slot + 1 == capacity ? 0 : slot + 1;
  }
  report(a, FBGEMM_B200_STATUS_TABLE_FULL, t, k, idx);
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
  const int64_t per_block = (int64_t)kThreads * (hashmap ? kHashPer : kPerThread);
  const int64_t blocks = (index_size + per_block - 1) / per_block;
  if (blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  if (!hashmap) {
    pruned_array_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(a);
  } else if (a.map64) {
    pruned_hashmap_kernel<true><<<(unsigned)blocks, kThreads, 0, stream>>>(a);
  } else {
    pruned_hashmap_kernel<false><<<(unsigned)blocks, kThreads, 0, stream>>>(a);
  }
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

namespace fbgemm_b200 {

cudaError_t launch_pruned_hashmap_insert(
    int32_t T,
    int32_t B,
    const void* indices,
    const void* dense_indices,
    const void* offsets,
    int index_bytes,
    int64_t index_size,
    void* hash_table,
    int hash_bytes,
    const int64_t* hash_table_offsets,
    int32_t* status,
    cudaStream_t stream) {
  if (index_size == 0) {
    return cudaSuccess;
  }
  PrunedArgs a{};
  a.indices = indices;
  a.offsets = offsets;
  a.map = hash_table;
  a.map_offsets = hash_table_offsets;
  a.status = status;
  a.index_size = index_size;
  a.T = T;
  a.B = B;
  a.index64 = index_bytes == 8;
  a.map64 = hash_bytes == 8;
  const int64_t blocks = (index_size + kThreads - 1) / kThreads;
  if (blocks > 0x7fffffffLL) {
    return cudaErrorInvalidValue;
  }
  if (a.map64) {
    pruned_hashmap_insert_kernel<true><<<(unsigned)blocks, kThreads, 0, stream>>>(a, dense_indices);
  } else {
    pruned_hashmap_insert_kernel<false><<<(unsigned)blocks, kThreads, 0, stream>>>(a, dense_indices);
  }
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

// Device-side ordering between the GPUs of a table-wise sharded lookup.
//
// The sharded lookup stores pooled rows straight into buffers that live in
// peer GPUs' memory.  Two things then have to be known on the device, per
// step and without a host round trip:
//   * consumer side: all producers' rows for my slice of buffer b have landed;
//   * producer side: every consumer has finished with buffer b's previous
//     contents, so it may be overwritten.
// Both are counters in each GPU's memory, one word per (buffer, peer), written
// by a one-block kernel that the writer enqueues on its stream after the work
// it announces (stores of earlier kernels on that stream have completed by the
// time it runs; the fence and the release store order it after them for
// observers anywhere in the system), and polled by a one-block kernel on the
// reader's stream.  The reference orders its peer copies with events between
// streams of one process
// (fbgemm_gpu/src/merge_pooled_embedding_ops/merge_pooled_embedding_ops_gpu.cpp:223-230,454-461);
// with one process per GPU the counters take that role.
//
// Plain system-scope stores and loads only: no multicast, no multimem.  The
// poll is bounded in wall time and in iterations; when it gives up it records
// FBGEMM_B200_STATUS_PEER_TIMEOUT in the caller's status record and returns,
// so the context stays usable and the host learns of it from the status read.
#include "internal.h"

namespace fbgemm_b200 {

namespace {

struct PeerFlags {
  unsigned long long* flag[FBGEMM_B200_MAX_PEERS];
};

__device__ __forceinline__ void store_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long load_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Thread i publishes `value` to flag[i] (a word in peer i's memory).
__global__ void peer_signal_kernel(const __grid_constant__ PeerFlags f, int n, unsigned long long value) {
  const int i = threadIdx.x;
  if (i < n) {
    __threadfence_system();
    store_release_sys(f.flag[i], value);
  }
}

// Thread i waits until flags[i] >= value, for at most timeout_ns (and at most
// max_polls polls, in case the timer does not advance).
__global__ void peer_wait_kernel(const unsigned long long* flags, int n, unsigned long long value,
                                 unsigned long long timeout_ns, unsigned long long max_polls, int32_t* status) {
  const int i = threadIdx.x;
  if (i >= n) {
    return;
  }
  const unsigned long long t0 = global_timer_ns();
  unsigned long long seen = load_acquire_sys(flags + i);
  for (unsigned long long poll = 0; seen < value; ++poll) {
    if (poll >= max_polls || global_timer_ns() - t0 > timeout_ns) {
      if (atomicCAS(status, 0, FBGEMM_B200_STATUS_PEER_TIMEOUT) == 0) {
        status[1] = i;                 // the peer that did not arrive
        status[2] = (int32_t)seen;     // the counter as last read (low 32 bits)
        status[3] = (int32_t)value;    // the value waited for (low 32 bits)
      }
      return;
    }
    __nanosleep(200);
    seen = load_acquire_sys(flags + i);
  }
}

}  // namespace

cudaError_t launch_peer_signal(void* const* flags, int n, uint64_t value, cudaStream_t stream) {
  if (n <= 0) {
    return cudaSuccess;
  }
  PeerFlags f{};
  for (int i = 0; i < n; ++i) {
    f.flag[i] = static_cast<unsigned long long*>(flags[i]);
  }
  peer_signal_kernel<<<1, 32, 0, stream>>>(f, n, (unsigned long long)value);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t launch_peer_wait(const void* flags, int n, uint64_t value, uint64_t timeout_us, int32_t* status,
                             cudaStream_t stream) {
  if (n <= 0) {
    return cudaSuccess;
  }
  // ~0.4 us per poll (the sleep plus a system-scope load): the poll cap is a
  // generous multiple of what the time limit allows.
  const unsigned long long max_polls = 16ull * (timeout_us + 1) + 1024;
  peer_wait_kernel<<<1, 32, 0, stream>>>(static_cast<const unsigned long long*>(flags), n, (unsigned long long)value,
                                         (unsigned long long)timeout_us * 1000ull, max_polls, status);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

}  // namespace fbgemm_b200

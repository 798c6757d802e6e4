// The context behind the C ABI and the small helpers its translation units
// share (c_api.cu, multi_host.cu).
#pragma once

#include <mutex>
#include <unordered_map>

#include "internal.h"

namespace fbgemm_b200 {

// Grow-only device buffer; contents are not preserved.
inline cudaError_t reserve(DeviceBuffer& b, size_t bytes) {
  if (bytes <= b.bytes) {
    return cudaSuccess;
  }
  if (b.ptr) {
    cudaFree(b.ptr);
    b.ptr = nullptr;
    b.bytes = 0;
  }
  const size_t want = bytes + bytes / 4 + 256;
  cudaError_t e = cudaMalloc(&b.ptr, want);
  if (e == cudaSuccess) {
    b.bytes = want;
  }
  return e;
}

struct PinnedBuffer {
  void* ptr = nullptr;
  size_t bytes = 0;
};

inline cudaError_t reserve(PinnedBuffer& b, size_t bytes) {
  if (bytes <= b.bytes) {
    return cudaSuccess;
  }
  if (b.ptr) {
    cudaFreeHost(b.ptr);
    b.ptr = nullptr;
    b.bytes = 0;
  }
  const size_t want = bytes + bytes / 4 + 256;
  cudaError_t e = cudaMallocHost(&b.ptr, want);
  if (e == cudaSuccess) {
    b.bytes = want;
  }
  return e;
}

// One staging lane of the host-pointer pipeline.
struct Lane {
  cudaStream_t stream = nullptr;
  DeviceBuffer d_in;    // indices | offsets | weights
  DeviceBuffer d_out;   // pooled rows
  DeviceBuffer d_scan;  // lengths-mode scratch of this lane
  PinnedBuffer h_in;
  PinnedBuffer h_out;
  PinnedBuffer h_status;
  bool busy = false;
  // what to do at wait()
  void* user_out = nullptr;
  size_t out_row_bytes = 0;   // bytes of one pooled row (block_size elements)
  size_t out_pitch_bytes = 0; // bytes between rows in the user's buffer
  int64_t out_rows = 0;
  bool trivially_true = false;
  bool trivially_false = false;
};

// A caller's host table made resident on the device.  `fingerprint` is taken
// over the host bytes at registration; `implicit` marks copies the host-pointer
// call made on its own (those are refreshed when they no longer match the
// caller's memory, explicit registrations are the caller's to refresh).
struct ResidentTable {
  DeviceBuffer buf;
  uint64_t fingerprint = 0;
  bool implicit = false;
};

// FNV-1a over the size and the first and last 256 bytes: cheap enough for
// every call, and a freed-and-reused host address hardly ever repeats all of it.
inline uint64_t table_fingerprint(const void* host, size_t bytes) {
  const uint8_t* b = static_cast<const uint8_t*>(host);
  uint64_t h = 1469598103934665603ull;
  auto mix = [&h](uint8_t v) {
    h ^= v;
    h *= 1099511628211ull;
  };
  for (int i = 0; i < 8; ++i) {
    mix((uint8_t)(bytes >> (8 * i)));
  }
  const size_t head = bytes < 256 ? bytes : 256;
  for (size_t i = 0; i < head; ++i) {
    mix(b[i]);
  }
  for (size_t i = bytes > 256 ? bytes - 256 : head; i < bytes; ++i) {
    mix(b[i]);
  }
  return h;
}

struct Derived {
  int data_bytes;
  int sb_bytes;
  int64_t input_stride;
  int64_t output_stride;
};

}  // namespace fbgemm_b200

struct fbgemm_b200_ctx {
  int device = 0;
  std::mutex mu;
  int32_t* status = nullptr;         // device, FBGEMM_B200_STATUS_SLOTS x 4
  int32_t* status_host = nullptr;    // pinned, same shape (read-back)
  // Lengths-mode scratch of the device-pointer path, one buffer per stream:
  // calls on one stream are ordered, calls on different streams must not
  // share the scanned offsets.
  std::unordered_map<cudaStream_t, fbgemm_b200::DeviceBuffer> scan;
  fbgemm_b200::DeviceBuffer remap_scratch;        // fbgemm_b200_compressed_indices_remap (one call at a time, it synchronises)
  std::unordered_map<const void*, fbgemm_b200::ResidentTable> tables;
  fbgemm_b200::Lane lanes[FBGEMM_B200_HOST_LANES];
};

struct fbgemm_b200_multi_plan {
  int device = 0;
  fbgemm_b200::MultiPlan plan;
};

namespace fbgemm_b200 {

class DeviceGuard {
 public:
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev_);
    if (prev_ != dev) {
      cudaSetDevice(dev);
      changed_ = true;
    }
  }
  ~DeviceGuard() {
    if (changed_) {
      cudaSetDevice(prev_);
    }
  }

 private:
  int prev_ = 0;
  bool changed_ = false;
};

}  // namespace fbgemm_b200

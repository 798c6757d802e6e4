// A lookup entry point for callers that must not allocate.
//
// Some programs hand every byte of device memory to their own allocator at
// start-up (inference servers with a fixed memory plan, frameworks with a
// caching allocator that assumes it owns the device) or run their request
// loop under a rule that nothing may call cudaMalloc after initialisation,
// because an allocation can stall the whole device or fail when the pool is
// already spoken for.  The lengths flavour of the lookup (use_offsets = 0)
// needs scratch memory - every bag has to learn where its indices start, so
// the lengths are scanned into offsets first - and the regular entry points
// take that scratch from a buffer the context grows with cudaMalloc.  This
// file offers the same lookup with the scratch placed in a fixed, file-scope
// device array instead: nothing is allocated, by this library or by anything
// it calls, at any time.
//
// What that costs: the array has a fixed size (FBGEMM_B200_NOALLOC_MAX_BAGS
// bags, about 8.4 MB) that every GPU which loads the library gives up until
// the process exits, and there is only one of it per GPU, so two calls that
// run on the GPU at the same time would overwrite each other's offsets.
#include <mutex>

#include "internal.h"

namespace {

constexpr int64_t kMaxBags = FBGEMM_B200_NOALLOC_MAX_BAGS;
constexpr int kMaxDevices = 64;
constexpr int64_t kScanTile = 4096;  // bags per block of the length scan
// int64 words: offsets[kMaxBags + 1], one partial sum per scan tile (+1), and
// the 4-word status record (2 int64 words), rounded up.
constexpr int64_t kScratchWords = (kMaxBags + 1) + (kMaxBags / kScanTile + 2) + 2 + 3;

// The scratch itself.  In host code this name is only a handle for the
// runtime, not an address a kernel could use: the device address is looked up
// once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) long long g_noalloc_scratch[kScratchWords];

std::mutex g_setup_mu;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch on the current device; resolved on the first
// call for that device.  Returns nullptr (and sets the error text) on failure.
void* scratch_for_current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    fbgemm_b200::fail_cuda(e, "cudaGetDevice");
    return nullptr;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    fbgemm_b200::set_error("device ordinal beyond the no-allocation entry point's table");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      fbgemm_b200::fail_cuda(e, "cudaGetSymbolAddress(no-allocation scratch)");
      return nullptr;
    }
    g_scratch_addr[dev] = ptr;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int fbgemm_b200_spmdm_lengths_noalloc(
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* lengths,
    const float* weights,
    void* out,
    const int32_t* compressed_indices_table,
    void* stream_v) {
  using namespace fbgemm_b200;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (!cfg || cfg->use_offsets) {
    set_error("the no-allocation entry point is the lengths flavour: cfg->use_offsets must be 0");
    return FBGEMM_B200_EINVAL;
  }
  // Everything is validated before the first kernel: the length scan below
  // would otherwise read `lengths` for configurations that carry none.
  const int cfg_rc = fbgemm_b200_spmdm_check_config(cfg);
  if (cfg_rc) {
    return cfg_rc;
  }
  if (cfg->no_bag || cfg->absolute_offsets || cfg->out_dtype == FBGEMM_B200_OUT_U8) {
    set_error("the no-allocation entry point pools bags given by lengths: no no_bag, absolute_offsets or 8-bit output");
    return FBGEMM_B200_EINVAL;
  }
  if (output_size < 0 || index_size < 0 || data_size < 0) {
    set_error("negative size");
    return FBGEMM_B200_EINVAL;
  }
  if (output_size > 0 && (!lengths || !out || (index_size > 0 && (!input || !indices)) ||
                          (cfg->has_weight && index_size > 0 && !weights))) {
    set_error("null lengths, table, indices, weights or output pointer");
    return FBGEMM_B200_EINVAL;
  }
  if (output_size > kMaxBags) {
    set_error("output_size " + std::to_string(output_size) + " exceeds FBGEMM_B200_NOALLOC_MAX_BAGS (" +
              std::to_string(kMaxBags) + "): the fixed scratch cannot hold the offsets; use fbgemm_b200_spmdm");
    return FBGEMM_B200_EINVAL;
  }
  if (output_size == 0) {
    return index_size == 0 ? 1 : 0;
  }
  if ((int64_t)scan_scratch_elems(output_size) > kMaxBags / kScanTile + 2) {
    set_error("length-scan tiling does not fit the fixed scratch");
    return FBGEMM_B200_EINVAL;
  }
  long long* scratch = static_cast<long long*>(scratch_for_current_device());
  if (!scratch) {
    return FBGEMM_B200_ECUDA;
  }
  int64_t* offsets = reinterpret_cast<int64_t*>(scratch);
  int64_t* tile_sums = offsets + kMaxBags + 1;
  int32_t* status = reinterpret_cast<int32_t*>(tile_sums + kMaxBags / kScanTile + 2);

  // The array keeps whatever the previous call left.  Offsets and tile sums
  // are fully rewritten by the scan; the status record has to start at zero.
  cudaError_t e = cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), stream);
  if (e != cudaSuccess) {
    return fail_cuda(e, "status clear");
  }
  e = launch_length_scan(lengths, cfg->offset_bytes, output_size, offsets, tile_sums, stream);
  if (e != cudaSuccess) {
    return fail_cuda(e, "length scan launch");
  }
  // From here on this is the offsets flavour reading the scanned int64 offsets.
  fbgemm_b200_spmdm_config scanned = *cfg;
  scanned.use_offsets = 1;
  scanned.offset_bytes = 8;
  DeviceBuffer unused;  // only the lengths flavour of enqueue_lookup would grow it
  int rc = enqueue_lookup(&scanned, output_size, index_size, data_size, input, indices, offsets, weights, out,
                          compressed_indices_table, status, unused, stream);
  if (rc) {
    return rc;
  }
  int32_t rec[4] = {0, 0, 0, 0};  // pageable stack memory: the copy below allocates nothing
  e = cudaMemcpyAsync(rec, status, sizeof(rec), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) {
    e = cudaStreamSynchronize(stream);
  }
  if (e != cudaSuccess) {
    return fail_cuda(e, "status read");
  }
  return rec[0] == 0 ? 1 : 0;
}

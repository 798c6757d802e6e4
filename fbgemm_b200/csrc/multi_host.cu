// Several tables per call on HOST pointers: what the reference's multi-table
// caller is given (host tensors in, output[B, total_D] out,
// fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:208-280,343-473),
// with the tables resident in HBM.  One step of a handle:
//
//   indices / offsets / weights of every table  --H2D-->  the handle's staging block
//   one lookup per table (spread over side streams), pooled rows stored into
//   `out_dev` - or, table-wise sharded, into the peers' buffers
//   [sharded]  publish "my rows for step s are stored" to every peer, wait
//              until every peer has published the same for my slice
//   out_dev  --D2H-->  the caller's host buffer
//   [sharded]  publish "I have consumed step s" to every peer; the next step's
//              lookups wait for those before they overwrite the buffers
//
// Everything is enqueued on the handle's own stream; submit returns at once and
// wait blocks until the rows are in the caller's buffer.  Two handles with two
// output buffers pipeline the transfers of one step behind the kernels of the
// other.
#include <cstring>
#include <new>
#include <vector>

#include "context.h"

using namespace fbgemm_b200;

namespace {
constexpr int kSideStreams = 3;
size_t up16(size_t v) {
  return (v + 15) & ~size_t(15);
}
// Consecutive host arrays that touch or overlap in memory go up as one copy.
struct HostRun {
  const uint8_t* src;
  size_t bytes;
  size_t at;  // byte offset inside the staging block
};
}  // namespace

struct fbgemm_b200_multi_host {
  fbgemm_b200_ctx* ctx = nullptr;
  int device = 0;
  int slot = 0;
  std::vector<fbgemm_b200_table_call> calls;
  std::vector<std::vector<void*>> peer_out;  // copies of the callers' pointer arrays
  std::vector<int64_t> capacity;             // indices a table's staging can hold
  std::vector<size_t> idx_at, off_at, w_at;  // this step's byte offsets inside the staging block
  std::vector<HostRun> runs;                 // this step's uploads
  std::vector<const void*> d_idx, d_off;     // this step's arrays as the lookups see them (device)
  std::vector<const float*> d_w;
  DeviceBuffer staging;
  int num_peers = 0;
  int64_t bags_per_peer = 0;
  void* out_dev = nullptr;
  size_t out_bytes = 0;
  bool has_sync = false;
  std::vector<void*> ready_flags, ack_flags;
  const void* ready_local = nullptr;
  const void* ack_local = nullptr;
  uint64_t timeout_us = 0;
  uint64_t step = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t side[kSideStreams] = {};
  cudaEvent_t fork = nullptr;
  cudaEvent_t join[kSideStreams] = {};
  PinnedBuffer h_status;
  bool busy = false;
  cudaEvent_t mark[4] = {};  // step start, uploads done, rows complete, download done
  bool timed = false;        // the marks belong to a step that wait() has returned
};

namespace {

// One lookup per table on device arrays, round-robin over `stream` and the handle's side streams, which are forked
// from `stream` and joined back into it.
int fan_out_lookups(fbgemm_b200_multi_host* h, cudaStream_t stream, const void* const* idx, const void* const* off,
                    const float* const* w, const int64_t* index_sizes, int32_t* status) {
  cudaError_t e = cudaEventRecord(h->fork, stream);
  for (int i = 0; i < kSideStreams && e == cudaSuccess; ++i) {
    e = cudaStreamWaitEvent(h->side[i], h->fork, 0);
  }
  if (e != cudaSuccess) {
    return fail_cuda(e, "multi-table step: fork");
  }
  DeviceBuffer unused;  // offsets mode: no scan scratch
  const size_t T = h->calls.size();
  for (size_t t = 0; t < T; ++t) {
    const fbgemm_b200_table_call& c = h->calls[t];
    const size_t k = t % (kSideStreams + 1);
    cudaStream_t s = k == 0 ? stream : h->side[k - 1];
    const int rc = enqueue_lookup(&c.cfg, c.output_size, index_sizes[t], c.data_size, c.input, idx[t], off[t],
                                  c.cfg.has_weight ? w[t] : nullptr, h->num_peers > 0 ? nullptr : c.out,
                                  c.compressed_indices_table, status, unused, s,
                                  h->num_peers > 0 ? h->peer_out[t].data() : nullptr, h->num_peers, h->bags_per_peer);
    if (rc) {
      return rc;
    }
  }
  for (int i = 0; i < kSideStreams && e == cudaSuccess; ++i) {
    e = cudaEventRecord(h->join[i], h->side[i]);
    if (e == cudaSuccess) {
      e = cudaStreamWaitEvent(stream, h->join[i], 0);
    }
  }
  return e == cudaSuccess ? 0 : fail_cuda(e, "multi-table step: join");
}

}  // namespace

extern "C" {

void fbgemm_b200_multi_host_destroy(fbgemm_b200_multi_host* h) {
  if (!h) {
    return;
  }
  DeviceGuard guard(h->device);
  if (h->stream) {
    cudaStreamSynchronize(h->stream);
  }
  for (int i = 0; i < kSideStreams; ++i) {
    if (h->side[i]) {
      cudaStreamDestroy(h->side[i]);
    }
    if (h->join[i]) {
      cudaEventDestroy(h->join[i]);
    }
  }
  if (h->fork) {
    cudaEventDestroy(h->fork);
  }
  for (cudaEvent_t m : h->mark) {
    if (m) {
      cudaEventDestroy(m);
    }
  }
  if (h->stream) {
    cudaStreamDestroy(h->stream);
  }
  cudaFree(h->staging.ptr);
  cudaFreeHost(h->h_status.ptr);
  delete h;
}

int fbgemm_b200_multi_host_create(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_table_call* calls,
    int32_t num_tables,
    const int64_t* index_capacity,
    int32_t num_peers,
    int64_t bags_per_peer,
    void* out_dev,
    size_t out_bytes,
    const fbgemm_b200_peer_sync* sync,
    int slot,
    fbgemm_b200_multi_host** out) {
  if (out) {
    *out = nullptr;
  }
  if (!ctx || !out || !calls || !index_capacity || num_tables <= 0 || num_peers < 0 ||
      num_peers > FBGEMM_B200_MAX_PEERS || slot < 0 || slot >= FBGEMM_B200_USER_SLOTS || !out_dev || out_bytes == 0) {
    set_error("multi_host_create: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  if (sync && (sync->num_peers != num_peers || num_peers == 0 || !sync->ready_flags || !sync->ready_local ||
               !sync->ack_flags || !sync->ack_local)) {
    set_error("multi_host_create: the peer counters must describe the same peers as the lookups");
    return FBGEMM_B200_EINVAL;
  }
  auto* h = new (std::nothrow) fbgemm_b200_multi_host;
  if (!h) {
    set_error("out of host memory");
    return FBGEMM_B200_ENOMEM;
  }
  h->ctx = ctx;
  h->device = ctx->device;
  h->slot = slot;
  h->num_peers = num_peers;
  h->bags_per_peer = bags_per_peer;
  h->out_dev = out_dev;
  h->out_bytes = out_bytes;
  size_t at = 0;
  for (int t = 0; t < num_tables; ++t) {
    const fbgemm_b200_table_call& c = calls[t];
    int rc = fbgemm_b200_spmdm_check_config(&c.cfg);
    if (rc == 0 && (!c.cfg.use_offsets || c.cfg.no_bag || c.cfg.absolute_offsets || index_capacity[t] < 0 ||
                    c.output_size <= 0 || !c.input || (num_peers > 0 ? !c.peer_out : !c.out) ||
                    (num_peers > 0 && c.compressed_indices_table))) {
      set_error("multi_host_create: a table needs offsets, bags, a resident table and an output (peer) pointer");
      rc = FBGEMM_B200_EINVAL;
    }
    if (rc) {
      delete h;
      return rc;
    }
    h->calls.push_back(c);
    h->peer_out.emplace_back();
    if (num_peers > 0) {
      h->peer_out.back().assign(c.peer_out, c.peer_out + num_peers);
    }
    h->capacity.push_back(index_capacity[t]);
    // every array may start on its own 16-byte line, shifted by its host address modulo 16
    at += up16((size_t)index_capacity[t] * c.cfg.index_bytes) + 32;
    at += up16((size_t)(c.output_size + 1) * c.cfg.offset_bytes) + 32;
    at += c.cfg.has_weight ? up16((size_t)index_capacity[t] * sizeof(float)) + 32 : 0;
  }
  h->idx_at.assign((size_t)num_tables, 0);
  h->off_at.assign((size_t)num_tables, 0);
  h->w_at.assign((size_t)num_tables, 0);
  h->d_idx.assign((size_t)num_tables, nullptr);
  h->d_off.assign((size_t)num_tables, nullptr);
  h->d_w.assign((size_t)num_tables, nullptr);
  if (sync) {
    h->has_sync = true;
    h->ready_flags.assign(sync->ready_flags, sync->ready_flags + num_peers);
    h->ack_flags.assign(sync->ack_flags, sync->ack_flags + num_peers);
    h->ready_local = sync->ready_local;
    h->ack_local = sync->ack_local;
    h->timeout_us = sync->timeout_us ? sync->timeout_us : 2000000;
  }
  DeviceGuard guard(ctx->device);
  cudaError_t e = reserve(h->staging, at);
  if (e == cudaSuccess) {
    e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
  }
  if (e == cudaSuccess) {
    e = cudaEventCreateWithFlags(&h->fork, cudaEventDisableTiming);
  }
  for (int i = 0; i < kSideStreams && e == cudaSuccess; ++i) {
    e = cudaStreamCreateWithFlags(&h->side[i], cudaStreamNonBlocking);
    if (e == cudaSuccess) {
      e = cudaEventCreateWithFlags(&h->join[i], cudaEventDisableTiming);
    }
  }
  for (int i = 0; i < 4 && e == cudaSuccess; ++i) {
    e = cudaEventCreate(&h->mark[i]);
  }
  if (e == cudaSuccess) {
    e = reserve(h->h_status, 16);
  }
  if (e != cudaSuccess) {
    const int rc = fail_cuda(e, "multi_host_create");
    fbgemm_b200_multi_host_destroy(h);
    return rc;
  }
  *out = h;
  return 0;
}

int fbgemm_b200_multi_host_submit(
    fbgemm_b200_multi_host* h,
    const void* const* indices,
    const void* const* offsets,
    const float* const* weights,
    const int64_t* index_sizes,
    void* out_host) {
  if (!h || !indices || !offsets || !index_sizes || !out_host) {
    set_error("multi_host_submit: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  if (h->busy) {
    set_error("the handle has a step in flight; call fbgemm_b200_multi_host_wait first");
    return FBGEMM_B200_EBUSY;
  }
  const size_t T = h->calls.size();
  for (size_t t = 0; t < T; ++t) {
    const fbgemm_b200_table_call& c = h->calls[t];
    if (index_sizes[t] < 0 || index_sizes[t] > h->capacity[t] || !offsets[t] || (index_sizes[t] > 0 && !indices[t]) ||
        (c.cfg.has_weight && index_sizes[t] > 0 && (!weights || !weights[t]))) {
      set_error("multi_host_submit: table " + std::to_string(t) + ": null array or more indices than the handle's capacity");
      return FBGEMM_B200_EINVAL;
    }
  }
  DeviceGuard guard(h->device);
  fbgemm_b200_ctx* ctx = h->ctx;
  int32_t* status = ctx->status + 4 * h->slot;
  uint8_t* st = static_cast<uint8_t*>(h->staging.ptr);
  const uint64_t step = h->step + 1;
  h->timed = false;
  cudaError_t e = cudaEventRecord(h->mark[0], h->stream);
  // The buffers this step writes were last read as step - 1: wait for every consumer's word.
  if (e == cudaSuccess && h->has_sync) {
    e = launch_peer_wait(h->ack_local, h->num_peers, step - 1, h->timeout_us, status, h->stream);
  }
  // Lay the step's arrays out in the staging block the way they lie in host memory: arrays that touch or overlap
  // there (per-table views of ONE indices, ONE offsets and ONE weights array, which is what the reference's
  // multi-table caller holds) go up as one copy.  The number of copies matters: each waits for its own completion
  // word, and while another handle's rows are on their way to the host those words queue behind that transfer -
  // measured with 64 separate tables, 192 copies took 7.7 ms beside a 330 MB download and 2.9 ms alone.
  for (int merge = 1; merge >= 0; --merge) {
    h->runs.clear();
    size_t cursor = 0;
    auto place = [&](const void* host, size_t bytes) -> size_t {
      const uint8_t* src = static_cast<const uint8_t*>(host);
      if (merge && !h->runs.empty()) {
        HostRun& r = h->runs.back();
        if (src >= r.src && src <= r.src + r.bytes) {
          const size_t off = (size_t)(src - r.src);
          r.bytes = off + bytes > r.bytes ? off + bytes : r.bytes;
          cursor = r.at + r.bytes;
          return r.at + off;
        }
      }
      cursor = up16(cursor) + (reinterpret_cast<uintptr_t>(src) & 15);
      h->runs.push_back(HostRun{src, bytes, cursor});
      cursor += bytes;
      return cursor - bytes;
    };
    // all indices, then all offsets, then all weights: the order in which a caller's three arrays are contiguous
    for (size_t t = 0; t < T; ++t) {
      const size_t n = (size_t)index_sizes[t];
      h->idx_at[t] = n ? place(indices[t], n * h->calls[t].cfg.index_bytes) : 0;
    }
    for (size_t t = 0; t < T; ++t) {
      h->off_at[t] = place(offsets[t], (size_t)(h->calls[t].output_size + 1) * h->calls[t].cfg.offset_bytes);
    }
    for (size_t t = 0; t < T; ++t) {
      const size_t n = (size_t)index_sizes[t];
      h->w_at[t] = h->calls[t].cfg.has_weight && n ? place(weights[t], n * sizeof(float)) : 0;
    }
    for (size_t k = 0; k < h->runs.size() && e == cudaSuccess; ++k) {
      const HostRun& r = h->runs[k];
      e = cudaMemcpyAsync(st + r.at, r.src, r.bytes, cudaMemcpyHostToDevice, h->stream);
    }
    // A merged range may span two page-locked allocations that happen to be neighbours; if the runtime refuses such
    // a copy, send every array on its own.
    if (e == cudaErrorInvalidValue && merge && h->runs.size() < 3 * T) {
      cudaGetLastError();
      e = cudaSuccess;
      continue;
    }
    break;
  }
  if (e != cudaSuccess) {
    return fail_cuda(e, "multi_host_submit: input upload");
  }
  e = cudaEventRecord(h->mark[1], h->stream);
  if (e != cudaSuccess) {
    return fail_cuda(e, "multi_host_submit");
  }
  for (size_t t = 0; t < T; ++t) {
    h->d_idx[t] = st + h->idx_at[t];
    h->d_off[t] = st + h->off_at[t];
    h->d_w[t] = reinterpret_cast<const float*>(st + h->w_at[t]);
  }
  if (const int rc = fan_out_lookups(h, h->stream, h->d_idx.data(), h->d_off.data(), h->d_w.data(), index_sizes, status)) {
    return rc;
  }
  if (e == cudaSuccess && h->has_sync) {
    e = launch_peer_signal(h->ready_flags.data(), h->num_peers, step, h->stream);
    if (e == cudaSuccess) {
      e = launch_peer_wait(h->ready_local, h->num_peers, step, h->timeout_us, status, h->stream);
    }
  }
  if (e == cudaSuccess) {
    e = cudaEventRecord(h->mark[2], h->stream);
  }
  if (e == cudaSuccess) {
    e = cudaMemcpyAsync(out_host, h->out_dev, h->out_bytes, cudaMemcpyDeviceToHost, h->stream);
  }
  if (e == cudaSuccess) {
    e = cudaEventRecord(h->mark[3], h->stream);
  }
  if (e == cudaSuccess && h->has_sync) {
    e = launch_peer_signal(h->ack_flags.data(), h->num_peers, step, h->stream);
  }
  if (e == cudaSuccess) {
    e = launch_status_to_host(status, static_cast<int32_t*>(h->h_status.ptr), h->stream);
  }
  if (e != cudaSuccess) {
    return fail_cuda(e, "multi_host_submit");
  }
  h->step = step;
  h->busy = true;
  return 0;
}

int64_t fbgemm_b200_multi_host_step_device(
    fbgemm_b200_multi_host* h,
    const void* const* indices,
    const void* const* offsets,
    const float* const* weights,
    const int64_t* index_sizes,
    int release,
    void* stream_) {
  if (!h || !indices || !offsets || !index_sizes) {
    set_error("multi_host_step_device: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  if (h->busy) {
    set_error("the handle has a host-array step in flight; call fbgemm_b200_multi_host_wait first");
    return FBGEMM_B200_EBUSY;
  }
  const size_t T = h->calls.size();
  for (size_t t = 0; t < T; ++t) {
    const fbgemm_b200_table_call& c = h->calls[t];
    if (index_sizes[t] < 0 || !offsets[t] || (index_sizes[t] > 0 && !indices[t]) ||
        (c.cfg.has_weight && index_sizes[t] > 0 && (!weights || !weights[t]))) {
      set_error("multi_host_step_device: table " + std::to_string(t) + ": null array");
      return FBGEMM_B200_EINVAL;
    }
  }
  DeviceGuard guard(h->device);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int32_t* status = h->ctx->status + 4 * h->slot;
  const uint64_t step = h->step + 1;
  cudaError_t e = cudaSuccess;
  if (h->has_sync) {
    e = launch_peer_wait(h->ack_local, h->num_peers, step - 1, h->timeout_us, status, stream);
    if (e != cudaSuccess) {
      return fail_cuda(e, "multi_host_step_device");
    }
  }
  for (size_t t = 0; t < T; ++t) {
    h->d_w[t] = weights ? weights[t] : nullptr;
  }
  if (const int rc = fan_out_lookups(h, stream, indices, offsets, h->d_w.data(), index_sizes, status)) {
    return rc;
  }
  if (h->has_sync) {
    e = launch_peer_signal(h->ready_flags.data(), h->num_peers, step, stream);
    if (e == cudaSuccess) {
      e = launch_peer_wait(h->ready_local, h->num_peers, step, h->timeout_us, status, stream);
    }
    if (e == cudaSuccess && release) {
      e = launch_peer_signal(h->ack_flags.data(), h->num_peers, step, stream);
    }
    if (e != cudaSuccess) {
      return fail_cuda(e, "multi_host_step_device");
    }
  }
  h->step = step;
  return (int64_t)step;
}

int fbgemm_b200_multi_host_release(fbgemm_b200_multi_host* h, int64_t step, void* stream) {
  if (!h || step <= 0 || (uint64_t)step > h->step) {
    set_error("multi_host_release: not a step of this handle");
    return FBGEMM_B200_EINVAL;
  }
  if (!h->has_sync) {
    return 0;
  }
  DeviceGuard guard(h->device);
  const cudaError_t e = launch_peer_signal(h->ack_flags.data(), h->num_peers, (uint64_t)step, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : fail_cuda(e, "multi_host_release");
}

int fbgemm_b200_multi_host_wait(fbgemm_b200_multi_host* h, int32_t* info) {
  if (!h || !h->busy) {
    set_error("multi_host_wait: nothing in flight");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(h->device);
  h->busy = false;
  const cudaError_t e = cudaStreamSynchronize(h->stream);
  if (e != cudaSuccess) {
    return fail_cuda(e, "multi_host_wait");
  }
  h->timed = true;
  const int32_t* rec = static_cast<const int32_t*>(h->h_status.ptr);
  if (info) {
    std::memcpy(info, rec, 16);
  }
  if (rec[0] != 0) {
    cudaMemsetAsync(h->ctx->status + 4 * h->slot, 0, 16, h->stream);
  }
  return rec[0] == 0 ? 1 : 0;
}

/* ---- buffers that peer processes can map ------------------------------------------- */

int fbgemm_b200_multi_host_last_step_ms(fbgemm_b200_multi_host* h, float* ms) {
  if (!h || !ms || !h->timed) {
    set_error("multi_host_last_step_ms: no step has been waited for");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(h->device);
  for (int i = 0; i < 3; ++i) {
    const cudaError_t e = cudaEventElapsedTime(&ms[i], h->mark[i], h->mark[i + 1]);
    if (e != cudaSuccess) {
      return fail_cuda(e, "multi_host_last_step_ms");
    }
  }
  return 0;
}

int fbgemm_b200_peer_buffer_alloc(fbgemm_b200_ctx* ctx, size_t bytes, void** ptr, unsigned char* handle) {
  if (!ctx || !ptr || !handle || bytes == 0) {
    set_error("peer_buffer_alloc: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == FBGEMM_B200_IPC_HANDLE_BYTES, "handle size");
  DeviceGuard guard(ctx->device);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) {
    e = cudaMemset(p, 0, bytes);
  }
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) {
    e = cudaIpcGetMemHandle(&h, p);
  }
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail_cuda(e, "peer_buffer_alloc");
  }
  std::memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return 0;
}

int fbgemm_b200_peer_buffer_open(fbgemm_b200_ctx* ctx, const unsigned char* handle, void** ptr) {
  if (!ctx || !ptr || !handle) {
    set_error("peer_buffer_open: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    return fail_cuda(e, "peer_buffer_open");
  }
  *ptr = p;
  return 0;
}

int fbgemm_b200_peer_buffer_close(fbgemm_b200_ctx* ctx, void* ptr) {
  if (!ctx || !ptr) {
    set_error("peer_buffer_close: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? 0 : fail_cuda(e, "peer_buffer_close");
}

int fbgemm_b200_peer_buffer_free(fbgemm_b200_ctx* ctx, void* ptr) {
  if (!ctx || !ptr) {
    set_error("peer_buffer_free: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? 0 : fail_cuda(e, "peer_buffer_free");
}

/* ---- the counters on their own --------------------------------------------------- */

int fbgemm_b200_peer_signal(fbgemm_b200_ctx* ctx, void* const* flags, int num_flags, uint64_t value, void* stream) {
  if (!ctx || !flags || num_flags < 1 || num_flags > FBGEMM_B200_MAX_PEERS) {
    set_error("peer_signal: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  for (int i = 0; i < num_flags; ++i) {
    if (!flags[i] || reinterpret_cast<uintptr_t>(flags[i]) % 8 != 0) {
      set_error("peer_signal: a counter address is null or not 8-byte aligned");
      return FBGEMM_B200_EINVAL;
    }
  }
  DeviceGuard guard(ctx->device);
  const cudaError_t e = launch_peer_signal(flags, num_flags, value, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : fail_cuda(e, "peer_signal launch");
}

int fbgemm_b200_peer_wait(fbgemm_b200_ctx* ctx, const void* flags, int num_flags, uint64_t value, uint64_t timeout_us,
                          int slot, void* stream) {
  if (!ctx || !flags || reinterpret_cast<uintptr_t>(flags) % 8 != 0 || num_flags < 1 ||
      num_flags > FBGEMM_B200_MAX_PEERS || slot < 0 || slot >= FBGEMM_B200_USER_SLOTS || timeout_us == 0 ||
      timeout_us > 60ull * 1000 * 1000) {
    set_error("peer_wait: bad argument (the time limit is 1 us .. 60 s)");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  const cudaError_t e =
      launch_peer_wait(flags, num_flags, value, timeout_us, ctx->status + 4 * slot, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : fail_cuda(e, "peer_wait launch");
}

}  // extern "C"

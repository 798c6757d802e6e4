// The C ABI of libfbgemm_b200.so: context, status slots, table registry,
// device-pointer and host-pointer functor calls.  See
// include/fbgemm_b200/embedding_c_api.h for the contract of each entry point.
#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>
#include <unordered_map>
#include <type_traits>
#include <vector>

#include "context.h"

namespace fbgemm_b200 {

namespace {
thread_local std::string t_error;
}

void set_error(const std::string& msg) {
  t_error = msg;
}

int fail_cuda(cudaError_t e, const char* what) {
  set_error(std::string(what) + ": " + cudaGetErrorString(e));
  return e == cudaErrorMemoryAllocation ? FBGEMM_B200_ENOMEM : FBGEMM_B200_ECUDA;
}

int max_chunks_per_bag(int bit_rate);  // spmdm_kernels.cu

}  // namespace fbgemm_b200

using namespace fbgemm_b200;

namespace {

// Status slots: callers own [0, FBGEMM_B200_USER_SLOTS); then one for the
// index remap; the last FBGEMM_B200_HOST_LANES belong to the host-pointer lanes.
constexpr int kRemapSlot = FBGEMM_B200_USER_SLOTS;
static_assert(FBGEMM_B200_USER_SLOTS + 1 + FBGEMM_B200_HOST_LANES == FBGEMM_B200_STATUS_SLOTS, "slot ranges");

// The lengths-mode scratch of `stream` (ctx->mu held).  A context that has
// seen very many streams drops the scratch of all of them once, after waiting
// for the device, instead of growing without bound.
DeviceBuffer& scan_scratch_of(fbgemm_b200_ctx* ctx, cudaStream_t stream) {
  constexpr size_t kMaxStreams = 256;
  auto it = ctx->scan.find(stream);
  if (it == ctx->scan.end() && ctx->scan.size() >= kMaxStreams) {
    cudaDeviceSynchronize();
    for (auto& kv : ctx->scan) {
      cudaFree(kv.second.ptr);
    }
    ctx->scan.clear();
  }
  return ctx->scan[stream];
}

int check_config(const fbgemm_b200_spmdm_config* c, Derived* d) {
  if (!c) {
    set_error("null config");
    return FBGEMM_B200_EINVAL;
  }
  if (c->in_dtype == FBGEMM_B200_IN_QUANTIZED && c->bit_rate != 8 && c->bit_rate != 4 && c->bit_rate != 2) {
    set_error("bit_rate must be 8, 4 or 2");
    return FBGEMM_B200_EINVAL;
  }
  if ((c->index_bytes != 4 && c->index_bytes != 8) || (c->offset_bytes != 4 && c->offset_bytes != 8)) {
    set_error("index/offset types must be int32 or int64");
    return FBGEMM_B200_EINVAL;
  }
  if (c->out_dtype != FBGEMM_B200_OUT_F32 && c->out_dtype != FBGEMM_B200_OUT_F16 &&
      c->out_dtype != FBGEMM_B200_OUT_BF16 && c->out_dtype != FBGEMM_B200_OUT_U8) {
    set_error("output type must be fp32, fp16, bf16 or (no_bag) u8");
    return FBGEMM_B200_EINVAL;
  }
  if (c->out_dtype == FBGEMM_B200_OUT_U8 &&
      (!c->no_bag || c->in_dtype != FBGEMM_B200_IN_QUANTIZED || (c->bit_rate != 8 && c->bit_rate != 4) ||
       c->scale_bias_first)) {
    set_error("8-bit output is the no_bag row copy of 8-bit or 4-bit rows");
    return FBGEMM_B200_EINVAL;
  }
  if (c->absolute_offsets && (!c->use_offsets || c->no_bag || c->is_weight_positional)) {
    set_error("absolute_offsets goes with use_offsets, bags and per-index weights");
    return FBGEMM_B200_EINVAL;
  }
  if (c->no_bag && c->bit_rate != 8 && c->in_dtype == FBGEMM_B200_IN_QUANTIZED &&
      c->out_dtype != FBGEMM_B200_OUT_U8) {
    // EmbeddingSpMDMNBit_ref: "no_bag is only supported for int4 to int4", a raw row copy
    set_error("no_bag is provided for 8-bit rows with fp32/fp16/bf16 output");
    return FBGEMM_B200_EINVAL;
  }
  if (c->block_size <= 0 || c->block_size > (1 << 20)) {
    set_error("block_size out of range");
    return FBGEMM_B200_EINVAL;
  }
  const bool plain = c->in_dtype != FBGEMM_B200_IN_QUANTIZED;
  if (c->in_dtype < 0 || c->in_dtype > FBGEMM_B200_IN_FP8) {
    set_error("unknown in_dtype");
    return FBGEMM_B200_EINVAL;
  }
  if (c->in_dtype == FBGEMM_B200_IN_FP8 &&
      (c->fp8_exponent_bits < 1 || c->fp8_exponent_bits > 7 || c->fp8_exponent_bias < 0 || c->fp8_exponent_bias > 253 ||
       c->no_bag || c->scale_bias_first)) {
    set_error("FP8 rows: exponent_bits 1..7, exponent_bias 0..253, bags only");
    return FBGEMM_B200_EINVAL;
  }
  const int ebytes = c->in_dtype == FBGEMM_B200_IN_F32 ? 4 : (c->in_dtype == FBGEMM_B200_IN_FP8 ? 1 : 2);
  const int epb = plain ? 1 : 8 / c->bit_rate;
  const int64_t data_bytes = plain ? c->block_size * ebytes : (c->block_size + epb - 1) / epb;
  if (!plain && (data_bytes + 3) / 4 > max_chunks_per_bag(c->bit_rate)) {
    set_error("block_size too large for the sm_100a kernels (1024 columns at most)");
    return FBGEMM_B200_EINVAL;
  }
  const int sb_bytes = plain ? 0 : ((c->bit_rate == 8 && !c->scale_bias_first) ? 8 : 4);
  const int64_t in_stride = c->input_stride == -1 ? data_bytes + sb_bytes : c->input_stride;
  const int64_t out_stride = c->output_stride == -1 ? c->block_size : c->output_stride;
  if (in_stride < data_bytes + sb_bytes || (plain && in_stride % ebytes != 0)) {
    set_error("input_stride smaller than a row (or not a whole number of elements)");
    return FBGEMM_B200_EINVAL;
  }
  if (out_stride < c->block_size && c->out_dtype != FBGEMM_B200_OUT_U8) {
    set_error("output_stride smaller than block_size");
    return FBGEMM_B200_EINVAL;
  }
  if (out_stride <= 0) {
    set_error("output_stride must be positive");
    return FBGEMM_B200_EINVAL;
  }
  if (d) {
    d->data_bytes = (int)data_bytes;
    d->sb_bytes = sb_bytes;
    d->input_stride = in_stride;
    d->output_stride = out_stride;
  }
  return 0;
}

}  // namespace

// Validate one functor call and fill the kernel parameters for it (everything
// but the offsets, which depend on the offsets/lengths mode).
int fbgemm_b200::build_lookup_params(
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const float* weights,
    void* out,
    const int32_t* cit,
    int32_t* status,
    void* const* peer_out,
    int num_peers,
    int64_t bags_per_peer,
    SpmdmParams* params) {
  SpmdmParams& p = *params;
  Derived d;
  int rc = check_config(cfg, &d);
  if (rc) {
    return rc;
  }
  if (output_size < 0 || index_size < 0 || data_size < 0) {
    set_error("negative size");
    return FBGEMM_B200_EINVAL;
  }
  if (cfg->has_weight && !weights && index_size > 0) {
    set_error("has_weight set but weights is null");
    return FBGEMM_B200_EINVAL;
  }
  if ((index_size > 0 && (!input || !indices)) || (output_size > 0 && !out && num_peers <= 0)) {
    set_error("null table, indices or output pointer");
    return FBGEMM_B200_EINVAL;
  }
  if (cfg->no_bag && (output_size != index_size || cit || cfg->is_weight_positional)) {
    set_error("no_bag: one index per output row, dense table, no positional weights");
    return FBGEMM_B200_EINVAL;
  }
  if (cit && cfg->scale_bias_first) {
    set_error("row-wise sparse lookup takes rows with scale, bias last");
    return FBGEMM_B200_EINVAL;
  }
  if (cit && (cfg->out_dtype != FBGEMM_B200_OUT_F32 || cfg->output_stride != -1 || cfg->input_stride != -1)) {
    // EmbeddingSpMDMRowWiseSparseKernelSignature: float* out, dense strides.
    set_error("row-wise sparse lookup takes fp32 output and default strides");
    return FBGEMM_B200_EINVAL;
  }

  p = SpmdmParams{};
  p.table = static_cast<const uint8_t*>(input);
  p.indices = indices;
  p.weights = cfg->has_weight ? weights : nullptr;
  p.cit = cit;
  p.out = out;
  p.status = status;
  p.data_size = data_size;
  p.input_stride = d.input_stride;
  p.output_stride = d.output_stride;
  p.output_size = output_size;
  p.index_size = index_size;
  p.block_size = (int32_t)cfg->block_size;
  p.in_kind = cfg->in_dtype;
  p.fp8_exponent_bits = cfg->fp8_exponent_bits;
  p.fp8_exponent_bias = cfg->fp8_exponent_bias;
  if (cfg->in_dtype != FBGEMM_B200_IN_QUANTIZED) {
    const int ebytes = cfg->in_dtype == FBGEMM_B200_IN_F32 ? 4 : (cfg->in_dtype == FBGEMM_B200_IN_FP8 ? 1 : 2);
    // EmbeddingSpMDMRowWiseSparse_ref exists for float and fp16 rows only (src/RefImplementations.cc:1688-1743).
    const bool map_ok = !cit || cfg->in_dtype == FBGEMM_B200_IN_F32 || cfg->in_dtype == FBGEMM_B200_IN_F16;
    if (!map_ok || reinterpret_cast<uintptr_t>(input) % ebytes != 0) {
      set_error("unquantized tables: a pruning map only with fp32 or fp16 rows, and the table must be aligned to "
                "its element type");
      return FBGEMM_B200_EINVAL;
    }
  }
  p.data_bytes = d.data_bytes;
  p.row_bytes = d.data_bytes + d.sb_bytes;
  p.data_row_off = cfg->scale_bias_first ? d.sb_bytes : 0;
  p.sb_row_off = cfg->scale_bias_first ? 0 : d.data_bytes;
  // In the shared-memory stage of the generic kernel the payload comes first
  // and scale,bias sit at the next 4-byte boundary, unless whole rows are
  // copied as they are (copy_width > 0 below).
  p.data_off = 0;
  p.sb_off = (d.data_bytes + 3) & ~3;
  p.pitch = p.sb_off + d.sb_bytes;

  // cp.async granule: the widest of 16/8/4 bytes that divides the table
  // address, the row pitch and the row width; otherwise byte loads.
  const uintptr_t base = reinterpret_cast<uintptr_t>(input);
  p.copy_width = 0;
  if (d.data_bytes % 4 == 0) {
    for (int w = 16; w >= 4; w >>= 1) {
      if (base % w == 0 && d.input_stride % w == 0 && p.row_bytes % w == 0) {
        p.copy_width = w;
        break;
      }
    }
  }
  if (p.copy_width > 0) {
    p.data_off = p.data_row_off;
    p.sb_off = p.sb_row_off;
  }
  if (p.copy_width > 4) {
    p.pitch = (p.pitch + p.copy_width - 1) / p.copy_width * p.copy_width;
  }

  uint32_t flags = 0;
  flags |= cfg->index_bytes == 8 ? kIdx64 : 0;
  flags |= cfg->out_dtype == FBGEMM_B200_OUT_F16 ? kOutHalf : 0;
  flags |= cfg->out_dtype == FBGEMM_B200_OUT_BF16 ? kOutBf16 : 0;
  flags |= cfg->scale_bias_first ? kSbFirst : 0;
  flags |= cfg->no_bag ? kNoBag : 0;
  flags |= cfg->absolute_offsets ? kAbsOffsets : 0;
  flags |= p.weights ? kWeighted : 0;
  flags |= (p.weights && cfg->is_weight_positional) ? kPositional : 0;
  flags |= (cfg->normalize_by_lengths && !cfg->no_bag) ? kNormalize : 0;
  flags |= cit ? kPruned : 0;
  const size_t esize = cfg->out_dtype == FBGEMM_B200_OUT_F32 ? 4 : 2;
  bool out_aligned = (d.output_stride * esize) % 16 == 0;
  if (num_peers > 0) {
    if (!peer_out || num_peers > FBGEMM_B200_MAX_PEERS || bags_per_peer <= 0 ||
        (int64_t)num_peers * bags_per_peer < output_size || cit) {
      set_error("bad peer output description");
      return FBGEMM_B200_EINVAL;
    }
    p.num_peers = num_peers;
    p.bags_per_peer = bags_per_peer;
    for (int i = 0; i < num_peers; ++i) {
      p.peer_out[i] = peer_out[i];
      out_aligned = out_aligned && reinterpret_cast<uintptr_t>(peer_out[i]) % 16 == 0;
    }
  } else {
    out_aligned = out_aligned && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  }
  if (out_aligned) {
    flags |= kOutVec;
  }
  p.flags = flags;
  return 0;
}

// Build the kernel parameters for one functor call and enqueue it.  All
// pointers are device pointers.  `scan` is the scratch for lengths mode.
int fbgemm_b200::enqueue_lookup(
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets_or_lengths,
    const float* weights,
    void* out,
    const int32_t* cit,
    int32_t* status,
    DeviceBuffer& scan,
    cudaStream_t stream,
    void* const* peer_out,
    int num_peers,
    int64_t bags_per_peer) {
  if (cfg && cfg->out_dtype == FBGEMM_B200_OUT_U8) {
    Derived d;
    const int rc = check_config(cfg, &d);
    if (rc) {
      return rc;
    }
    if (output_size < 0 || data_size < 0 || cit || num_peers > 0 || (output_size > 0 && (!input || !indices || !out))) {
      set_error("row copy: dense table, device pointers, no peers");
      return FBGEMM_B200_EINVAL;
    }
    if (output_size == 0) {
      return 0;
    }
    const int64_t width = cfg->bit_rate == 8 ? std::min(d.output_stride, d.input_stride) : d.input_stride;
    const int64_t pitch = cfg->bit_rate == 8 ? d.output_stride : d.input_stride;
    const cudaError_t e = launch_rows_copy(static_cast<const uint8_t*>(input), indices, cfg->index_bytes, output_size,
                                           data_size, d.input_stride, static_cast<uint8_t*>(out), pitch, width, status,
                                           stream);
    return e == cudaSuccess ? 0 : fail_cuda(e, "row copy launch");
  }
  SpmdmParams p;
  const int rc = build_lookup_params(cfg, output_size, index_size, data_size, input, indices, weights, out, cit, status,
                                     peer_out, num_peers, bags_per_peer, &p);
  if (rc) {
    return rc;
  }
  uint32_t flags = p.flags;
  if (!cfg->no_bag && !offsets_or_lengths) {
    set_error("null offsets (or lengths) pointer");
    return FBGEMM_B200_EINVAL;
  }
  if (cfg->no_bag) {
    p.offsets = nullptr;  // bag m is the single index m
  } else if (cfg->use_offsets) {
    p.offsets = offsets_or_lengths;
    flags |= cfg->offset_bytes == 8 ? kOff64 : 0;
  } else {
    // lengths -> int64 offsets in scratch
    const size_t need = ((size_t)output_size + 1 + scan_scratch_elems(output_size)) * sizeof(int64_t);
    cudaError_t e = reserve(scan, need);
    if (e != cudaSuccess) {
      return fail_cuda(e, "scratch for the length scan");
    }
    int64_t* offs = static_cast<int64_t*>(scan.ptr);
    e = launch_length_scan(offsets_or_lengths, cfg->offset_bytes, output_size, offs, offs + output_size + 1, stream);
    if (e != cudaSuccess) {
      return fail_cuda(e, "length scan launch");
    }
    p.offsets = offs;
    flags |= kOff64;
  }
  p.flags = flags;

  cudaError_t e = launch_spmdm(p, cfg->bit_rate, stream);
  if (e != cudaSuccess) {
    return fail_cuda(e, "lookup launch");
  }
  return 0;
}

namespace {

int pruned_lookup(
    bool hashmap,
    fbgemm_b200_ctx* ctx,
    int32_t T,
    int32_t B,
    const void* indices,
    const void* offsets,
    int32_t index_bytes,
    int64_t index_size,
    const void* map,
    int32_t map_bytes,
    const int64_t* map_offsets,
    void* dense_indices,
    int32_t slot,
    void* stream) {
  const char* what = hashmap ? "pruned_hashmap_lookup: bad argument" : "pruned_array_lookup: bad argument";
  if (!ctx || slot < 0 || slot >= FBGEMM_B200_STATUS_SLOTS) {
    set_error("bad context or status slot");
    return FBGEMM_B200_EINVAL;
  }
  const size_t map_align = hashmap ? 2 * (size_t)map_bytes : (size_t)map_bytes;
  if (T < 1 || B < 1 || (index_bytes != 4 && index_bytes != 8) || (map_bytes != 4 && map_bytes != 8) ||
      index_size < 0 || !offsets || !map_offsets || (index_size > 0 && (!indices || !dense_indices)) ||
      reinterpret_cast<uintptr_t>(map) % map_align != 0) {
    set_error(what);
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  const cudaError_t e =
      launch_pruned_lookup(hashmap, T, B, indices, offsets, index_bytes, index_size, map, map_bytes, map_offsets,
                           dense_indices, ctx->status + 4 * slot, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    return fail_cuda(e, "pruned index lookup launch");
  }
  return 0;
}

template <typename Index, typename Hash>
bool hashmap_insert(
    int32_t T,
    int32_t B,
    const Index* indices,
    const Index* dense,
    const Index* offsets,
    Hash* table,
    const int64_t* table_offsets) {
  using Unsigned = typename std::make_unsigned<Index>::type;
  bool ok = true;
  for (int32_t t = 0; t < T; ++t) {
    const int64_t first = table_offsets[t];
    const uint64_t capacity = (uint64_t)(table_offsets[t + 1] - first);
    if (capacity == 0) {
      continue;
    }
    Hash* slots = table + 2 * first;
    for (int64_t k = offsets[(int64_t)t * B]; k < (int64_t)offsets[(int64_t)(t + 1) * B]; ++k) {
      if (dense[k] == -1) {
        continue;
      }
      const Unsigned key = (Unsigned)indices[k];
      uint64_t h;
      if (sizeof(Index) == 8) {
        uint64_t x = (uint64_t)key;
        x ^= x >> 33;
        x *= 0xff51afd7ed558ccdULL;
        x ^= x >> 33;
        x *= 0xc4ceb9fe1a85ec53ULL;
        x ^= x >> 33;
        h = x;
      } else {
        uint32_t x = (uint32_t)key;
        x ^= x >> 16;
        x *= 0x85ebca6bu;
        x ^= x >> 13;
        x *= 0xc2b2ae35u;
        x ^= x >> 16;
        h = x;
      }
      uint64_t slot = h % capacity, tried = 0;
      while (tried < capacity && slots[2 * slot] != -1 && (int64_t)slots[2 * slot] != (int64_t)indices[k]) {
        slot = slot + 1 == capacity ? 0 : slot + 1;
        ++tried;
      }
      if (tried == capacity) {
        ok = false;
        continue;
      }
      slots[2 * slot] = (Hash)indices[k];
      slots[2 * slot + 1] = (Hash)dense[k];
    }
  }
  return ok;
}

}  // namespace

extern "C" {

int fbgemm_b200_ctx_create(int device, fbgemm_b200_ctx** out) {
  if (!out) {
    set_error("null ctx out");
    return FBGEMM_B200_EINVAL;
  }
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    set_error(std::string("no usable CUDA device: ") + cudaGetErrorString(e));
    return FBGEMM_B200_ECUDA;
  }
  if (device < 0 || device >= count) {
    set_error("device ordinal out of range");
    return FBGEMM_B200_EINVAL;
  }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    return fail_cuda(e, "cudaGetDeviceProperties");
  }
  if (prop.major != 10) {
    set_error("fbgemm_b200 kernels are built for sm_100a only; device is sm_" + std::to_string(prop.major) +
              std::to_string(prop.minor));
    return FBGEMM_B200_ECUDA;
  }
  DeviceGuard guard(device);
  auto* ctx = new (std::nothrow) fbgemm_b200_ctx();
  if (!ctx) {
    return FBGEMM_B200_ENOMEM;
  }
  ctx->device = device;
  const size_t sbytes = sizeof(int32_t) * 4 * FBGEMM_B200_STATUS_SLOTS;
  e = cudaMalloc(&ctx->status, sbytes);
  if (e == cudaSuccess) {
    e = cudaMemset(ctx->status, 0, sbytes);
  }
  if (e == cudaSuccess) {
    e = cudaMallocHost(&ctx->status_host, sbytes);
  }
  if (e != cudaSuccess) {
    fbgemm_b200_ctx_destroy(ctx);
    return fail_cuda(e, "status slots");
  }
  *out = ctx;
  return 0;
}

void fbgemm_b200_ctx_destroy(fbgemm_b200_ctx* ctx) {
  if (!ctx) {
    return;
  }
  DeviceGuard guard(ctx->device);
  cudaDeviceSynchronize();
  for (auto& l : ctx->lanes) {
    if (l.stream) {
      cudaStreamDestroy(l.stream);
    }
    cudaFree(l.d_in.ptr);
    cudaFree(l.d_out.ptr);
    cudaFree(l.d_scan.ptr);
    cudaFreeHost(l.h_in.ptr);
    cudaFreeHost(l.h_out.ptr);
    cudaFreeHost(l.h_status.ptr);
  }
  for (auto& kv : ctx->tables) {
    cudaFree(kv.second.buf.ptr);
  }
  for (auto& kv : ctx->scan) {
    cudaFree(kv.second.ptr);
  }
  cudaFree(ctx->remap_scratch.ptr);
  cudaFree(ctx->status);
  cudaFreeHost(ctx->status_host);
  delete ctx;
}

const char* fbgemm_b200_last_error(void) {
  return t_error.c_str();
}

uint64_t fbgemm_b200_launch_count(void) {
  return g_launch_count.load(std::memory_order_relaxed);
}

int fbgemm_b200_set_kernel_choice(int choice) {
  if (choice != FBGEMM_B200_KERNEL_AUTO && choice != FBGEMM_B200_KERNEL_GENERIC) {
    set_error("unknown kernel choice");
    return FBGEMM_B200_EINVAL;
  }
  return g_kernel_choice.exchange(choice, std::memory_order_relaxed);
}

int fbgemm_b200_spmdm_check_config(const fbgemm_b200_spmdm_config* cfg) {
  return check_config(cfg, nullptr);
}

int fbgemm_b200_spmdm_launch(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets_or_lengths,
    const float* weights,
    void* out,
    const int32_t* compressed_indices_table,
    int slot,
    void* stream) {
  if (!ctx || slot < 0 || slot >= FBGEMM_B200_USER_SLOTS) {
    set_error("bad context or status slot (callers own slots 0 .. FBGEMM_B200_USER_SLOTS - 1)");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  if (output_size == 0) {
    // No bag to pool: the reference returns `0 == index_size`.
    int rc = check_config(cfg, nullptr);
    if (rc) {
      return rc;
    }
    if (index_size != 0) {
      const int32_t rec[4] = {FBGEMM_B200_STATUS_SIZE_MISMATCH, 0, 0, (int32_t)index_size};
      cudaError_t e = cudaMemcpyAsync(ctx->status + 4 * slot, rec, sizeof(rec), cudaMemcpyHostToDevice,
                                      static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) {
        return fail_cuda(e, "status write");
      }
    }
    return 0;
  }
  if (cfg && !cfg->use_offsets && !cfg->no_bag) {
    // Lengths mode: the scanned offsets live in scratch that belongs to the
    // stream, so that launches on different streams never share it.
    std::lock_guard<std::mutex> lock(ctx->mu);
    return enqueue_lookup(cfg, output_size, index_size, data_size, input, indices, offsets_or_lengths, weights, out,
                          compressed_indices_table, ctx->status + 4 * slot,
                          scan_scratch_of(ctx, static_cast<cudaStream_t>(stream)), static_cast<cudaStream_t>(stream));
  }
  DeviceBuffer unused;  // only lengths mode touches the scratch
  return enqueue_lookup(cfg, output_size, index_size, data_size, input, indices, offsets_or_lengths, weights, out,
                        compressed_indices_table, ctx->status + 4 * slot, unused, static_cast<cudaStream_t>(stream));
}

int fbgemm_b200_spmdm_launch_sharded(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets,
    const float* weights,
    void* const* peer_out,
    int num_peers,
    int64_t bags_per_peer,
    int slot,
    void* stream) {
  if (!ctx || slot < 0 || slot >= FBGEMM_B200_USER_SLOTS) {
    set_error("bad context or status slot (callers own slots 0 .. FBGEMM_B200_USER_SLOTS - 1)");
    return FBGEMM_B200_EINVAL;
  }
  if (!cfg || !cfg->use_offsets || output_size <= 0 || num_peers <= 0) {
    set_error("sharded launch needs offsets, at least one bag and at least one peer");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  DeviceBuffer unused;  // offsets mode: no scratch
  return enqueue_lookup(cfg, output_size, index_size, data_size, input, indices, offsets, weights, nullptr, nullptr,
                        ctx->status + 4 * slot, unused, static_cast<cudaStream_t>(stream), peer_out, num_peers,
                        bags_per_peer);
}

int fbgemm_b200_multi_plan_create(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_table_call* calls,
    int32_t num_tables,
    int32_t num_peers,
    int64_t bags_per_peer,
    int slot,
    fbgemm_b200_multi_plan** out) {
  if (out) {
    *out = nullptr;
  }
  if (!ctx || !out || slot < 0 || slot >= FBGEMM_B200_USER_SLOTS) {
    set_error("bad context, plan pointer or status slot");
    return FBGEMM_B200_EINVAL;
  }
  if (!calls || num_tables <= 0 || num_peers < 0) {
    set_error("a plan needs at least one table");
    return FBGEMM_B200_EINVAL;
  }
  std::vector<SpmdmParams> params((size_t)num_tables);
  std::vector<int> bit_rates((size_t)num_tables);
  for (int t = 0; t < num_tables; ++t) {
    const fbgemm_b200_table_call& c = calls[t];
    if (!c.cfg.use_offsets && !c.cfg.no_bag) {
      set_error("a plan takes offsets, not lengths");
      return FBGEMM_B200_EINVAL;
    }
    if (num_peers > 0 && !c.peer_out) {
      set_error("num_peers > 0 but a table has no peer_out");
      return FBGEMM_B200_EINVAL;
    }
    const int rc = build_lookup_params(&c.cfg, c.output_size, c.index_size, c.data_size, c.input, c.indices, c.weights,
                                       c.out, c.compressed_indices_table, ctx->status + 4 * slot, c.peer_out,
                                       num_peers, bags_per_peer, &params[(size_t)t]);
    if (rc) {
      return rc;
    }
    if (!c.cfg.no_bag && !c.offsets) {
      set_error("a table of the plan has no offsets");
      return FBGEMM_B200_EINVAL;
    }
    params[(size_t)t].offsets = c.cfg.no_bag ? nullptr : c.offsets;
    params[(size_t)t].flags |= c.cfg.offset_bytes == 8 ? kOff64 : 0;
    bit_rates[(size_t)t] = c.cfg.bit_rate;
  }
  DeviceGuard guard(ctx->device);
  auto* plan = new (std::nothrow) fbgemm_b200_multi_plan;
  if (!plan) {
    set_error("out of host memory");
    return FBGEMM_B200_ENOMEM;
  }
  plan->device = ctx->device;
  const cudaError_t e = build_multi_plan(params, bit_rates, &plan->plan);
  if (e != cudaSuccess) {
    delete plan;
    return fail_cuda(e, "multi-table plan");
  }
  *out = plan;
  return 0;
}

int fbgemm_b200_multi_plan_launch(fbgemm_b200_multi_plan* plan, void* stream) {
  if (!plan) {
    set_error("null plan");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(plan->device);
  const cudaError_t e = launch_multi_plan(plan->plan, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    return fail_cuda(e, "multi-table launch");
  }
  return 0;
}

int fbgemm_b200_multi_plan_num_launches(const fbgemm_b200_multi_plan* plan) {
  return plan ? (int)(plan->plan.groups.size() + plan->plan.singles.size()) : 0;
}

void fbgemm_b200_multi_plan_destroy(fbgemm_b200_multi_plan* plan) {
  if (plan) {
    DeviceGuard guard(plan->device);
    delete plan;
  }
}

int fbgemm_b200_status_read(fbgemm_b200_ctx* ctx, int slot, void* stream, int32_t* info) {
  if (!ctx || slot < 0 || slot >= FBGEMM_B200_STATUS_SLOTS) {
    set_error("bad context or status slot");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t* h = ctx->status_host + 4 * slot;
  cudaError_t e = cudaMemcpyAsync(h, ctx->status + 4 * slot, 16, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) {
    e = cudaStreamSynchronize(s);
  }
  if (e != cudaSuccess) {
    return fail_cuda(e, "status read");
  }
  int32_t rec[4] = {h[0], h[1], h[2], h[3]};
  if (info) {
    std::memcpy(info, rec, sizeof(rec));
  }
  if (rec[0] != 0) {
    e = cudaMemsetAsync(ctx->status + 4 * slot, 0, 16, s);
    if (e != cudaSuccess) {
      return fail_cuda(e, "status clear");
    }
  }
  return rec[0] == 0 ? 1 : 0;
}

int fbgemm_b200_spmdm(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets_or_lengths,
    const float* weights,
    void* out,
    const int32_t* compressed_indices_table,
    void* stream) {
  if (!ctx) {
    set_error("null context");
    return FBGEMM_B200_EINVAL;
  }
  // Slot 0 is shared by all synchronous calls of this context.
  static std::mutex sync_mu;
  std::lock_guard<std::mutex> lock(sync_mu);
  int rc = fbgemm_b200_spmdm_launch(ctx, cfg, output_size, index_size, data_size, input, indices,
                                    offsets_or_lengths, weights, out, compressed_indices_table, 0, stream);
  if (rc) {
    return rc;
  }
  return fbgemm_b200_status_read(ctx, 0, stream, nullptr);
}

int fbgemm_b200_compressed_indices_remap(
    fbgemm_b200_ctx* ctx,
    int32_t offsets_len,
    const void* indices,
    int32_t index_bytes,
    int64_t index_size,
    const int32_t* compressed_indices_mapping,
    int64_t mapping_size,
    const void* offsets,
    const float* weights,
    void* out_indices,
    void* out_offsets,
    float* out_weights,
    void* stream) {
  if (!ctx) {
    set_error("null context");
    return FBGEMM_B200_EINVAL;
  }
  if (offsets_len < 1 || (index_bytes != 4 && index_bytes != 8) || index_size < 0 || mapping_size < 0 || !offsets ||
      !out_offsets || (index_size > 0 && (!indices || !out_indices || !compressed_indices_mapping)) ||
      (weights && !out_weights)) {
    set_error("compressed_indices_remap: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  // The scratch and the status slot (one reserved for this call, outside the
  // callers' and the lanes' ranges) are the context's: one remap at a time;
  // the call returns only after its kernels have finished.
  std::lock_guard<std::mutex> lock(ctx->mu);
  cudaError_t e = reserve(ctx->remap_scratch, remap_scratch_bytes(index_size));
  if (e != cudaSuccess) {
    return fail_cuda(e, "scratch for the index remap");
  }
  const int slot = kRemapSlot;
  e = launch_compressed_indices_remap(offsets_len, indices, index_bytes, index_size, compressed_indices_mapping,
                                      mapping_size, offsets, weights, out_indices, out_offsets, out_weights,
                                      ctx->status + 4 * slot, ctx->remap_scratch.ptr, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    return fail_cuda(e, "index remap launch");
  }
  return fbgemm_b200_status_read(ctx, slot, stream, nullptr);
}

int fbgemm_b200_pruned_hashmap_lookup(
    fbgemm_b200_ctx* ctx,
    int32_t T,
    int32_t B,
    const void* indices,
    const void* offsets,
    int32_t index_bytes,
    int64_t index_size,
    const void* hash_table,
    int32_t hash_bytes,
    const int64_t* hash_table_offsets,
    void* dense_indices,
    int32_t slot,
    void* stream) {
  return pruned_lookup(true, ctx, T, B, indices, offsets, index_bytes, index_size, hash_table, hash_bytes,
                       hash_table_offsets, dense_indices, slot, stream);
}

int fbgemm_b200_pruned_array_lookup(
    fbgemm_b200_ctx* ctx,
    int32_t T,
    int32_t B,
    const void* indices,
    const void* offsets,
    int32_t index_bytes,
    int64_t index_size,
    const void* remappings,
    int32_t remap_bytes,
    const int64_t* remappings_offsets,
    void* dense_indices,
    int32_t slot,
    void* stream) {
  return pruned_lookup(false, ctx, T, B, indices, offsets, index_bytes, index_size, remappings, remap_bytes,
                       remappings_offsets, dense_indices, slot, stream);
}

int fbgemm_b200_sequence_lookup(
    fbgemm_b200_ctx* ctx,
    const void* dev_weights,
    const fbgemm_b200_sequence_table* tables,
    int32_t T,
    int32_t B,
    int32_t D,
    const void* indices,
    const void* offsets,
    int32_t index_bytes,
    int64_t index_size,
    void* out,
    int32_t out_dtype,
    int64_t out_row_bytes,
    int32_t scale_bias_last,
    int32_t fp8_exponent_bits,
    int32_t fp8_exponent_bias,
    int32_t slot,
    void* stream) {
  if (!ctx || slot < 0 || slot >= FBGEMM_B200_STATUS_SLOTS) {
    set_error("bad context or status slot");
    return FBGEMM_B200_EINVAL;
  }
  int64_t min_row = 0;
  switch (out_dtype) {
    case FBGEMM_B200_OUT_F32: min_row = 4 * (int64_t)D; break;
    case FBGEMM_B200_OUT_F16:
    case FBGEMM_B200_OUT_BF16: min_row = 2 * (int64_t)D; break;
    case FBGEMM_B200_OUT_U8:
    case FBGEMM_B200_OUT_INT4: min_row = 1; break;
    default: min_row = -1;
  }
  const int64_t elem = out_dtype == FBGEMM_B200_OUT_F32 ? 4 : (out_dtype <= FBGEMM_B200_OUT_BF16 ? 2 : 1);
  if (T < 1 || B < 1 || D < 1 || min_row < 0 || out_row_bytes < min_row || out_row_bytes % elem != 0 ||
      (index_bytes != 4 && index_bytes != 8) || index_size < 0 || !offsets || !tables ||
      (index_size > 0 && (!indices || !out || !dev_weights)) || reinterpret_cast<uintptr_t>(out) % elem != 0 ||
      fp8_exponent_bits < 0 || fp8_exponent_bits > 7 || fp8_exponent_bias < 0 || fp8_exponent_bias > 253) {
    set_error("sequence_lookup: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  const cudaError_t e = launch_sequence_lookup(
      static_cast<const uint8_t*>(dev_weights), tables, T, B, D, indices, offsets, index_bytes, index_size, out,
      out_dtype, out_row_bytes, scale_bias_last != 0, fp8_exponent_bits, fp8_exponent_bias, ctx->status + 4 * slot,
      static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    return fail_cuda(e, "sequence lookup launch");
  }
  return 0;
}

int fbgemm_b200_pruned_hashmap_insert(
    fbgemm_b200_ctx* ctx,
    int32_t T,
    int32_t B,
    const void* indices,
    const void* dense_indices,
    const void* offsets,
    int32_t index_bytes,
    int64_t index_size,
    void* hash_table,
    int32_t hash_bytes,
    const int64_t* hash_table_offsets,
    int32_t slot,
    void* stream) {
  if (!ctx || slot < 0 || slot >= FBGEMM_B200_STATUS_SLOTS) {
    set_error("bad context or status slot");
    return FBGEMM_B200_EINVAL;
  }
  if (T < 1 || B < 1 || (index_bytes != 4 && index_bytes != 8) || (hash_bytes != 4 && hash_bytes != 8) ||
      index_size < 0 || !offsets || !hash_table_offsets || (index_size > 0 && (!indices || !dense_indices)) ||
      reinterpret_cast<uintptr_t>(hash_table) % (2 * (size_t)hash_bytes) != 0) {
    set_error("pruned_hashmap_insert: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  const cudaError_t e = launch_pruned_hashmap_insert(
      T, B, indices, dense_indices, offsets, index_bytes, index_size, hash_table, hash_bytes, hash_table_offsets,
      ctx->status + 4 * slot, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    return fail_cuda(e, "hash-map insert launch");
  }
  return 0;
}

int fbgemm_b200_pruned_hashmap_insert_host(
    int32_t T,
    int32_t B,
    const void* indices,
    const void* dense_indices,
    const void* offsets,
    int32_t index_bytes,
    void* hash_table,
    int32_t hash_bytes,
    const int64_t* hash_table_offsets) {
  if (T < 1 || B < 1 || !offsets || !hash_table_offsets || (index_bytes != 4 && index_bytes != 8) ||
      (hash_bytes != 4 && hash_bytes != 8)) {
    set_error("pruned_hashmap_insert: bad argument");
    return FBGEMM_B200_EINVAL;
  }
  // Empty inputs may come as null pointers (an empty tensor has no storage).
  const int64_t last = (int64_t)T * B;
  const int64_t covered = index_bytes == 8 ? static_cast<const int64_t*>(offsets)[last]
                                           : (int64_t) static_cast<const int32_t*>(offsets)[last];
  if ((covered > 0 && (!indices || !dense_indices)) || (hash_table_offsets[T] > 0 && !hash_table)) {
    set_error("pruned_hashmap_insert: null indices or hash table");
    return FBGEMM_B200_EINVAL;
  }
  bool ok;
  if (index_bytes == 8 && hash_bytes == 8) {
    ok = hashmap_insert(T, B, static_cast<const int64_t*>(indices), static_cast<const int64_t*>(dense_indices),
                        static_cast<const int64_t*>(offsets), static_cast<int64_t*>(hash_table), hash_table_offsets);
  } else if (index_bytes == 8) {
    ok = hashmap_insert(T, B, static_cast<const int64_t*>(indices), static_cast<const int64_t*>(dense_indices),
                        static_cast<const int64_t*>(offsets), static_cast<int32_t*>(hash_table), hash_table_offsets);
  } else if (hash_bytes == 8) {
    ok = hashmap_insert(T, B, static_cast<const int32_t*>(indices), static_cast<const int32_t*>(dense_indices),
                        static_cast<const int32_t*>(offsets), static_cast<int64_t*>(hash_table), hash_table_offsets);
  } else {
    ok = hashmap_insert(T, B, static_cast<const int32_t*>(indices), static_cast<const int32_t*>(dense_indices),
                        static_cast<const int32_t*>(offsets), static_cast<int32_t*>(hash_table), hash_table_offsets);
  }
  return ok ? 1 : 0;
}

/* ---- table registry ----------------------------------------------------- */

int fbgemm_b200_table_register(fbgemm_b200_ctx* ctx, const void* host_ptr, size_t bytes) {
  if (!ctx || !host_ptr) {
    set_error("null context or table");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  DeviceBuffer buf;
  // 16 bytes of slack: no vector access of the last row can leave the buffer.
  cudaError_t e = cudaMalloc(&buf.ptr, bytes + 16);
  if (e != cudaSuccess) {
    return fail_cuda(e, "table allocation");
  }
  buf.bytes = bytes;
  e = cudaMemcpy(buf.ptr, host_ptr, bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(buf.ptr);
    return fail_cuda(e, "table upload");
  }
  ResidentTable entry;
  entry.buf = buf;
  entry.fingerprint = table_fingerprint(host_ptr, bytes);
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->tables.find(host_ptr);
  if (it != ctx->tables.end()) {
    cudaDeviceSynchronize();  // a lookup still in flight may be reading the old copy
    cudaFree(it->second.buf.ptr);
    it->second = entry;
  } else {
    ctx->tables.emplace(host_ptr, entry);
  }
  return 0;
}

int fbgemm_b200_table_unregister(fbgemm_b200_ctx* ctx, const void* host_ptr) {
  if (!ctx) {
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->tables.find(host_ptr);
  if (it == ctx->tables.end()) {
    set_error("table not registered");
    return FBGEMM_B200_EINVAL;
  }
  cudaDeviceSynchronize();
  cudaFree(it->second.buf.ptr);
  ctx->tables.erase(it);
  return 0;
}

const void* fbgemm_b200_table_device_ptr(fbgemm_b200_ctx* ctx, const void* host_ptr) {
  if (!ctx) {
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->tables.find(host_ptr);
  return it == ctx->tables.end() ? nullptr : it->second.buf.ptr;
}

namespace {

// The resident copy of the caller's host array `host` for a call that will
// read its first `need_bytes` bytes (0: the size is not part of the call).
// A copy is keyed by the host address alone, and an address can come back
// from the allocator with another table behind it: the copy is used only if
// it is at least as large as the call needs and the caller's memory still has
// the fingerprint taken at registration.  Otherwise a copy this library made
// on its own is refreshed, and an explicit registration is refused with a
// clear error (the caller registers again).  Returns 0 or a negative code.
int resident_table(fbgemm_b200_ctx* ctx, const void* host, size_t need_bytes, bool may_create, const void** dptr) {
  *dptr = nullptr;
  bool stale = false, found = false, implicit = false;
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = ctx->tables.find(host);
    if (it != ctx->tables.end()) {
      found = true;
      implicit = it->second.implicit;
      stale = need_bytes > it->second.buf.bytes ||
          table_fingerprint(host, it->second.buf.bytes) != it->second.fingerprint;
      if (!stale) {
        *dptr = it->second.buf.ptr;
        return 0;
      }
    }
  }
  if (found && !implicit) {
    set_error("the table registered under this host address no longer matches the caller's memory (the call needs " +
              std::to_string(need_bytes) + " bytes, or the contents changed): register it again");
    return FBGEMM_B200_EINVAL;
  }
  if (!may_create || need_bytes == 0) {
    set_error("table not resident: register it first (its size is not part of the call)");
    return FBGEMM_B200_EINVAL;
  }
  const int rc = fbgemm_b200_table_register(ctx, host, need_bytes);
  if (rc) {
    return rc;
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->tables.find(host);
  it->second.implicit = true;
  *dptr = it->second.buf.ptr;
  return 0;
}

}  // namespace

/* ---- host-pointer pipeline ---------------------------------------------- */

int fbgemm_b200_spmdm_host_submit(
    fbgemm_b200_ctx* ctx,
    int lane_id,
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets_or_lengths,
    const float* weights,
    void* out,
    const int32_t* cit) {
  if (!ctx || lane_id < 0 || lane_id >= FBGEMM_B200_HOST_LANES) {
    set_error("bad context or lane");
    return FBGEMM_B200_EINVAL;
  }
  Derived d;
  int rc = check_config(cfg, &d);
  if (rc) {
    return rc;
  }
  if (output_size < 0 || index_size < 0 || data_size < 0) {
    set_error("negative size");
    return FBGEMM_B200_EINVAL;
  }
  if (cfg->no_bag || cfg->absolute_offsets) {
    set_error("no_bag and absolute_offsets are provided for device pointers only");
    return FBGEMM_B200_EINVAL;
  }
  DeviceGuard guard(ctx->device);
  Lane& L = ctx->lanes[lane_id];
  if (L.busy) {
    set_error("lane has work in flight; call fbgemm_b200_spmdm_host_wait first");
    return FBGEMM_B200_EBUSY;
  }
  cudaError_t e;
  if (!L.stream) {
    e = cudaStreamCreateWithFlags(&L.stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
      return fail_cuda(e, "lane stream");
    }
    e = reserve(L.h_status, 16);
    if (e != cudaSuccess) {
      return fail_cuda(e, "lane status");
    }
  }
  L.trivially_true = L.trivially_false = false;
  L.user_out = out;
  L.out_rows = 0;
  if (output_size == 0) {
    L.trivially_true = index_size == 0;
    L.trivially_false = !L.trivially_true;
    L.busy = true;
    return 0;
  }

  // Tables live on the device; find (or create) the resident copies.  With a
  // pruning map the compressed row count is not part of the signature (the
  // reference has the same gap: FbgemmEmbedding.h:212 "TODO: add
  // compressed_data_size"), so that table has to be registered beforehand.
  if (!input || (index_size > 0 && !indices) || !offsets_or_lengths || !out) {
    set_error("null table, indices, offsets or output pointer");
    return FBGEMM_B200_EINVAL;
  }
  const void* d_table = nullptr;
  rc = resident_table(ctx, input, cit ? 0 : (size_t)(data_size * d.input_stride), !cit, &d_table);
  if (rc) {
    return rc;
  }
  const int32_t* d_cit = nullptr;
  if (cit) {
    const void* v = nullptr;
    rc = resident_table(ctx, cit, (size_t)data_size * sizeof(int32_t), true, &v);
    if (rc) {
      return rc;
    }
    d_cit = static_cast<const int32_t*>(v);
  }

  // Pack indices | offsets | weights into one pinned block, one H2D copy.
  const size_t n_off = (size_t)output_size + (cfg->use_offsets ? 1 : 0);
  const size_t idx_bytes = (size_t)index_size * cfg->index_bytes;
  const size_t off_bytes = n_off * cfg->offset_bytes;
  size_t n_w = 0;
  if (cfg->has_weight) {
    if (!weights && index_size > 0) {
      set_error("has_weight set but weights is null");
      return FBGEMM_B200_EINVAL;
    }
    n_w = (size_t)index_size;
    if (cfg->is_weight_positional) {
      // weights[i] with i the position inside a bag: the array is only as
      // long as the longest bag.
      int64_t longest = 0;
      for (int64_t m = 0; m < output_size; ++m) {
        int64_t len;
        if (cfg->offset_bytes == 8) {
          const int64_t* o = static_cast<const int64_t*>(offsets_or_lengths);
          len = cfg->use_offsets ? o[m + 1] - o[m] : o[m];
        } else {
          const int32_t* o = static_cast<const int32_t*>(offsets_or_lengths);
          len = cfg->use_offsets ? (int64_t)o[m + 1] - o[m] : o[m];
        }
        longest = len > longest ? len : longest;
      }
      n_w = (size_t)(longest < index_size ? longest : index_size);
    }
  }
  auto up16 = [](size_t v) { return (v + 15) & ~size_t(15); };
  const size_t off_at = up16(idx_bytes);
  const size_t w_at = off_at + up16(off_bytes);
  const size_t in_bytes = w_at + up16(n_w * sizeof(float));
  const size_t esize = cfg->out_dtype == FBGEMM_B200_OUT_F32 ? 4 : 2;
  // The device copy of the output is dense in block_size-wide rows only when
  // the user's rows are; otherwise keep the user's pitch.
  const size_t out_pitch = (size_t)d.output_stride * esize;
  const size_t out_bytes = (size_t)output_size * out_pitch;

  if ((e = reserve(L.d_in, in_bytes)) != cudaSuccess || (e = reserve(L.d_out, out_bytes)) != cudaSuccess) {
    return fail_cuda(e, "lane staging buffers");
  }
  uint8_t* di = static_cast<uint8_t*>(L.d_in.ptr);
  // Page-locked caller buffers are read by the GPU where they lie: ONE small
  // kernel streams indices, offsets and weights into the lane's device block
  // with wide coalesced loads (three DMA copies of this size spend more time
  // starting than moving data).  Pageable buffers are first packed into the
  // lane's pinned block so that the copy stays asynchronous.
  auto device_view = [](const void* ptr) -> const void* {
    cudaPointerAttributes a{};
    const bool yes = ptr && cudaPointerGetAttributes(&a, ptr) == cudaSuccess && a.type == cudaMemoryTypeHost;
    cudaGetLastError();
    return yes ? a.devicePointer : nullptr;
  };
  const void* v_idx = idx_bytes ? device_view(indices) : nullptr;
  const void* v_off = device_view(offsets_or_lengths);
  const void* v_w = n_w ? device_view(weights) : nullptr;
  // The kernel's reads slow a concurrent device-to-host DMA down (measured:
  // 88 -> 104 us per step where 4.2 MB of output leave per 2 MB of input), so
  // it is used only where the upload is the larger transfer; otherwise the
  // three pieces go up as DMA copies.
  const bool all_pinned = (!idx_bytes || v_idx) && v_off && (!n_w || v_w);
  const bool upload_dominant = all_pinned && in_bytes > out_bytes;
  if (upload_dominant) {
    const StageSegment seg[3] = {
        {v_idx, di, idx_bytes}, {v_off, di + off_at, off_bytes}, {v_w, di + w_at, n_w * sizeof(float)}};
    e = launch_stage_inputs(seg, L.stream);
  } else if (all_pinned) {
    e = cudaSuccess;
    if (idx_bytes) {
      e = cudaMemcpyAsync(di, indices, idx_bytes, cudaMemcpyHostToDevice, L.stream);
    }
    if (e == cudaSuccess) {
      e = cudaMemcpyAsync(di + off_at, offsets_or_lengths, off_bytes, cudaMemcpyHostToDevice, L.stream);
    }
    if (e == cudaSuccess && n_w) {
      e = cudaMemcpyAsync(di + w_at, weights, n_w * sizeof(float), cudaMemcpyHostToDevice, L.stream);
    }
  } else {
    if ((e = reserve(L.h_in, in_bytes)) != cudaSuccess) {
      return fail_cuda(e, "lane staging buffers");
    }
    uint8_t* h = static_cast<uint8_t*>(L.h_in.ptr);
    if (idx_bytes) {
      std::memcpy(h, indices, idx_bytes);
    }
    std::memcpy(h + off_at, offsets_or_lengths, off_bytes);
    if (n_w) {
      std::memcpy(h + w_at, weights, n_w * sizeof(float));
    }
    e = cudaMemcpyAsync(di, h, in_bytes, cudaMemcpyHostToDevice, L.stream);
  }
  if (e != cudaSuccess) {
    return fail_cuda(e, "input upload");
  }

  // Status of this lane: the last FBGEMM_B200_HOST_LANES slots of the context.
  const int slot = FBGEMM_B200_STATUS_SLOTS - FBGEMM_B200_HOST_LANES + lane_id;
  rc = enqueue_lookup(cfg, output_size, index_size, data_size, d_table, di, di + off_at,
                      cfg->has_weight ? reinterpret_cast<const float*>(di + w_at) : nullptr, L.d_out.ptr, d_cit,
                      ctx->status + 4 * slot, L.d_scan, L.stream);
  if (rc) {
    return rc;
  }
  // Results: into pinned memory when the user's buffer is pageable, so that
  // the copy stays asynchronous; straight into the user's buffer otherwise.
  cudaPointerAttributes attr{};
  const bool user_pinned = cudaPointerGetAttributes(&attr, out) == cudaSuccess && attr.type == cudaMemoryTypeHost;
  cudaGetLastError();  // pageable memory reports an error on older drivers
  void* dst = out;
  if (!user_pinned) {
    if ((e = reserve(L.h_out, out_bytes)) != cudaSuccess) {
      return fail_cuda(e, "lane output staging");
    }
    dst = L.h_out.ptr;
    L.out_rows = output_size;
    L.out_row_bytes = (size_t)cfg->block_size * esize;
    L.out_pitch_bytes = out_pitch;
  }
  const size_t row_bytes = (size_t)cfg->block_size * esize;
  if (row_bytes == out_pitch) {
    e = cudaMemcpyAsync(dst, L.d_out.ptr, out_bytes, cudaMemcpyDeviceToHost, L.stream);
  } else {
    // Only block_size columns of each row are this call's: the caller's rows
    // may hold other tables' columns in between (output_stride).
    e = cudaMemcpy2DAsync(dst, out_pitch, L.d_out.ptr, out_pitch, row_bytes, (size_t)output_size,
                          cudaMemcpyDeviceToHost, L.stream);
  }
  if (e == cudaSuccess) {
    // The status record follows the rows.  As a DMA copy it takes its turn in the copy engine behind the other
    // lanes' rows; where the uploads are the larger transfer that wait is what holds the lane back, and a one-warp
    // kernel writes the record to the page-locked word instead (measured on the 4-bit configuration with 8 lanes:
    // 31.8 -> 27.5 us per call).  Where the rows are the larger transfer the copy stays: with the kernel the 8-bit
    // configuration ran 9 % faster and the pruned 2-bit one 15 % slower.
    e = upload_dominant
            ? launch_status_to_host(ctx->status + 4 * slot, static_cast<int32_t*>(L.h_status.ptr), L.stream)
            : cudaMemcpyAsync(L.h_status.ptr, ctx->status + 4 * slot, 16, cudaMemcpyDeviceToHost, L.stream);
  }
  if (e != cudaSuccess) {
    return fail_cuda(e, "result download");
  }
  L.busy = true;
  return 0;
}

int fbgemm_b200_spmdm_host_wait(fbgemm_b200_ctx* ctx, int lane_id) {
  if (!ctx || lane_id < 0 || lane_id >= FBGEMM_B200_HOST_LANES) {
    set_error("bad context or lane");
    return FBGEMM_B200_EINVAL;
  }
  Lane& L = ctx->lanes[lane_id];
  if (!L.busy) {
    set_error("lane has nothing in flight");
    return FBGEMM_B200_EINVAL;
  }
  L.busy = false;
  if (L.trivially_true) {
    return 1;
  }
  if (L.trivially_false) {
    return 0;
  }
  DeviceGuard guard(ctx->device);
  cudaError_t e = cudaStreamSynchronize(L.stream);
  if (e != cudaSuccess) {
    return fail_cuda(e, "lane synchronize");
  }
  if (L.out_rows) {
    // Only the block_size columns of each row belong to this call: the user's
    // buffer may hold other tables' columns between them (output_stride).
    const uint8_t* src = static_cast<const uint8_t*>(L.h_out.ptr);
    uint8_t* dst = static_cast<uint8_t*>(L.user_out);
    if (L.out_row_bytes == L.out_pitch_bytes) {
      std::memcpy(dst, src, (size_t)L.out_rows * L.out_pitch_bytes);
    } else {
      for (int64_t r = 0; r < L.out_rows; ++r) {
        std::memcpy(dst + r * L.out_pitch_bytes, src + r * L.out_pitch_bytes, L.out_row_bytes);
      }
    }
  }
  const int32_t code = static_cast<const int32_t*>(L.h_status.ptr)[0];
  if (code != 0) {
    const int slot = FBGEMM_B200_STATUS_SLOTS - FBGEMM_B200_HOST_LANES + lane_id;
    cudaMemsetAsync(ctx->status + 4 * slot, 0, 16, L.stream);
  }
  return code == 0 ? 1 : 0;
}

int fbgemm_b200_spmdm_host(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets_or_lengths,
    const float* weights,
    void* out,
    const int32_t* compressed_indices_table) {
  static std::mutex lane0_mu;
  std::lock_guard<std::mutex> lock(lane0_mu);
  int rc = fbgemm_b200_spmdm_host_submit(ctx, 0, cfg, output_size, index_size, data_size, input, indices,
                                         offsets_or_lengths, weights, out, compressed_indices_table);
  if (rc) {
    return rc;
  }
  return fbgemm_b200_spmdm_host_wait(ctx, 0);
}

/* ---- quantizers ---------------------------------------------------------- */

int fbgemm_b200_float_to_fused_8bit_rowwise(
    const float* input,
    int64_t rows,
    int32_t cols,
    uint8_t* output,
    void* stream) {
  if (rows < 0 || cols < 0) {
    set_error("negative shape");
    return FBGEMM_B200_EINVAL;
  }
  if (rows == 0 || cols == 0) {
    return 0;
  }
  cudaError_t e = launch_quantize_8bit(input, rows, cols, output, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : fail_cuda(e, "8-bit quantizer launch");
}

int fbgemm_b200_float_to_fused_nbit_rowwise(
    int32_t bit_rate,
    const float* input,
    int64_t rows,
    int32_t cols,
    uint8_t* output,
    void* stream) {
  if (bit_rate != 2 && bit_rate != 4 && bit_rate != 8) {
    set_error("bit_rate must be 2, 4 or 8");
    return FBGEMM_B200_EINVAL;
  }
  if (rows < 0 || cols < 0 || cols % (8 / bit_rate) != 0) {
    set_error("Unsupported number of columns");
    return FBGEMM_B200_EINVAL;
  }
  if (rows == 0 || cols == 0) {
    return 0;
  }
  cudaError_t e = launch_quantize_nbit(bit_rate, input, rows, cols, output, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : fail_cuda(e, "N-bit quantizer launch");
}

}  // extern "C"

// The C++ kernel-generator API over the C ABI: explicit instantiations of the
// templates declared in include/fbgemm_b200/FbgemmEmbedding.h, for the type
// combinations the reference instantiates for quantized rows
// (src/EmbeddingSpMDM.cc:1680-1703, src/EmbeddingSpMDMNBit.cc:1461-1484).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <type_traits>

#include "fbgemm_b200/FbgemmEmbedding.h"

namespace fbgemm_b200 {

namespace {

thread_local void* t_stream = nullptr;

std::mutex g_ctx_mu;
std::map<int, fbgemm_b200_ctx*> g_ctx;

[[noreturn]] void throw_runtime(const char* what) {
  throw std::runtime_error(std::string(what) + ": " + fbgemm_b200_last_error());
}

int resolve_device(int device) {
  if (device >= 0) {
    return device;
  }
  int cur = 0;
  if (cudaGetDevice(&cur) != cudaSuccess) {
    throw std::runtime_error("fbgemm_b200: no CUDA device (there is no CPU fallback)");
  }
  return cur;
}

// Device pointers (and managed ones) go straight to the kernel; everything
// else is host memory and takes the staging path.
bool on_device(const void* p) {
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

template <typename OutType>
constexpr int out_dtype() {
  static_assert(
      std::is_same<OutType, float>::value || std::is_same<OutType, std::uint16_t>::value ||
          std::is_same<OutType, float16>::value || std::is_same<OutType, std::uint8_t>::value,
      "OutType must be float, uint16_t (fp16 bits), float16 or (no_bag) uint8_t");
  return std::is_same<OutType, float>::value ? FBGEMM_B200_OUT_F32
      : std::is_same<OutType, std::uint8_t>::value ? FBGEMM_B200_OUT_U8
                                                   : FBGEMM_B200_OUT_F16;
}

fbgemm_b200_spmdm_config make_config(
    int bit_rate,
    int index_bytes,
    int offset_bytes,
    int out_dt,
    std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    bool is_weight_positional,
    bool use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride,
    bool scale_bias_last = true,
    bool no_bag = false,
    bool is_bf16_out = false,
    int in = FBGEMM_B200_IN_QUANTIZED,
    int fp8_exponent_bits = 0,
    int fp8_exponent_bias = 0) {
  fbgemm_b200_spmdm_config c{};
  c.bit_rate = bit_rate;
  c.index_bytes = index_bytes;
  c.offset_bytes = offset_bytes;
  // A 16-bit OutType holds bf16 when is_bf16_out is set (convert_from_float_ref,
  // src/RefImplementations.h:443-453); a float OutType ignores the flag.
  c.out_dtype = (is_bf16_out && out_dt == FBGEMM_B200_OUT_F16) ? FBGEMM_B200_OUT_BF16 : out_dt;
  c.scale_bias_first = !scale_bias_last;
  c.no_bag = no_bag;
  c.in_dtype = in;
  c.fp8_exponent_bits = fp8_exponent_bits;
  c.fp8_exponent_bias = fp8_exponent_bias;
  c.block_size = block_size;
  c.output_stride = output_stride;
  c.input_stride = input_stride;
  c.has_weight = has_weight;
  c.normalize_by_lengths = normalize_by_lengths;
  c.is_weight_positional = is_weight_positional;
  c.use_offsets = use_offsets;
  if (fbgemm_b200_spmdm_check_config(&c) != 0) {
    throw std::invalid_argument(std::string("fbgemm_b200: ") + fbgemm_b200_last_error());
  }
  GetContext(-1);  // fail at generation time when there is no sm_100 device
  return c;
}

// One functor call.  Returns the reference's bool; throws on runtime errors
// (CUDA failures), which have no counterpart in the reference.
bool call(
    const fbgemm_b200_spmdm_config& cfg,
    std::int64_t output_size,
    std::int64_t index_size,
    std::int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets_or_lengths,
    const float* weights,
    void* out,
    const std::int32_t* cit) {
  fbgemm_b200_ctx* ctx = GetContext(-1);
  int rc;
  if (on_device(input)) {
    rc = fbgemm_b200_spmdm(
        ctx, &cfg, output_size, index_size, data_size, input, indices, offsets_or_lengths,
        cfg.has_weight ? weights : nullptr, out, cit, t_stream);
  } else {
    rc = fbgemm_b200_spmdm_host(
        ctx, &cfg, output_size, index_size, data_size, input, indices, offsets_or_lengths,
        cfg.has_weight ? weights : nullptr, out, cit);
  }
  if (rc < 0) {
    throw_runtime("fbgemm_b200 lookup failed");
  }
  return rc == 1;
}

}  // namespace

void SetStream(void* stream) {
  t_stream = stream;
}

fbgemm_b200_ctx* GetContext(int device) {
  device = resolve_device(device);
  std::lock_guard<std::mutex> lock(g_ctx_mu);
  auto it = g_ctx.find(device);
  if (it != g_ctx.end()) {
    return it->second;
  }
  fbgemm_b200_ctx* ctx = nullptr;
  if (fbgemm_b200_ctx_create(device, &ctx) != 0) {
    throw_runtime("fbgemm_b200: cannot create a context (there is no CPU fallback)");
  }
  g_ctx[device] = ctx;
  return ctx;
}

void RegisterTable(const void* host_table, std::size_t bytes, int device) {
  if (fbgemm_b200_table_register(GetContext(device), host_table, bytes) != 0) {
    throw_runtime("fbgemm_b200: table registration failed");
  }
}

void InvalidateTable(const void* host_table, int device) {
  fbgemm_b200_table_unregister(GetContext(device), host_table);
}

template <typename IndexType>
void compressed_indices_remap(
    std::int32_t offsets_numel,
    const IndexType* indices,
    const std::int32_t* compressed_indices_mapping,
    const IndexType* offsets,
    const float* weights,
    IndexType* out_indices,
    IndexType* out_offsets,
    float* out_weights) {
  if (offsets_numel < 1) {
    return;
  }
  fbgemm_b200_ctx* ctx = GetContext(-1);
  auto check = [](cudaError_t e) {
    if (e != cudaSuccess) {
      throw std::runtime_error(std::string("fbgemm_b200 compressed_indices_remap: ") + cudaGetErrorString(e));
    }
  };
  if (on_device(offsets)) {
    // entries in `indices`: the last offset (one small read-back)
    IndexType last = 0;
    check(cudaMemcpyAsync(&last, offsets + offsets_numel - 1, sizeof(IndexType), cudaMemcpyDeviceToHost,
                          static_cast<cudaStream_t>(t_stream)));
    check(cudaStreamSynchronize(static_cast<cudaStream_t>(t_stream)));
    const int rc = fbgemm_b200_compressed_indices_remap(
        ctx, offsets_numel, indices, (std::int32_t)sizeof(IndexType), (std::int64_t)last, compressed_indices_mapping,
        INT64_MAX, offsets, weights, out_indices, out_offsets, out_weights, t_stream);
    if (rc < 0) {
      throw_runtime("fbgemm_b200 compressed_indices_remap failed");
    }
    return;
  }
  // Host arrays: stage everything, remap on the device, bring the results back.
  const std::int64_t first = (std::int64_t)offsets[0];
  const std::int64_t n = (std::int64_t)offsets[offsets_numel - 1];
  std::int64_t max_index = -1;
  for (std::int64_t k = first < 0 ? 0 : first; k < n; ++k) {
    max_index = std::max<std::int64_t>(max_index, (std::int64_t)indices[k]);
  }
  const std::int64_t map_size = max_index + 1;
  const std::size_t idx_bytes = (std::size_t)(n > 0 ? n : 0) * sizeof(IndexType);
  const std::size_t off_bytes = (std::size_t)offsets_numel * sizeof(IndexType);
  const std::size_t w_bytes = weights ? (std::size_t)(n > 0 ? n : 0) * sizeof(float) : 0;
  const std::size_t map_bytes = (std::size_t)map_size * sizeof(std::int32_t);
  auto up = [](std::size_t v) { return (v + 255) & ~std::size_t(255); };
  const std::size_t total = 2 * up(idx_bytes) + 2 * up(off_bytes) + 2 * up(w_bytes) + up(map_bytes) + 256;
  char* d = nullptr;
  check(cudaMalloc(&d, total));
  char* d_idx = d;
  char* d_off = d_idx + up(idx_bytes);
  char* d_w = d_off + up(off_bytes);
  char* d_map = d_w + up(w_bytes);
  char* d_oidx = d_map + up(map_bytes);
  char* d_ooff = d_oidx + up(idx_bytes);
  char* d_ow = d_ooff + up(off_bytes);
  int rc = 0;
  try {
    if (idx_bytes) {
      check(cudaMemcpy(d_idx, indices, idx_bytes, cudaMemcpyHostToDevice));
    }
    check(cudaMemcpy(d_off, offsets, off_bytes, cudaMemcpyHostToDevice));
    if (w_bytes) {
      check(cudaMemcpy(d_w, weights, w_bytes, cudaMemcpyHostToDevice));
    }
    if (map_bytes) {
      check(cudaMemcpy(d_map, compressed_indices_mapping, map_bytes, cudaMemcpyHostToDevice));
    }
    rc = fbgemm_b200_compressed_indices_remap(
        ctx, offsets_numel, d_idx, (std::int32_t)sizeof(IndexType), n > 0 ? n : 0,
        reinterpret_cast<const std::int32_t*>(d_map), map_size, d_off, weights ? reinterpret_cast<const float*>(d_w) : nullptr,
        d_oidx, d_ooff, weights ? reinterpret_cast<float*>(d_ow) : nullptr, nullptr);
    if (rc >= 0) {
      check(cudaMemcpy(out_offsets, d_ooff, off_bytes, cudaMemcpyDeviceToHost));
      const std::int64_t kept = (std::int64_t)out_offsets[offsets_numel - 1];
      if (kept > 0) {
        check(cudaMemcpy(out_indices, d_oidx, (std::size_t)kept * sizeof(IndexType), cudaMemcpyDeviceToHost));
        if (weights) {
          check(cudaMemcpy(out_weights, d_ow, (std::size_t)kept * sizeof(float), cudaMemcpyDeviceToHost));
        }
      }
    }
  } catch (...) {
    cudaFree(d);
    throw;
  }
  cudaFree(d);
  if (rc < 0) {
    throw_runtime("fbgemm_b200 compressed_indices_remap failed");
  }
}

template FBGEMM_B200_API void compressed_indices_remap<std::int32_t>(
    std::int32_t, const std::int32_t*, const std::int32_t*, const std::int32_t*, const float*, std::int32_t*,
    std::int32_t*, float*);
template FBGEMM_B200_API void compressed_indices_remap<std::int64_t>(
    std::int32_t, const std::int64_t*, const std::int32_t*, const std::int64_t*, const float*, std::int64_t*,
    std::int64_t*, float*);

// InType of the 8-bit generator: the fused quantized row (uint8_t) or a table
// that is not quantized (float, float16, or 16-bit storage that is_bf16_in
// makes bf16 - convert_to_float_ref, src/RefImplementations.h:428-440).
template <typename InType>
int in_dtype(bool is_bf16_in) {
  static_assert(
      std::is_same<InType, std::uint8_t>::value || std::is_same<InType, float>::value ||
          std::is_same<InType, float16>::value || std::is_same<InType, std::uint16_t>::value,
      "InType must be uint8_t, float, float16 or uint16_t");
  if (std::is_same<InType, std::uint8_t>::value) {
    if (is_bf16_in) {
      throw std::invalid_argument("fbgemm_b200: is_bf16_in belongs to 16-bit tables");
    }
    return FBGEMM_B200_IN_QUANTIZED;
  }
  if (std::is_same<InType, float>::value) {
    return FBGEMM_B200_IN_F32;
  }
  return (std::is_same<InType, std::uint16_t>::value && is_bf16_in) ? FBGEMM_B200_IN_BF16 : FBGEMM_B200_IN_F16;
}

template <typename InType, typename IndexType, typename OffsetType, typename OutType, bool THREAD_LOCAL>
typename EmbeddingSpMDMKernelSignature<InType, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDMWithStrides(
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int /*prefetch*/,
    bool is_weight_positional,
    bool use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride,
    bool scale_bias_last,
    bool no_bag,
    bool is_bf16_out,
    bool is_bf16_in) {
  const int in = in_dtype<InType>(is_bf16_in);
  // the reference counts input_stride in elements of InType, the C ABI in bytes
  const std::int64_t stride_bytes = input_stride == -1 ? -1 : input_stride * (std::int64_t)sizeof(InType);
  const fbgemm_b200_spmdm_config cfg = make_config(
      8, sizeof(IndexType), sizeof(OffsetType), out_dtype<OutType>(), block_size, has_weight,
      normalize_by_lengths, is_weight_positional, use_offsets, output_stride, stride_bytes, scale_bias_last, no_bag,
      is_bf16_out, in);
  return [cfg](
             std::int64_t output_size,
             std::int64_t index_size,
             std::int64_t data_size,
             const InType* input,
             const IndexType* indices,
             const OffsetType* offsets_or_lengths,
             const float* weights,
             OutType* out) {
    return call(cfg, output_size, index_size, data_size, input, indices, offsets_or_lengths, weights, out, nullptr);
  };
}

template <typename IndexType, typename OffsetType, typename OutType>
typename EmbeddingSpMDMKernelSignature<std::uint8_t, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDMFP8WithStrides(
    const std::int64_t block_size,
    bool normalize_by_lengths,
    bool is_weight_positional,
    bool use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride,
    int exponent_bits,
    int exponent_bias,
    bool is_bf16_out) {
  fbgemm_b200_spmdm_config plain = make_config(
      8, sizeof(IndexType), sizeof(OffsetType), out_dtype<OutType>(), block_size, false, normalize_by_lengths,
      is_weight_positional, use_offsets, output_stride, input_stride, true, false, is_bf16_out, FBGEMM_B200_IN_FP8,
      exponent_bits, exponent_bias);
  fbgemm_b200_spmdm_config weighted = plain;
  weighted.has_weight = 1;
  return [plain, weighted](
             std::int64_t output_size,
             std::int64_t index_size,
             std::int64_t data_size,
             const std::uint8_t* input,
             const IndexType* indices,
             const OffsetType* offsets_or_lengths,
             const float* weights,
             OutType* out) {
    return call(weights ? weighted : plain, output_size, index_size, data_size, input, indices, offsets_or_lengths,
                weights, out, nullptr);
  };
}

template <typename InType, typename IndexType, typename OffsetType, typename OutType, bool THREAD_LOCAL>
typename EmbeddingSpMDMKernelSignature<InType, IndexType, OffsetType, OutType>::Type GenerateEmbeddingSpMDM(
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int prefetch,
    bool is_weight_positional,
    bool use_offsets,
    bool is_bf16_out,
    bool is_bf16_in) {
  return GenerateEmbeddingSpMDMWithStrides<InType, IndexType, OffsetType, OutType, THREAD_LOCAL>(
      block_size, has_weight, normalize_by_lengths, prefetch, is_weight_positional, use_offsets, -1, -1, true,
      false, is_bf16_out, is_bf16_in);
}

template <typename IndexType, typename OffsetType, typename OutType, bool THREAD_LOCAL>
typename EmbeddingSpMDMKernelSignature<std::uint8_t, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDMNBitWithStrides(
    const int input_bit_rate,
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int /*prefetch*/,
    bool is_weight_positional,
    bool use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride,
    bool scale_bias_last,
    const bool is_bf16_out,
    const bool no_bag,
    int output_bit_rate) {
  if (input_bit_rate != 2 && input_bit_rate != 4) {
    throw std::invalid_argument("fbgemm_b200: bit_rate must be 2 or 4");
  }
  if (no_bag) {
    // the reference's N-bit no_bag is the int4 -> int4 sequence lookup, a byte copy of the rows
    // (src/RefImplementations.cc:1467-1485)
    if (input_bit_rate != 4 || output_bit_rate != 4 || !std::is_same<OutType, std::uint8_t>::value) {
      throw std::invalid_argument("fbgemm_b200: no_bag is only supported for int4 to int4");
    }
  } else if (
      std::is_same<OutType, std::uint8_t>::value ||
      (output_bit_rate != -1 && output_bit_rate != (int)(8 * sizeof(OutType)))) {
    throw std::invalid_argument("fbgemm_b200: N-bit output is provided for no_bag only");
  }
  const fbgemm_b200_spmdm_config cfg = make_config(
      input_bit_rate, sizeof(IndexType), sizeof(OffsetType), out_dtype<OutType>(), block_size, has_weight,
      normalize_by_lengths, is_weight_positional, use_offsets, output_stride, input_stride, scale_bias_last, no_bag,
      is_bf16_out);
  return [cfg](
             std::int64_t output_size,
             std::int64_t index_size,
             std::int64_t data_size,
             const std::uint8_t* input,
             const IndexType* indices,
             const OffsetType* offsets_or_lengths,
             const float* weights,
             OutType* out) {
    return call(cfg, output_size, index_size, data_size, input, indices, offsets_or_lengths, weights, out, nullptr);
  };
}

template <typename IndexType, typename OffsetType, typename OutType>
typename EmbeddingSpMDMKernelSignature<std::uint8_t, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDMNBit(
    int bit_rate,
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int prefetch,
    bool is_weight_positional,
    bool use_offsets) {
  return GenerateEmbeddingSpMDMNBitWithStrides<IndexType, OffsetType, OutType, false>(
      bit_rate, block_size, has_weight, normalize_by_lengths, prefetch, is_weight_positional, use_offsets, -1, -1,
      true, false, false, -1);
}

template <typename InType, typename IndexType, typename OffsetType>
typename EmbeddingSpMDMRowWiseSparseKernelSignature<InType, IndexType, OffsetType>::Type
GenerateEmbeddingSpMDMRowWiseSparse(
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int /*prefetch*/,
    bool is_weight_positional,
    bool use_offsets) {
  // InType uint8_t: fused 8-bit rows; float, float16 and uint16_t (read as fp16 here, as in
  // EmbeddingSpMDMRowWiseSparse_ref, src/RefImplementations.cc:1720-1728): rows of block_size elements.
  const fbgemm_b200_spmdm_config cfg = make_config(
      8, sizeof(IndexType), sizeof(OffsetType), FBGEMM_B200_OUT_F32, block_size, has_weight, normalize_by_lengths,
      is_weight_positional, use_offsets, -1, -1, true, false, false, in_dtype<InType>(false));
  return [cfg](
             std::int64_t output_size,
             std::int64_t index_size,
             std::int64_t uncompressed_data_size,
             const InType* input,
             const IndexType* indices,
             const OffsetType* offsets_or_lengths,
             const float* weights,
             float* out,
             const std::int32_t* compressed_indices_table) {
    if (!compressed_indices_table) {
      throw std::invalid_argument("fbgemm_b200: compressed_indices_table is null");
    }
    return call(
        cfg, output_size, index_size, uncompressed_data_size, input, indices, offsets_or_lengths, weights, out,
        compressed_indices_table);
  };
}

template <typename IndexType, typename OffsetType>
typename EmbeddingSpMDMRowWiseSparseKernelSignature<std::uint8_t, IndexType, OffsetType>::Type
GenerateEmbeddingSpMDMNBitRowWiseSparse(
    int bit_rate,
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int /*prefetch*/,
    bool is_weight_positional,
    bool use_offsets) {
  if (bit_rate != 2 && bit_rate != 4) {
    throw std::invalid_argument("fbgemm_b200: bit_rate must be 2 or 4");
  }
  const fbgemm_b200_spmdm_config cfg = make_config(
      bit_rate, sizeof(IndexType), sizeof(OffsetType), FBGEMM_B200_OUT_F32, block_size, has_weight,
      normalize_by_lengths, is_weight_positional, use_offsets, -1, -1);
  return [cfg](
             std::int64_t output_size,
             std::int64_t index_size,
             std::int64_t uncompressed_data_size,
             const std::uint8_t* input,
             const IndexType* indices,
             const OffsetType* offsets_or_lengths,
             const float* weights,
             float* out,
             const std::int32_t* compressed_indices_table) {
    if (!compressed_indices_table) {
      throw std::invalid_argument("fbgemm_b200: compressed_indices_table is null");
    }
    return call(
        cfg, output_size, index_size, uncompressed_data_size, input, indices, offsets_or_lengths, weights, out,
        compressed_indices_table);
  };
}

// ---- explicit instantiations -------------------------------------------------

#define INST_IN(IN, IDX, OFF, OUT, TL)                                                               \
  template FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<IN, IDX, OFF, OUT>::Type           \
  GenerateEmbeddingSpMDM<IN, IDX, OFF, OUT, TL>(                                                     \
      const std::int64_t, bool, bool, int, bool, bool, bool, bool);                                  \
  template FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<IN, IDX, OFF, OUT>::Type           \
  GenerateEmbeddingSpMDMWithStrides<IN, IDX, OFF, OUT, TL>(                                          \
      const std::int64_t, bool, bool, int, bool, bool, std::int64_t, std::int64_t, bool, bool, bool, bool);

#define INST_8BIT(IDX, OFF, OUT, TL)        \
  INST_IN(std::uint8_t, IDX, OFF, OUT, TL)  \
  INST_IN(float, IDX, OFF, OUT, TL)         \
  INST_IN(float16, IDX, OFF, OUT, TL)       \
  INST_IN(std::uint16_t, IDX, OFF, OUT, TL)

#define INST_FP8(IDX, OFF, OUT)                                                                      \
  template FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<std::uint8_t, IDX, OFF, OUT>::Type \
  GenerateEmbeddingSpMDMFP8WithStrides<IDX, OFF, OUT>(                                               \
      const std::int64_t, bool, bool, bool, std::int64_t, std::int64_t, int, int, bool);

#define INST_NBIT(IDX, OFF, OUT)                                                                               \
  template FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<std::uint8_t, IDX, OFF, OUT>::Type           \
  GenerateEmbeddingSpMDMNBit<IDX, OFF, OUT>(int, const std::int64_t, bool, bool, int, bool, bool);             \
  template FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<std::uint8_t, IDX, OFF, OUT>::Type           \
  GenerateEmbeddingSpMDMNBitWithStrides<IDX, OFF, OUT, false>(                                                 \
      const int, const std::int64_t, bool, bool, int, bool, bool, std::int64_t, std::int64_t, bool, const bool, \
      const bool, int);                                                                                        \
  template FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<std::uint8_t, IDX, OFF, OUT>::Type           \
  GenerateEmbeddingSpMDMNBitWithStrides<IDX, OFF, OUT, true>(                                                  \
      const int, const std::int64_t, bool, bool, int, bool, bool, std::int64_t, std::int64_t, bool, const bool, \
      const bool, int);

#define INST_SPARSE_IN(IN, IDX, OFF)                                                                 \
  template FBGEMM_B200_API typename EmbeddingSpMDMRowWiseSparseKernelSignature<IN, IDX, OFF>::Type   \
  GenerateEmbeddingSpMDMRowWiseSparse<IN, IDX, OFF>(const std::int64_t, bool, bool, int, bool, bool);

#define INST_SPARSE(IDX, OFF)                                                                                  \
  INST_SPARSE_IN(std::uint8_t, IDX, OFF)                                                                       \
  INST_SPARSE_IN(float, IDX, OFF)                                                                              \
  INST_SPARSE_IN(float16, IDX, OFF)                                                                            \
  INST_SPARSE_IN(std::uint16_t, IDX, OFF)                                                                      \
  template FBGEMM_B200_API typename EmbeddingSpMDMRowWiseSparseKernelSignature<std::uint8_t, IDX, OFF>::Type   \
  GenerateEmbeddingSpMDMNBitRowWiseSparse<IDX, OFF>(int, const std::int64_t, bool, bool, int, bool, bool);

#define INST_OUT(IDX, OFF)                 \
  INST_8BIT(IDX, OFF, float, false)        \
  INST_8BIT(IDX, OFF, float, true)         \
  INST_8BIT(IDX, OFF, std::uint16_t, false) \
  INST_8BIT(IDX, OFF, std::uint16_t, true) \
  INST_8BIT(IDX, OFF, float16, false)      \
  INST_8BIT(IDX, OFF, float16, true)       \
  INST_NBIT(IDX, OFF, float)               \
  INST_NBIT(IDX, OFF, std::uint16_t)       \
  INST_NBIT(IDX, OFF, float16)             \
  INST_NBIT(IDX, OFF, std::uint8_t)        \
  INST_IN(std::uint8_t, IDX, OFF, std::uint8_t, false) \
  INST_IN(std::uint8_t, IDX, OFF, std::uint8_t, true)  \
  INST_FP8(IDX, OFF, float)                \
  INST_FP8(IDX, OFF, std::uint16_t)        \
  INST_FP8(IDX, OFF, float16)              \
  INST_SPARSE(IDX, OFF)

INST_OUT(std::int32_t, std::int32_t)
INST_OUT(std::int32_t, std::int64_t)
INST_OUT(std::int64_t, std::int32_t)
INST_OUT(std::int64_t, std::int64_t)

}  // namespace fbgemm_b200

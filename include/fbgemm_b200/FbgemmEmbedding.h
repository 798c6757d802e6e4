/*
 * fbgemm_b200 - C++ kernel-generator API of the quantized embedding-bag path.
 *
 * The templates below have the names, template parameters, arguments and
 * defaults of FBGEMM's include/fbgemm/FbgemmEmbedding.h (lines cited at each
 * declaration) and return a std::function of the same signature, so a caller
 * of fbgemm::GenerateEmbeddingSpMDM / ...NBit / ...RowWiseSparse can switch by
 * changing the namespace (or by defining FBGEMM_B200_AS_FBGEMM before
 * including this header, which makes the names visible as fbgemm::).
 *
 * What runs underneath is not x86 code generated at run time but hand-written
 * sm_100a CUDA kernels behind the C ABI in embedding_c_api.h:
 *
 *   - If `input` is a device (or managed) pointer, every pointer of the call is
 *     taken to be a device pointer; the kernel is enqueued on the stream set
 *     with SetStream() and the functor returns after reading the kernel's
 *     status word (one 16-byte device-to-host copy).
 *   - If `input` is a host pointer the table is made resident in HBM on first
 *     use (keyed by its address; call InvalidateTable() after rewriting it)
 *     and the per-call arrays travel through pinned staging buffers.
 *
 * Differences from the reference, all reported at generation time by
 * std::invalid_argument: N-bit no_bag (an int4 -> int4 row copy), 8-bit output
 * and the row-wise sparse form of unquantized tables are not provided;
 * block_size of quantized rows is limited to 1024; host pointers do not take
 * no_bag.  InType uint8_t (fused 8-bit rows), float, float16 and uint16_t
 * (fp16 or, with is_bf16_in, bf16 storage) are instantiated.  `prefetch` and
 * THREAD_LOCAL are accepted and ignored.  There is no CPU fallback: without an
 * sm_100 device the generators throw std::runtime_error.
 */
#pragma once

#include <cstdint>
#include <functional>

#include "fbgemm_b200/embedding_c_api.h"

namespace fbgemm_b200 {

/* Same layout as fbgemm::float16 (include/fbgemm/Types.h:16-19). */
struct float16 {
  std::uint16_t val;
};

/* include/fbgemm/FbgemmEmbedding.h:17-50 */
template <
    typename InType,
    typename IndexType,
    typename OffsetType = std::int32_t,
    typename OutType = float>
class EmbeddingSpMDMKernelSignature {
 public:
  using Type = std::function<bool(
      std::int64_t output_size,
      std::int64_t index_size,
      std::int64_t data_size,
      const InType* input,
      const IndexType* indices,
      const OffsetType* offsets_or_lengths,
      const float* weights,  // optional, can be null for non-weighted sum
      OutType* out)>;
};

/* include/fbgemm/FbgemmEmbedding.h:65-84 */
template <
    typename InType,
    typename IndexType,
    typename OffsetType = std::int32_t,
    typename OutType = float,
    bool THREAD_LOCAL = false>
FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<InType, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDM(
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int prefetch = 16,
    bool is_weight_positional = false,
    bool use_offsets = true,
    bool is_bf16_out = false,
    bool is_bf16_in = false);

/* include/fbgemm/FbgemmEmbedding.h:94-117 */
template <
    typename InType,
    typename IndexType,
    typename OffsetType = std::int32_t,
    typename OutType = float,
    bool THREAD_LOCAL = false>
FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<InType, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDMWithStrides(
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int prefetch = 16,
    bool is_weight_positional = false,
    bool use_offsets = true,
    std::int64_t output_stride = -1,
    std::int64_t input_stride = -1,
    bool scale_bias_last = true,
    bool no_bag = false,
    bool is_bf16_out = false,
    bool is_bf16_in = false);

/* include/fbgemm/FbgemmEmbedding.h:124-140 */
template <typename IndexType, typename OffsetType = std::int32_t, typename OutType = float>
FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<std::uint8_t, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDMNBit(
    int bit_rate,
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int prefetch = 16,
    bool is_weight_positional = false,
    bool use_offsets = true);

/* include/fbgemm/FbgemmEmbedding.h:149-174 */
template <
    typename IndexType,
    typename OffsetType = std::int32_t,
    typename OutType = float,
    bool THREAD_LOCAL = false>
FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<std::uint8_t, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDMNBitWithStrides(
    const int input_bit_rate,
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int prefetch = 16,
    bool is_weight_positional = false,
    bool use_offsets = true,
    std::int64_t output_stride = -1,
    std::int64_t input_stride = -1,
    bool scale_bias_last = true,
    const bool is_bf16_out = false,
    const bool no_bag = false,
    int output_bit_rate = -1);

/* include/fbgemm/FbgemmEmbedding.h:185-203: rows of FP8 values, no scale or
 * bias; the functor pools with weights whenever its `weights` is not null. */
template <typename IndexType, typename OffsetType = std::int32_t, typename OutType = float>
FBGEMM_B200_API typename EmbeddingSpMDMKernelSignature<std::uint8_t, IndexType, OffsetType, OutType>::Type
GenerateEmbeddingSpMDMFP8WithStrides(
    const std::int64_t block_size,
    bool normalize_by_lengths,
    bool is_weight_positional = false,
    bool use_offsets = true,
    std::int64_t output_stride = -1,
    std::int64_t input_stride = -1,
    int exponent_bits = 4,
    int exponent_bias = 7,
    bool is_bf16_out = false);

/* include/fbgemm/FbgemmEmbedding.h:205-222 */
template <typename InType, typename IndexType, typename OffsetType = std::int32_t>
class EmbeddingSpMDMRowWiseSparseKernelSignature {
 public:
  using Type = std::function<bool(
      std::int64_t output_size,
      std::int64_t index_size,
      std::int64_t uncompressed_data_size,
      const InType* input,
      const IndexType* indices,
      const OffsetType* offsets_or_lengths,
      const float* weights,  // optional, can be null for non-weighted sum
      float* out,
      const std::int32_t* compressed_indices_table)>;
};

/* include/fbgemm/FbgemmEmbedding.h:229-243 */
template <typename InType, typename IndexType, typename OffsetType = std::int32_t>
FBGEMM_B200_API typename EmbeddingSpMDMRowWiseSparseKernelSignature<InType, IndexType, OffsetType>::Type
GenerateEmbeddingSpMDMRowWiseSparse(
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int prefetch = 16,
    bool is_weight_positional = false,
    bool use_offsets = true);

/* include/fbgemm/FbgemmEmbedding.h:250-262 */
template <typename IndexType, typename OffsetType = std::int32_t>
FBGEMM_B200_API typename EmbeddingSpMDMRowWiseSparseKernelSignature<std::uint8_t, IndexType, OffsetType>::Type
GenerateEmbeddingSpMDMNBitRowWiseSparse(
    int bit_rate,
    const std::int64_t block_size,
    bool has_weight,
    bool normalize_by_lengths,
    int prefetch = 16,
    bool is_weight_positional = false,
    bool use_offsets = true);

/* include/fbgemm/FbgemmEmbedding.h:392-401 (src/EmbeddingSpMDM.cc:1714-1770,
 * scalar form src/RefImplementations.cc:2308-2333): rewrite (indices, offsets,
 * weights) so that rows the map prunes (-1) disappear and the rest address
 * the compressed table.  The arrays are all host pointers or all device
 * pointers.  With host pointers the map is read up to the largest index that
 * occurs; with device pointers the entries of the map are trusted to cover
 * every index, as in the reference (the C ABI form takes the map's size and
 * checks).  Throws std::runtime_error on a CUDA failure. */
template <typename IndexType>
FBGEMM_B200_API void compressed_indices_remap(
    std::int32_t offsets_numel,
    const IndexType* indices,
    const std::int32_t* compressed_indices_mapping,
    const IndexType* offsets,
    const float* weights,  // optional, can be null
    IndexType* out_indices,
    IndexType* out_offsets,
    float* out_weights);

/* ---- not in the reference: what a GPU back end additionally needs -------- */

/* Stream (cudaStream_t as void*) that functors called from this thread with
 * device pointers enqueue on.  Default: the legacy default stream. */
FBGEMM_B200_API void SetStream(void* stream);

/* The C-ABI context the functors use on `device` (-1: the current device);
 * created on first use.  Throws std::runtime_error if there is none. */
FBGEMM_B200_API fbgemm_b200_ctx* GetContext(int device = -1);

/* Make a host table resident before the first lookup (optional; the functor
 * does it on first use for dense tables).  Required for the compressed table
 * of a pruned lookup, whose row count is not part of the functor signature. */
FBGEMM_B200_API void RegisterTable(const void* host_table, std::size_t bytes, int device = -1);

/* Forget the resident copy of a host table (after the host rewrote it). */
FBGEMM_B200_API void InvalidateTable(const void* host_table, int device = -1);

}  // namespace fbgemm_b200

#ifdef FBGEMM_B200_AS_FBGEMM
namespace fbgemm {
using namespace fbgemm_b200;
}
#endif

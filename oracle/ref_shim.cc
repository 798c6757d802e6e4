/*
 * TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.
 *
 * extern "C" entry points around the reference's OWN scalar and
 * auto-vectorised CPU implementations of the quantized embedding-bag path.
 * This file is compiled together with source files taken where they lie in
 * the FBGEMM tree (src/RefImplementations.cc, src/EmbeddingSpMDMAutovec.cc,
 * src/QuantUtils*.cc, ...; see the Makefile beside this file) into
 * _ref/libfbgemm_ref.so.  Nothing of the reference is copied into this
 * repository; only its public declarations are included at build time.
 *
 * Tests use this library to validate the C restatement in embedding_oracle.c
 * and to generate the committed golden fixtures; the benchmark may time it as
 * the CPU baseline.  The product never loads it.
 *
 * The argument conventions are those of embedding_oracle.c: element widths of
 * indices/offsets are passed in bytes, booleans as int, result 1 = true.
 */
#include <cstdint>
#include <functional>
#include <type_traits>
#include <vector>

#include "fbgemm/FbgemmEmbedding.h"
#include "fbgemm/QuantUtils.h"
#include "src/EmbeddingSpMDMAutovec.h"
#include "src/RefImplementations.h"

using fbgemm::float16;

namespace {

template <typename F>
int dispatch_idx_off(int index_bytes, int offset_bytes, F&& f) {
  if (index_bytes == 8 && offset_bytes == 8) {
    return f(std::int64_t{}, std::int64_t{});
  } else if (index_bytes == 8 && offset_bytes == 4) {
    return f(std::int64_t{}, std::int32_t{});
  } else if (index_bytes == 4 && offset_bytes == 8) {
    return f(std::int32_t{}, std::int64_t{});
  } else if (index_bytes == 4 && offset_bytes == 4) {
    return f(std::int32_t{}, std::int32_t{});
  }
  return -1;
}

} // namespace

extern "C" {

// fbgemm::EmbeddingSpMDM_ref<uint8_t, ...> (src/RefImplementations.cc:1196).
int ref_embedding_spmdm_8bit(
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t index_size,
    std::int64_t data_size,
    const std::uint8_t* input,
    const void* indices,
    int index_bytes,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    void* out,
    int out_is_half,
    int is_weight_positional,
    int use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride) {
  return dispatch_idx_off(index_bytes, offset_bytes, [&](auto i, auto o) {
    using I = decltype(i);
    using O = decltype(o);
    if (out_is_half) {
      return (int)fbgemm::EmbeddingSpMDM_ref<std::uint8_t, I, O, float16>(
          block_size, output_size, index_size, data_size, input,
          static_cast<const I*>(indices),
          static_cast<const O*>(offsets_or_lengths), weights,
          normalize_by_lengths != 0, static_cast<float16*>(out),
          is_weight_positional != 0, use_offsets != 0, output_stride,
          input_stride);
    }
    return (int)fbgemm::EmbeddingSpMDM_ref<std::uint8_t, I, O, float>(
        block_size, output_size, index_size, data_size, input,
        static_cast<const I*>(indices),
        static_cast<const O*>(offsets_or_lengths), weights,
        normalize_by_lengths != 0, static_cast<float*>(out),
        is_weight_positional != 0, use_offsets != 0, output_stride,
        input_stride);
  });
}

// fbgemm::EmbeddingSpMDMNBit_ref (src/RefImplementations.cc:1427).
int ref_embedding_spmdm_nbit(
    int bit_rate,
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t index_size,
    std::int64_t data_size,
    const std::uint8_t* input,
    const void* indices,
    int index_bytes,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    void* out,
    int out_is_half,
    int is_weight_positional,
    int use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride) {
  return dispatch_idx_off(index_bytes, offset_bytes, [&](auto i, auto o) {
    using I = decltype(i);
    using O = decltype(o);
    if (out_is_half) {
      return (int)fbgemm::EmbeddingSpMDMNBit_ref<I, O, float16>(
          bit_rate, block_size, output_size, index_size, data_size, input,
          static_cast<const I*>(indices),
          static_cast<const O*>(offsets_or_lengths), weights,
          normalize_by_lengths != 0, static_cast<float16*>(out),
          is_weight_positional != 0, use_offsets != 0, output_stride,
          input_stride);
    }
    return (int)fbgemm::EmbeddingSpMDMNBit_ref<I, O, float>(
        bit_rate, block_size, output_size, index_size, data_size, input,
        static_cast<const I*>(indices),
        static_cast<const O*>(offsets_or_lengths), weights,
        normalize_by_lengths != 0, static_cast<float*>(out),
        is_weight_positional != 0, use_offsets != 0, output_stride,
        input_stride);
  });
}

// The same two reference functions with their remaining arguments exposed:
// scale_bias_last, no_bag (8-bit only) and is_bf16_out.  out_kind: 0 = float,
// 1 = fp16, 2 = bf16 (OutType uint16_t in both 16-bit cases).
int ref_embedding_spmdm_ex(
    int bit_rate,
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t index_size,
    std::int64_t data_size,
    const std::uint8_t* input,
    const void* indices,
    int index_bytes,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    void* out,
    int out_kind,
    int is_weight_positional,
    int use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride,
    int scale_bias_last,
    int no_bag) {
  return dispatch_idx_off(index_bytes, offset_bytes, [&](auto i, auto o) {
    using I = decltype(i);
    using O = decltype(o);
    auto run = [&](auto* typed_out) {
      using Out = std::remove_pointer_t<decltype(typed_out)>;
      if (bit_rate == 8) {
        return (int)fbgemm::EmbeddingSpMDM_ref<std::uint8_t, I, O, Out>(
            block_size, output_size, index_size, data_size, input,
            static_cast<const I*>(indices),
            static_cast<const O*>(offsets_or_lengths), weights,
            normalize_by_lengths != 0, typed_out, is_weight_positional != 0,
            use_offsets != 0, output_stride, input_stride,
            scale_bias_last != 0, no_bag != 0, out_kind == 2, false);
      }
      return (int)fbgemm::EmbeddingSpMDMNBit_ref<I, O, Out>(
          bit_rate, block_size, output_size, index_size, data_size, input,
          static_cast<const I*>(indices),
          static_cast<const O*>(offsets_or_lengths), weights,
          normalize_by_lengths != 0, typed_out, is_weight_positional != 0,
          use_offsets != 0, output_stride, input_stride, scale_bias_last != 0,
          out_kind == 2, no_bag != 0, -1);
    };
    if (out_kind == 0) {
      return run(static_cast<float*>(out));
    }
    return run(static_cast<std::uint16_t*>(out));
  });
}

// Tables that are not row-wise quantized: fbgemm::EmbeddingSpMDM_ref<float>
// (in_kind 1), <float16> (2), <uint16_t> with is_bf16_in (3) and
// fbgemm::EmbeddingSpMDMFP8_ref (4).  input_stride in elements.
int ref_embedding_spmdm_plain(
    int in_kind,
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t index_size,
    std::int64_t data_size,
    const void* input,
    const void* indices,
    int index_bytes,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    void* out,
    int out_kind,
    int is_weight_positional,
    int use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride,
    int scale_bias_last,
    int no_bag,
    int exponent_bits,
    int exponent_bias) {
  return dispatch_idx_off(index_bytes, offset_bytes, [&](auto i, auto o) {
    using I = decltype(i);
    using O = decltype(o);
    auto run = [&](auto* typed_out) {
      using Out = std::remove_pointer_t<decltype(typed_out)>;
      const I* idx = static_cast<const I*>(indices);
      const O* off = static_cast<const O*>(offsets_or_lengths);
      if (in_kind == 1) {
        return (int)fbgemm::EmbeddingSpMDM_ref<float, I, O, Out>(
            block_size, output_size, index_size, data_size,
            static_cast<const float*>(input), idx, off, weights,
            normalize_by_lengths != 0, typed_out, is_weight_positional != 0,
            use_offsets != 0, output_stride, input_stride,
            scale_bias_last != 0, no_bag != 0, out_kind == 2, false);
      }
      if (in_kind == 2) {
        return (int)fbgemm::EmbeddingSpMDM_ref<float16, I, O, Out>(
            block_size, output_size, index_size, data_size,
            static_cast<const float16*>(input), idx, off, weights,
            normalize_by_lengths != 0, typed_out, is_weight_positional != 0,
            use_offsets != 0, output_stride, input_stride,
            scale_bias_last != 0, no_bag != 0, out_kind == 2, false);
      }
      if (in_kind == 3) {
        // 16-bit storage whose meaning is_bf16_in selects (InType uint16_t;
        // the float16 struct is always fp16, src/RefImplementations.h:428-440)
        return (int)fbgemm::EmbeddingSpMDM_ref<std::uint16_t, I, O, Out>(
            block_size, output_size, index_size, data_size,
            static_cast<const std::uint16_t*>(input), idx, off, weights,
            normalize_by_lengths != 0, typed_out, is_weight_positional != 0,
            use_offsets != 0, output_stride, input_stride,
            scale_bias_last != 0, no_bag != 0, out_kind == 2, true);
      }
      return (int)fbgemm::EmbeddingSpMDMFP8_ref<I, O, Out>(
          block_size, output_size, index_size, data_size,
          static_cast<const std::uint8_t*>(input), idx, off, weights,
          normalize_by_lengths != 0, typed_out, is_weight_positional != 0,
          use_offsets != 0, output_stride, input_stride, exponent_bits,
          exponent_bias, out_kind == 2);
    };
    if (out_kind == 0) {
      return run(static_cast<float*>(out));
    }
    return run(static_cast<std::uint16_t*>(out));
  });
}

// no_bag with 8-bit output: the reference's row copies.  bit_rate 8:
// EmbeddingSpMDM_ref<uint8_t, I, I, uint8_t>(no_bag = true); bit_rate 4:
// EmbeddingSpMDMNBit_ref<I, I, uint8_t>(4, ..., no_bag = true, output_bit_rate = 4).
int ref_embedding_rows_copy(
    int bit_rate,
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t data_size,
    const std::uint8_t* input,
    const void* indices,
    int index_bytes,
    std::uint8_t* out,
    std::int64_t output_stride,
    std::int64_t input_stride) {
  return dispatch_idx_off(index_bytes, index_bytes, [&](auto i, auto o) {
    using I = decltype(i);
    using O = decltype(o);
    const O dummy_offsets[1] = {0};
    if (bit_rate == 8) {
      return (int)fbgemm::EmbeddingSpMDM_ref<std::uint8_t, I, O, std::uint8_t>(
          block_size, output_size, output_size, data_size, input,
          static_cast<const I*>(indices), dummy_offsets, nullptr, false, out,
          false, true, output_stride, input_stride, true, true, false, false);
    }
    return (int)fbgemm::EmbeddingSpMDMNBit_ref<I, O, std::uint8_t>(
        bit_rate, block_size, output_size, output_size, data_size, input,
        static_cast<const I*>(indices), dummy_offsets, nullptr, false, out,
        false, true, output_stride, input_stride, true, false, true, 4);
  });
}

// fbgemm::EmbeddingSpMDMRowWiseSparse_ref<uint8_t> (:1617) for bit_rate 8,
// fbgemm::EmbeddingSpMDMNBitRowWiseSparse_ref (:1746) for 4 and 2.
int ref_embedding_spmdm_rowwise_sparse(
    int bit_rate,
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t index_size,
    std::int64_t uncompressed_data_size,
    const std::uint8_t* input,
    const void* indices,
    int index_bytes,
    const std::int32_t* compressed_indices_table,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    float* out,
    int is_weight_positional,
    int use_offsets) {
  return dispatch_idx_off(index_bytes, offset_bytes, [&](auto i, auto o) {
    using I = decltype(i);
    using O = decltype(o);
    if (bit_rate == 8) {
      return (int)fbgemm::EmbeddingSpMDMRowWiseSparse_ref<std::uint8_t, I, O>(
          block_size, output_size, index_size, uncompressed_data_size, input,
          static_cast<const I*>(indices), compressed_indices_table,
          static_cast<const O*>(offsets_or_lengths), weights,
          normalize_by_lengths != 0, out, is_weight_positional != 0,
          use_offsets != 0);
    }
    return (int)fbgemm::EmbeddingSpMDMNBitRowWiseSparse_ref<I, O>(
        bit_rate, block_size, output_size, index_size, uncompressed_data_size,
        input, static_cast<const I*>(indices), compressed_indices_table,
        static_cast<const O*>(offsets_or_lengths), weights,
        normalize_by_lengths != 0, out, is_weight_positional != 0,
        use_offsets != 0);
  });
}

// fbgemm::EmbeddingSpMDMRowWiseSparse_ref<float | float16 | uint16_t> (:1617,
// the branch at :1688-1743).  in_kind 1 float, 2 float16, 3 uint16_t (which
// that function reads as fp16 as well).
int ref_embedding_spmdm_plain_rowwise_sparse(
    int in_kind,
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t index_size,
    std::int64_t uncompressed_data_size,
    const void* input,
    const void* indices,
    int index_bytes,
    const std::int32_t* compressed_indices_table,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    float* out,
    int is_weight_positional,
    int use_offsets) {
  return dispatch_idx_off(index_bytes, offset_bytes, [&](auto i, auto o) {
    using I = decltype(i);
    using O = decltype(o);
    auto run = [&](auto* table) {
      using T = std::remove_cv_t<std::remove_pointer_t<decltype(table)>>;
      return (int)fbgemm::EmbeddingSpMDMRowWiseSparse_ref<T, I, O>(
          block_size, output_size, index_size, uncompressed_data_size, table, static_cast<const I*>(indices),
          compressed_indices_table, static_cast<const O*>(offsets_or_lengths), weights, normalize_by_lengths != 0,
          out, is_weight_positional != 0, use_offsets != 0);
    };
    if (in_kind == 1) {
      return run(static_cast<const float*>(input));
    }
    if (in_kind == 2) {
      return run(static_cast<const fbgemm::float16*>(input));
    }
    return run(static_cast<const std::uint16_t*>(input));
  });
}

// The reference's auto-vectorised kernels (src/EmbeddingSpMDMAutovec.cc),
// reached through their generators.  bit_rate 8 -> ...WithStrides_autovec,
// 4/2 -> ...NBitWithStrides_autovec.  A CPU baseline for timing.
int ref_autovec_embedding_spmdm(
    int bit_rate,
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t index_size,
    std::int64_t data_size,
    const std::uint8_t* input,
    const void* indices,
    int index_bytes,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    void* out,
    int out_is_half,
    int is_weight_positional,
    int use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride) {
  const std::int64_t epb = 8 / bit_rate;
  if (output_stride == -1) {
    output_stride = block_size;
  }
  if (input_stride == -1) {
    input_stride = bit_rate == 8 ? block_size + 8
                                 : (block_size + epb - 1) / epb + 4;
  }
  return dispatch_idx_off(index_bytes, offset_bytes, [&](auto i, auto o) {
    using I = decltype(i);
    using O = decltype(o);
    auto run = [&](auto outtag) {
      using OutT = decltype(outtag);
      if (bit_rate == 8) {
        auto fn = fbgemm::GenerateEmbeddingSpMDMWithStrides_autovec<
            std::uint8_t, I, O, OutT>(
            block_size, weights != nullptr, normalize_by_lengths != 0, 16,
            is_weight_positional != 0, use_offsets != 0, output_stride,
            input_stride, true, false, false, false);
        return (int)fn(
            output_size, index_size, data_size, input,
            static_cast<const I*>(indices),
            static_cast<const O*>(offsets_or_lengths), weights,
            static_cast<OutT*>(out));
      }
      auto fn = fbgemm::GenerateEmbeddingSpMDMNBitWithStrides_autovec<
          I, O, OutT>(
          bit_rate, block_size, weights != nullptr, normalize_by_lengths != 0,
          16, is_weight_positional != 0, use_offsets != 0, output_stride,
          input_stride, true, false, false, -1);
      return (int)fn(
          output_size, index_size, data_size, input,
          static_cast<const I*>(indices),
          static_cast<const O*>(offsets_or_lengths), weights,
          static_cast<OutT*>(out));
    };
    return out_is_half ? run(float16{}) : run(float{});
  });
}

// Quantizers.  `use_ref` selects the plain scalar version
// (src/QuantUtils.cc:534-611, :677-718); otherwise the dispatching entry point
// (AVX2 when the CPU has it, src/QuantUtils.cc:613-675, :720-741).
void ref_float_to_fused_8bit_rowwise_sbfloat(
    const float* input,
    std::int64_t rows,
    int cols,
    std::uint8_t* output,
    int use_ref) {
  if (use_ref) {
    fbgemm::FloatOrHalfToFused8BitRowwiseQuantizedSBFloatRef<float>(
        input, (size_t)rows, cols, output);
  } else {
    fbgemm::FloatOrHalfToFused8BitRowwiseQuantizedSBFloat<float>(
        input, (size_t)rows, cols, output);
  }
}

void ref_float_to_fused_nbit_rowwise_sbhalf(
    int bit_rate,
    const float* input,
    std::int64_t rows,
    int cols,
    std::uint8_t* output,
    int use_ref) {
  if (use_ref) {
    fbgemm::FloatOrHalfToFusedNBitRowwiseQuantizedSBHalfRef<float>(
        bit_rate, input, (size_t)rows, cols, output);
  } else {
    fbgemm::FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf<float>(
        bit_rate, input, (size_t)rows, cols, output);
  }
}

// fbgemm::compressed_indices_remap_ref (src/RefImplementations.cc:2308).
void ref_compressed_indices_remap(
    std::int32_t offsets_len,
    const void* indices,
    int index_bytes,
    const std::int32_t* compressed_indices_mapping,
    const void* offsets,
    const float* weights,
    void* out_indices,
    void* out_offsets,
    float* out_weights) {
  if (index_bytes == 8) {
    fbgemm::compressed_indices_remap_ref<std::int64_t>(
        offsets_len, static_cast<const std::int64_t*>(indices),
        compressed_indices_mapping, static_cast<const std::int64_t*>(offsets),
        weights, static_cast<std::int64_t*>(out_indices),
        static_cast<std::int64_t*>(out_offsets), out_weights);
  } else {
    fbgemm::compressed_indices_remap_ref<std::int32_t>(
        offsets_len, static_cast<const std::int32_t*>(indices),
        compressed_indices_mapping, static_cast<const std::int32_t*>(offsets),
        weights, static_cast<std::int32_t*>(out_indices),
        static_cast<std::int32_t*>(out_offsets), out_weights);
  }
}

std::uint16_t ref_float_to_half_rn(float f) {
  return fbgemm::cpu_float2half_rn(f).val;
}

float ref_half_to_float(std::uint16_t h) {
  return fbgemm::cpu_half2float_ref(float16{h});
}

} // extern "C"

/*
 * TEST AND CPU-BASELINE INFRASTRUCTURE - NOT PART OF THE PRODUCT.
 *
 * The reference's fast CPU path for the quantized embedding bag is x86 code
 * that FBGEMM emits at run time with asmjit (src/EmbeddingSpMDM.cc:161-968,
 * src/EmbeddingSpMDMNBit.cc:149-971).  asmjit is an un-vendored submodule of
 * the reference tree, so that path cannot be compiled from the tree alone.
 * PyTorch's libtorch_cpu.so statically bundles a build of FBGEMM, JIT
 * included, and exports the generator templates; this shim reaches the JIT
 * kernels through it.  It is compiled against the FBGEMM headers that ship
 * inside the torch wheel and linked with -ltorch_cpu (see Makefile).
 *
 * Used only by the benchmark's CPU legs (timing) and by a CPU test that checks
 * the JIT result against the scalar reference.  Generators are cached per
 * configuration, as the reference's callers do; each call may be issued from
 * several host threads on disjoint bag ranges.
 */
#include <cstdint>
#include <functional>
#include <map>
#include <mutex>
#include <tuple>

#include "fbgemm/FbgemmEmbedding.h"

namespace {

using Key = std::tuple<int, std::int64_t, int, int, int, int, int, int, int,
                       std::int64_t, std::int64_t, int>;

template <typename I, typename O, typename OutT>
using Fn = typename fbgemm::
    EmbeddingSpMDMKernelSignature<std::uint8_t, I, O, OutT>::Type;

template <typename I, typename O, typename OutT>
Fn<I, O, OutT>& cached(
    int bit_rate,
    std::int64_t block_size,
    bool has_weight,
    bool normalize,
    bool positional,
    bool use_offsets,
    std::int64_t output_stride,
    std::int64_t input_stride) {
  static std::mutex mu;
  static std::map<Key, Fn<I, O, OutT>> cache;
  const Key key{bit_rate, block_size, has_weight, normalize, positional,
                use_offsets, (int)sizeof(I), (int)sizeof(O), (int)sizeof(OutT),
                output_stride, input_stride, 0};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it == cache.end()) {
    Fn<I, O, OutT> fn;
    if (bit_rate == 8) {
      fn = fbgemm::GenerateEmbeddingSpMDMWithStrides<std::uint8_t, I, O, OutT>(
          block_size, has_weight, normalize, 16, positional, use_offsets,
          output_stride, input_stride, true, false, false, false);
    } else {
      fn = fbgemm::GenerateEmbeddingSpMDMNBitWithStrides<I, O, OutT>(
          bit_rate, block_size, has_weight, normalize, 16, positional,
          use_offsets, output_stride, input_stride, true, false, false, -1);
    }
    it = cache.emplace(key, std::move(fn)).first;
  }
  return it->second;
}

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

// fbgemm::GenerateEmbeddingSpMDMWithStrides<uint8_t,...> (bit_rate 8) or
// fbgemm::GenerateEmbeddingSpMDMNBitWithStrides (bit_rate 4, 2), then one call
// of the returned functor.
int jit_embedding_spmdm(
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
      auto& fn = cached<I, O, std::uint16_t>(
          bit_rate, block_size, weights != nullptr, normalize_by_lengths != 0,
          is_weight_positional != 0, use_offsets != 0, output_stride,
          input_stride);
      return (int)fn(
          output_size, index_size, data_size, input,
          static_cast<const I*>(indices),
          static_cast<const O*>(offsets_or_lengths), weights,
          static_cast<std::uint16_t*>(out));
    }
    auto& fn = cached<I, O, float>(
        bit_rate, block_size, weights != nullptr, normalize_by_lengths != 0,
        is_weight_positional != 0, use_offsets != 0, output_stride,
        input_stride);
    return (int)fn(
        output_size, index_size, data_size, input,
        static_cast<const I*>(indices),
        static_cast<const O*>(offsets_or_lengths), weights,
        static_cast<float*>(out));
  });
}

// fbgemm::GenerateEmbeddingSpMDMRowWiseSparse<uint8_t,...> (bit_rate 8) or
// fbgemm::GenerateEmbeddingSpMDMNBitRowWiseSparse (4, 2).
int jit_embedding_spmdm_rowwise_sparse(
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
    typename fbgemm::EmbeddingSpMDMRowWiseSparseKernelSignature<
        std::uint8_t, I, O>::Type fn;
    if (bit_rate == 8) {
      fn = fbgemm::GenerateEmbeddingSpMDMRowWiseSparse<std::uint8_t, I, O>(
          block_size, weights != nullptr, normalize_by_lengths != 0, 16,
          is_weight_positional != 0, use_offsets != 0);
    } else {
      fn = fbgemm::GenerateEmbeddingSpMDMNBitRowWiseSparse<I, O>(
          bit_rate, block_size, weights != nullptr, normalize_by_lengths != 0,
          16, is_weight_positional != 0, use_offsets != 0);
    }
    return (int)fn(
        output_size, index_size, uncompressed_data_size, input,
        static_cast<const I*>(indices),
        static_cast<const O*>(offsets_or_lengths), weights, out,
        compressed_indices_table);
  });
}

// One whole batch split into `threads` contiguous bag ranges, one OpenMP thread
// each - how the reference's callers and benchmarks parallelise this kernel
// (fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:67-72,
// bench/EmbeddingSpMDM8BitBenchmark.cc:394-396): the kernel itself is
// single-threaded.  Offsets flavour; every range is one functor call on a
// slice (offsets need not start at zero).  compressed_indices_table may be
// null.  Returns 1 if every range returned true.
int jit_embedding_spmdm_batch_parallel(
    int bit_rate,
    std::int64_t block_size,
    std::int64_t output_size,
    std::int64_t data_size,
    const std::uint8_t* input,
    const void* indices,
    int index_bytes,
    const void* offsets,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    void* out,
    int out_is_half,
    const std::int32_t* compressed_indices_table,
    int threads) {
  if (threads < 1) {
    threads = 1;
  }
  auto off_at = [&](std::int64_t m) -> std::int64_t {
    return offset_bytes == 8 ? static_cast<const std::int64_t*>(offsets)[m]
                             : static_cast<const std::int32_t*>(offsets)[m];
  };
  const std::int64_t base = off_at(0);
  int all_ok = 1;
#pragma omp parallel for num_threads(threads) schedule(static, 1) reduction(&& : all_ok)
  for (int t = 0; t < threads; ++t) {
    const std::int64_t lo = output_size * t / threads;
    const std::int64_t hi = output_size * (t + 1) / threads;
    if (hi <= lo) {
      continue;
    }
    const std::int64_t i0 = off_at(lo) - base;
    const std::int64_t n = off_at(hi) - off_at(lo);
    const char* idx = static_cast<const char*>(indices) + i0 * index_bytes;
    const char* off = static_cast<const char*>(offsets) + lo * offset_bytes;
    const float* w = weights ? weights + i0 : nullptr;
    const std::size_t esize = out_is_half ? 2 : 4;
    char* o = static_cast<char*>(out) + (std::size_t)lo * block_size * esize;
    int ok;
    if (compressed_indices_table) {
      ok = jit_embedding_spmdm_rowwise_sparse(
          bit_rate, block_size, hi - lo, n, data_size, input, idx, index_bytes,
          compressed_indices_table, off, offset_bytes, w, normalize_by_lengths,
          reinterpret_cast<float*>(o), 0, 1);
    } else {
      ok = jit_embedding_spmdm(
          bit_rate, block_size, hi - lo, n, data_size, input, idx, index_bytes,
          off, offset_bytes, w, normalize_by_lengths, o, out_is_half, 0, 1, -1,
          -1);
    }
    all_ok = all_ok && ok == 1;
  }
  return all_ok;
}

} // extern "C"

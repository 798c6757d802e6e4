// extern "C" access to the reference's table-batched CPU operator.
//
// TEST INFRASTRUCTURE.  The functions called here are the reference's own:
// fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp of
// FBGEMM, rendered by oracle/render_tbe_template.py and compiled by
// oracle/Makefile (target `tbe`) against torch's ATen headers, with the
// generators they call (fbgemm::GenerateEmbeddingSpMDM*WithStrides) coming
// from the FBGEMM bundled in libtorch_cpu.so.  This file only wraps caller
// memory in at::Tensor views and copies results out.
#include <ATen/ATen.h>

#include <cstdint>
#include <cstring>
#include <string>

using at::Tensor;

// Declarations as in the rendered template (:124-129, :208-226, :678-697, :1142-1146, :1223-1227 of the rendering).
void pruned_hashmap_insert_unweighted_cpu(Tensor indices, Tensor dense_indices, Tensor offsets, Tensor hash_table,
                                          Tensor hash_table_offsets);
Tensor pruned_hashmap_lookup_unweighted_cpu(Tensor indices, Tensor offsets, Tensor hash_table, Tensor hash_table_offsets);
Tensor pruned_array_lookup_cpu(Tensor indices, Tensor offsets, Tensor index_remappings, Tensor index_remappings_offsets);
Tensor int_nbit_split_embedding_codegen_forward_unweighted_cpu(
    Tensor dev_weights, Tensor uvm_weights, Tensor weights_placements, Tensor weights_offsets, Tensor weights_tys,
    Tensor D_offsets, int64_t total_D, Tensor indices, Tensor offsets, int64_t pooling_mode, int64_t row_alignment,
    int64_t output_dtype, int64_t fp8_exponent_bits, int64_t fp8_exponent_bias, bool scale_bias_last);
Tensor int_nbit_split_embedding_codegen_forward_weighted_cpu(
    Tensor dev_weights, Tensor uvm_weights, Tensor weights_placements, Tensor weights_offsets, Tensor weights_tys,
    Tensor D_offsets, int64_t total_D, Tensor indices, Tensor offsets, int64_t pooling_mode, int64_t row_alignment,
    Tensor indice_weights, int64_t output_dtype, int64_t fp8_exponent_bits, int64_t fp8_exponent_bias,
    bool scale_bias_last);
Tensor int_nbit_split_embedding_nobag_codegen_forward_unweighted_cpu(
    Tensor dev_weights, Tensor uvm_weights, Tensor weights_placements, Tensor weights_offsets, Tensor weights_tys,
    int64_t D, Tensor indices, Tensor offsets, int64_t pooling_mode, int64_t row_alignment, int64_t output_dtype,
    int64_t fp8_exponent_bits, int64_t fp8_exponent_bias, bool scale_bias_last);

namespace {

thread_local std::string g_error;

at::ScalarType int_type(int bytes) {
  return bytes == 8 ? at::kLong : at::kInt;
}

Tensor view(const void* p, int64_t n, at::ScalarType ty) {
  return at::from_blob(const_cast<void*>(p), {n}, at::TensorOptions().dtype(ty));
}

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}

}  // namespace

extern "C" {

__attribute__((visibility("default"))) const char* ref_tbe_last_error() {
  return g_error.c_str();
}

// hash_table: [hash_rows][2] integers of hash_bytes, -1 = empty; filled in place.
__attribute__((visibility("default"))) int ref_tbe_pruned_hashmap_insert(
    int32_t T, int32_t B, const void* indices, const void* dense_indices, const void* offsets, int index_bytes,
    void* hash_table, int hash_bytes, int64_t hash_rows, const int64_t* hash_table_offsets) {
  return guarded([&] {
    const auto it = int_type(index_bytes);
    Tensor off = view(offsets, (int64_t)T * B + 1, it);
    const int64_t n = index_bytes == 8 ? off[-1].item<int64_t>() : (int64_t)off[-1].item<int32_t>();
    Tensor ht = at::from_blob(hash_table, {hash_rows, 2}, at::TensorOptions().dtype(int_type(hash_bytes)));
    pruned_hashmap_insert_unweighted_cpu(view(indices, n, it), view(dense_indices, n, it), off, ht,
                                         view(hash_table_offsets, T + 1, at::kLong));
  });
}

__attribute__((visibility("default"))) int ref_tbe_pruned_hashmap_lookup(
    int32_t T, int32_t B, const void* indices, const void* offsets, int index_bytes, const void* hash_table,
    int hash_bytes, int64_t hash_rows, const int64_t* hash_table_offsets, void* dense_indices) {
  return guarded([&] {
    const auto it = int_type(index_bytes);
    Tensor off = view(offsets, (int64_t)T * B + 1, it);
    const int64_t n = index_bytes == 8 ? off[-1].item<int64_t>() : (int64_t)off[-1].item<int32_t>();
    Tensor ht = at::from_blob(const_cast<void*>(hash_table), {hash_rows, 2},
                              at::TensorOptions().dtype(int_type(hash_bytes)));
    Tensor out = pruned_hashmap_lookup_unweighted_cpu(view(indices, n, it), off, ht,
                                                      view(hash_table_offsets, T + 1, at::kLong));
    std::memcpy(dense_indices, out.data_ptr(), (size_t)n * index_bytes);
  });
}

__attribute__((visibility("default"))) int ref_tbe_pruned_array_lookup(
    int32_t T, int32_t B, const void* indices, const void* offsets, int index_bytes, const void* remappings,
    int remap_bytes, int64_t remap_len, const int64_t* remappings_offsets, void* dense_indices) {
  return guarded([&] {
    const auto it = int_type(index_bytes);
    Tensor off = view(offsets, (int64_t)T * B + 1, it);
    const int64_t n = index_bytes == 8 ? off[-1].item<int64_t>() : (int64_t)off[-1].item<int32_t>();
    Tensor out = pruned_array_lookup_cpu(view(indices, n, it), off, view(remappings, remap_len, int_type(remap_bytes)),
                                         view(remappings_offsets, T + 1, at::kLong));
    std::memcpy(dense_indices, out.data_ptr(), (size_t)n * index_bytes);
  });
}

// The pooled operator (nobag = 0; `dims` = D_offsets[T + 1], `dim` = total_D)
// or the sequence operator (nobag = 1; `dims` unused, `dim` = D).  All tables
// live in `dev_weights` (placement HOST).  `indice_weights` null = unweighted.
// The result is copied to `out` (out_bytes must match its size).
__attribute__((visibility("default"))) int ref_tbe_forward(
    int nobag, const uint8_t* dev_weights, int64_t weights_bytes, const int64_t* weights_offsets,
    const uint8_t* weights_tys, int32_t T, const int32_t* dims, int64_t dim, const void* indices, const void* offsets,
    int index_bytes, int32_t B, int64_t pooling_mode, int64_t row_alignment, const float* indice_weights,
    int64_t output_dtype, int64_t fp8_exponent_bits, int64_t fp8_exponent_bias, int scale_bias_last, void* out,
    int64_t out_bytes) {
  return guarded([&] {
    const auto it = int_type(index_bytes);
    Tensor off = view(offsets, (int64_t)T * B + 1, it);
    const int64_t n = index_bytes == 8 ? off[-1].item<int64_t>() : (int64_t)off[-1].item<int32_t>();
    Tensor w = view(dev_weights, weights_bytes, at::kByte);
    Tensor uvm = at::empty({0}, at::kByte);
    Tensor placements = at::full({T}, 3, at::kInt);  // PlacementType::HOST (embedding_common.h)
    Tensor w_off = view(weights_offsets, T, at::kLong);
    Tensor tys = view(weights_tys, T, at::kByte);
    Tensor idx = view(indices, n, it);
    Tensor res;
    if (nobag) {
      res = int_nbit_split_embedding_nobag_codegen_forward_unweighted_cpu(
          w, uvm, placements, w_off, tys, dim, idx, off, pooling_mode, row_alignment, output_dtype, fp8_exponent_bits,
          fp8_exponent_bias, scale_bias_last != 0);
    } else if (indice_weights) {
      res = int_nbit_split_embedding_codegen_forward_weighted_cpu(
          w, uvm, placements, w_off, tys, view(dims, T + 1, at::kInt), dim, idx, off, pooling_mode, row_alignment,
          view(indice_weights, n, at::kFloat), output_dtype, fp8_exponent_bits, fp8_exponent_bias,
          scale_bias_last != 0);
    } else {
      res = int_nbit_split_embedding_codegen_forward_unweighted_cpu(
          w, uvm, placements, w_off, tys, view(dims, T + 1, at::kInt), dim, idx, off, pooling_mode, row_alignment,
          output_dtype, fp8_exponent_bits, fp8_exponent_bias, scale_bias_last != 0);
    }
    res = res.contiguous();
    TORCH_CHECK((int64_t)res.nbytes() == out_bytes, "result has ", res.nbytes(), " bytes, caller expects ", out_bytes);
    std::memcpy(out, res.data_ptr(), (size_t)out_bytes);
  });
}

}  // extern "C"

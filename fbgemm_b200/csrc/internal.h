// Declarations shared by the translation units of libfbgemm_b200.so.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "fbgemm_b200/embedding_c_api.h"

namespace fbgemm_b200 {

// Flag bits of SpmdmParams::flags.
enum : uint32_t {
  kIdx64 = 1u << 0,       // indices are int64 (else int32)
  kOff64 = 1u << 1,       // offsets are int64 (else int32)
  kOutHalf = 1u << 2,     // fp16 output (else fp32)
  kWeighted = 1u << 3,    // per-sample weights present
  kPositional = 1u << 4,  // weights indexed by position inside the bag
  kNormalize = 1u << 5,   // multiply the pooled row by 1/len
  kPruned = 1u << 6,      // indices go through compressed_indices_table
  kOutVec = 1u << 7,      // output rows allow vector stores
  kSbFirst = 1u << 8,     // fp16 scale,bias at the start of the row; index -1 = pruned row
  kOutBf16 = 1u << 9,     // bf16 output
  kNoBag = 1u << 10,      // one index per output row, no offsets
  kAbsOffsets = 1u << 11, // offsets index the whole index array (no rebasing, no final size check)
};

// Everything one lookup launch needs; passed by value to the kernel.
struct SpmdmParams {
  const uint8_t* table;       // fused rows
  const void* indices;        // int32/int64 [index_size]
  const void* offsets;        // int32/int64 [output_size + 1]
  const float* weights;       // [index_size] or positional, may be null
  const int32_t* cit;         // compressed_indices_table or null
  void* out;                  // fp32/fp16 [output_size x output_stride]
  int32_t* status;            // {code, bag, position, value}
  int64_t data_size;          // rows an index may address
  int64_t input_stride;       // bytes between table rows
  int64_t output_stride;      // elements between output rows
  int64_t output_size;        // bags
  int64_t index_size;         // indices
  int32_t block_size;         // D
  int32_t data_bytes;         // packed payload bytes per row
  int32_t data_row_off;       // offset of the payload inside a table row (0, or 4 when scale,bias come first)
  int32_t sb_row_off;         // offset of scale,bias inside a table row
  int32_t data_off;           // offset of the payload inside a staged row
  int32_t sb_off;             // offset of scale,bias inside a staged row
  int32_t row_bytes;          // payload + scale,bias bytes actually read
  int32_t pitch;              // bytes between staged rows in shared memory
  int32_t rows_per_wave;      // rows one bag stages at a time
  int32_t group_smem;         // shared-memory bytes per bag slot
  int32_t copy_width;         // 16/8/4: cp.async granule; 0: byte-wise path
  uint32_t flags;
  // Tables that are not row-wise quantized (plain_kernels.cu): 0 = quantized,
  // else FBGEMM_B200_IN_F32 / _F16 / _BF16 / _FP8 and the FP8 format.
  int32_t in_kind;
  int32_t fp8_exponent_bits;
  int32_t fp8_exponent_bias;
  // Batch-wise redistribution of the pooled rows (table-wise sharding): when
  // num_peers > 0, bag b is written to peer_out[b / bags_per_peer] at row
  // b % bags_per_peer instead of `out`.  The pointers may be peer-GPU memory.
  int32_t num_peers;
  int64_t bags_per_peer;
  void* peer_out[FBGEMM_B200_MAX_PEERS];
};

// Where the pooled row of `bag` goes (byte pointer; esize = bytes per element).
__device__ __forceinline__ char* output_row(const SpmdmParams& p, int64_t bag, int esize) {
  if (p.num_peers > 0) {
    const int64_t d = bag / p.bags_per_peer;
    return static_cast<char*>(p.peer_out[d]) + (bag - d * p.bags_per_peer) * p.output_stride * esize;
  }
  return static_cast<char*>(p.out) + bag * p.output_stride * esize;
}

// One lookup kernel launch (spmdm_kernels.cu).  Returns cudaSuccess or the
// launch error; never synchronises.
cudaError_t launch_spmdm(const SpmdmParams& p, int bit_rate, cudaStream_t stream);

// The argument of one multi-table launch: up to kMultiTables tables of the
// same kernel variant, passed by value so that, like the single-table
// kernel's, their parameters live in constant memory.  Table t owns the blocks
// [first_block[t], first_block[t + 1]).
constexpr int kMultiTables = 16;
struct MultiArgs {
  int32_t count;
  int32_t first_block[kMultiTables + 1];
  SpmdmParams t[kMultiTables];
};
static_assert(sizeof(MultiArgs) <= 4096, "one kernel argument, within the classic 4 KB of parameter space");

// Several tables per call (spmdm_kernels.cu): the tables grouped by kernel
// variant, each group cut into launches of up to kMultiTables tables.  Built
// once for a fixed set of pointers, launched as often as wanted.
struct MultiPlan {
  struct Launch {
    void (*fn)(const MultiArgs);
    unsigned blocks;    // grid size
    MultiArgs args;
  };
  std::vector<Launch> groups;
  std::vector<std::pair<SpmdmParams, int>> singles;  // (parameters, bit rate): one launch each
  // The launches of one call overlap: all but the first go to side streams
  // that fork from, and join, the caller's stream through these events.
  static constexpr int kSideStreams = 3;
  cudaStream_t side[kSideStreams] = {};
  cudaEvent_t fork = nullptr;
  cudaEvent_t join[kSideStreams] = {};
  MultiPlan() = default;
  MultiPlan(const MultiPlan&) = delete;
  MultiPlan& operator=(const MultiPlan&) = delete;
  ~MultiPlan();
};
cudaError_t build_multi_plan(const std::vector<SpmdmParams>& tables, const std::vector<int>& bit_rates, MultiPlan* plan);
cudaError_t launch_multi_plan(const MultiPlan& plan, cudaStream_t stream);

// The lookup on a table that is not row-wise quantized (plain_kernels.cu).
cudaError_t launch_plain_rows(const SpmdmParams& p, cudaStream_t stream);

// no_bag with 8-bit output: byte copies of the indexed rows (plain_kernels.cu).
cudaError_t launch_rows_copy(
    const uint8_t* table,
    const void* indices,
    int index_bytes,
    int64_t rows_out,
    int64_t data_size,
    int64_t input_stride,
    uint8_t* out,
    int64_t out_pitch,
    int64_t width,
    int32_t* status,
    cudaStream_t stream);

// Exclusive scan of `n` int32/int64 lengths into int64 offsets[n + 1]
// (scan_kernels.cu).  `block_sums` is scratch of scan_scratch_elems(n) int64.
size_t scan_scratch_elems(int64_t n);
cudaError_t launch_length_scan(
    const void* lengths,
    int length_bytes,
    int64_t n,
    int64_t* offsets,
    int64_t* block_sums,
    cudaStream_t stream);

// compressed_indices_remap (remap_kernels.cu).  `scratch` holds
// remap_scratch_bytes(index_size) bytes; out-of-range indices are recorded in
// `status` and dropped.
size_t remap_scratch_bytes(int64_t index_size);
cudaError_t launch_compressed_indices_remap(
    int32_t offsets_len,
    const void* indices,
    int index_bytes,
    int64_t index_size,
    const int32_t* mapping,
    int64_t mapping_size,
    const void* offsets,
    const float* weights,
    void* out_indices,
    void* out_offsets,
    float* out_weights,
    int32_t* status,
    void* scratch,
    cudaStream_t stream);

// Sparse -> dense index remapping of table-batched pruned tables through a
// per-table hash map (hashmap = true; map is [.][2] integers) or a per-table
// array (pruned_lookup_kernels.cu).  One launch, nothing allocated.
cudaError_t launch_pruned_lookup(
    bool hashmap,
    int32_t T,
    int32_t B,
    const void* indices,
    const void* offsets,
    int index_bytes,
    int64_t index_size,
    const void* map,
    int map_bytes,
    const int64_t* map_offsets,
    void* dense_indices,
    int32_t* status,
    cudaStream_t stream);

// Fills the hash maps of launch_pruned_lookup on the device (compare-and-swap per position).
cudaError_t launch_pruned_hashmap_insert(
    int32_t T,
    int32_t B,
    const void* indices,
    const void* dense_indices,
    const void* offsets,
    int index_bytes,
    int64_t index_size,
    void* hash_table,
    int hash_bytes,
    const int64_t* hash_table_offsets,
    int32_t* status,
    cudaStream_t stream);

// Sequence ("nobag") lookup over the tables of a table-batched call
// (sequence_kernels.cu): one output row per index position, one launch.
using SequenceTable = fbgemm_b200_sequence_table;
cudaError_t launch_sequence_lookup(
    const uint8_t* weights,
    const SequenceTable* tables,
    int32_t T,
    int32_t B,
    int32_t D,
    const void* indices,
    const void* offsets,
    int index_bytes,
    int64_t index_size,
    void* out,
    int out_kind,
    int64_t out_row_bytes,
    bool scale_bias_last,
    int fp8_exponent_bits,
    int fp8_exponent_bias,
    int32_t* status,
    cudaStream_t stream);

// One contiguous piece of a call's inputs, from page-locked host memory (the
// address the GPU sees it at) to device memory; three of them per launch
// (stage_kernels.cu).  Empty segments have bytes = 0.
struct StageSegment {
  const void* src;
  void* dst;
  size_t bytes;
};
cudaError_t launch_stage_inputs(const StageSegment (&seg)[3], cudaStream_t stream);
// A call's 4-word error record to page-locked host memory (`host_view` is the address the GPU sees it at).
cudaError_t launch_status_to_host(const int32_t* status, int32_t* host_view, cudaStream_t stream);

// Counters between the GPUs of a sharded lookup (peer_sync_kernels.cu): publish
// `value` to n words (one per peer, possibly in peer memory), and wait until n
// local words have reached `value`, giving up after timeout_us with a
// FBGEMM_B200_STATUS_PEER_TIMEOUT record in `status`.
cudaError_t launch_peer_signal(void* const* flags, int n, uint64_t value, cudaStream_t stream);
cudaError_t launch_peer_wait(const void* flags, int n, uint64_t value, uint64_t timeout_us, int32_t* status,
                             cudaStream_t stream);

// Row-wise quantizers (quantize_kernels.cu).
cudaError_t launch_quantize_8bit(const float* in, int64_t rows, int cols, uint8_t* out, cudaStream_t s);
cudaError_t launch_quantize_nbit(int bit_rate, const float* in, int64_t rows, int cols, uint8_t* out, cudaStream_t s);

// A device allocation and its size.
struct DeviceBuffer {
  void* ptr = nullptr;
  size_t bytes = 0;
};

// Validate `cfg`, build the kernel parameters of one functor call and enqueue
// it on `stream` (c_api.cu).  All pointers are device pointers; `status` is
// the 4-word error record.  In lengths mode `scan` is grown on demand to hold
// the scanned offsets.  Returns 0 or a negative FBGEMM_B200_E* code.
int enqueue_lookup(
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
    void* const* peer_out = nullptr,
    int num_peers = 0,
    int64_t bags_per_peer = 0);

// The validation and parameter set-up half of enqueue_lookup (offsets are left
// for the caller to fill in).
int build_lookup_params(
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
    SpmdmParams* params);

// Process-wide count of kernels launched by this library.
extern std::atomic<uint64_t> g_launch_count;

// fbgemm_b200_set_kernel_choice: which lookup kernel quantized rows take.
extern std::atomic<int> g_kernel_choice;

// Thread-local error text behind fbgemm_b200_last_error().
void set_error(const std::string& msg);
int fail_cuda(cudaError_t e, const char* what);

}  // namespace fbgemm_b200

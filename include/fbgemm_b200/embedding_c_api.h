/*
 * fbgemm_b200 - C ABI of the B200 (sm_100a) quantized embedding-bag path.
 *
 * This is the drop-in boundary: plain pointers and sizes, no C++ or torch
 * types.  The C++ generator templates in FbgemmEmbedding.h (same directory)
 * and the Python mirror in fbgemm_b200/ are thin layers over these entry
 * points.  Each entry point names the interface of the reference (FBGEMM,
 * paths relative to its source tree) that it stands in for.
 *
 * Conventions
 *   - "lookup" entry points return 1 where the reference functor returns
 *     true, 0 where it returns false (index out of range, a bag that runs
 *     past index_size, or offsets that do not add up to index_size), and a
 *     negative FBGEMM_B200_E* code when the call itself failed.  As in the
 *     reference, the output is unspecified when the result is 0.
 *   - Nothing here falls back to the CPU: without a usable CUDA device every
 *     call fails with FBGEMM_B200_ECUDA.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream).
 */
#ifndef FBGEMM_B200_EMBEDDING_C_API_H_
#define FBGEMM_B200_EMBEDDING_C_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FBGEMM_B200_API __attribute__((visibility("default")))
#else
#define FBGEMM_B200_API
#endif

/* Error codes (negative). */
#define FBGEMM_B200_EINVAL (-1) /* bad or unsupported argument              */
#define FBGEMM_B200_ECUDA (-2)  /* a CUDA runtime call failed               */
#define FBGEMM_B200_ENOMEM (-3) /* device or pinned allocation failed       */
#define FBGEMM_B200_EBUSY (-4)  /* pipeline lane still has work in flight   */

/* Output element types (OutType of the reference generators). */
#define FBGEMM_B200_OUT_F32 0
#define FBGEMM_B200_OUT_F16 1
#define FBGEMM_B200_OUT_BF16 2 /* is_bf16_out = true with a 16-bit OutType:
                                  (bits + 0x8000) >> 16, as cpu_float2bfloat16,
                                  include/fbgemm/FloatConversion.h:312-315 */

#define FBGEMM_B200_OUT_U8 3   /* no_bag only: output row m is a byte copy of
                                  table row indices[m].  8-bit rows: the first
                                  min(output_stride, input_stride) bytes, output
                                  rows output_stride bytes apart; 4-bit rows
                                  (the reference's int4 -> int4 sequence
                                  lookup): input_stride bytes, rows input_stride
                                  apart (src/RefImplementations.cc:1235-1254,
                                  :1467-1485)                                  */

/* Input row types (InType of the reference generators). */
#define FBGEMM_B200_IN_QUANTIZED 0
#define FBGEMM_B200_IN_F32 1
#define FBGEMM_B200_IN_F16 2
#define FBGEMM_B200_IN_BF16 3
#define FBGEMM_B200_IN_FP8 4

/* Why a lookup returned 0 (first word of the status record). */
#define FBGEMM_B200_STATUS_OK 0
#define FBGEMM_B200_STATUS_BAD_INDEX 1   /* idx < 0 || idx >= data_size      */
#define FBGEMM_B200_STATUS_BAG_OVERRUN 2 /* current + len > index_size       */
#define FBGEMM_B200_STATUS_SIZE_MISMATCH 3 /* sum of lengths != index_size   */
#define FBGEMM_B200_STATUS_TABLE_FULL 4 /* hash-map insert found no free slot */
#define FBGEMM_B200_STATUS_PEER_TIMEOUT 5 /* a peer's counter did not arrive in time */

/* Number of status slots a context owns (see fbgemm_b200_spmdm_launch). */
#define FBGEMM_B200_STATUS_SLOTS 1024
/* Number of staging lanes of the host-pointer pipeline. */
#define FBGEMM_B200_HOST_LANES 16
/* Status slots a caller may pass: 0 .. FBGEMM_B200_USER_SLOTS - 1.  The rest
 * are the library's (one for the index remap, one per host-pointer lane). */
#define FBGEMM_B200_USER_SLOTS (FBGEMM_B200_STATUS_SLOTS - FBGEMM_B200_HOST_LANES - 1)

typedef struct fbgemm_b200_ctx fbgemm_b200_ctx;

/*
 * What a generator call fixes.  Mirrors the arguments of
 *   GenerateEmbeddingSpMDMWithStrides      include/fbgemm/FbgemmEmbedding.h:94-117
 *   GenerateEmbeddingSpMDMNBitWithStrides  include/fbgemm/FbgemmEmbedding.h:149-174
 *   GenerateEmbeddingSpMDM[NBit]RowWiseSparse               ...:229-262
 * (`prefetch` and THREAD_LOCAL have no meaning on a GPU and are not carried.)
 */
typedef struct fbgemm_b200_spmdm_config {
  int32_t bit_rate;     /* 8: rows of uint8 + fp32 scale,bias; 4 or 2: packed
                           little-endian within the byte + fp16 scale,bias
                           (see scale_bias_first for the other row layout)   */
  int32_t index_bytes;  /* sizeof(IndexType): 4 or 8                         */
  int32_t offset_bytes; /* sizeof(OffsetType): 4 or 8                        */
  int32_t out_dtype;    /* FBGEMM_B200_OUT_F32 / _F16                        */
  int64_t block_size;   /* embedding dimension D (elements)                  */
  int64_t output_stride; /* elements between output rows; -1 = block_size    */
  int64_t input_stride; /* bytes between table rows; -1 = fused row size     */
  int32_t has_weight;
  int32_t normalize_by_lengths;
  int32_t is_weight_positional;
  int32_t use_offsets;  /* 1: offsets[output_size+1]; 0: lengths[output_size]*/
  int32_t scale_bias_first; /* 1 = the generators' scale_bias_last = false, the
                           row layout of table-batched embeddings: fp16 scale
                           and bias (4 bytes) at the START of the row, for
                           8-bit rows too, and an index of -1 is a pruned row
                           that is skipped (src/RefImplementations.cc:1223-1229,
                           :1299-1303, :1316-1324).  0 = scale, bias last.   */
  int32_t no_bag;       /* 1 = the generators' no_bag = true: output row m is
                           the dequantized row indices[m] (times weights[m]),
                           output_size rows, no offsets, no normalisation
                           (src/RefImplementations.cc:1235-1288); 8-bit rows,
                           fp32 / fp16 / bf16 output                         */
  int32_t absolute_offsets; /* 1 = offsets index the caller's WHOLE index (and
                           weight) array: bag m covers indices[offsets[m] ..
                           offsets[m+1]) with `indices` not advanced to the
                           table's first index, index_size = length of the
                           whole array, and the final check "sum of lengths ==
                           index_size" does not apply.  This is how one table of
                           a table-batched call (offsets of shape T*B+1,
                           fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:381-387)
                           is pooled without reading offsets[t*B] on the host.
                           Offsets flavour only.  0 = the functor's convention */
  int32_t in_dtype;     /* FBGEMM_B200_IN_QUANTIZED (0): fused row-wise quantized
                           rows, bit_rate applies.  Otherwise the table is not
                           quantized - InType float / float16 / uint16_t of
                           GenerateEmbeddingSpMDM[WithStrides] or the rows of
                           GenerateEmbeddingSpMDMFP8WithStrides
                           (include/fbgemm/FbgemmEmbedding.h:65-117,185-203):
                           _F32, _F16, _BF16 (is_bf16_in), _FP8.  bit_rate is
                           ignored, there is no scale or bias, and
                           scale_bias_first only makes -1 a pruned index       */
  int32_t fp8_exponent_bits; /* FP8 rows only (the generator's exponent_bits)  */
  int32_t fp8_exponent_bias; /* FP8 rows only (the generator's exponent_bias)  */
} fbgemm_b200_spmdm_config;

/* ---- context ----------------------------------------------------------- */

/* One context per (process, device).  Owns the status slots, the scratch used
 * by the lengths (use_offsets = 0) mode, the registry of device-resident
 * tables and the staging lanes of the host-pointer pipeline.  Thread-safe. */
FBGEMM_B200_API int fbgemm_b200_ctx_create(int device, fbgemm_b200_ctx** ctx);
FBGEMM_B200_API void fbgemm_b200_ctx_destroy(fbgemm_b200_ctx* ctx);

/* Text of the last error raised on the calling thread ("" if none). */
FBGEMM_B200_API const char* fbgemm_b200_last_error(void);

/* Kernels launched by this library in this process so far. */
FBGEMM_B200_API uint64_t fbgemm_b200_launch_count(void);

/* Generation-time check of a configuration.  Stands in for the argument
 * checks of the reference generators (src/EmbeddingSpMDMNBit.cc:999-1001,
 * src/EmbeddingSpMDM.cc:999-1017).  Returns 0 or FBGEMM_B200_EINVAL. */
FBGEMM_B200_API int fbgemm_b200_spmdm_check_config(const fbgemm_b200_spmdm_config* cfg);

/* ---- pooled lookup, device pointers ------------------------------------ */

/*
 * One call of the functor that the reference generators return
 * (EmbeddingSpMDMKernelSignature<>::Type, include/fbgemm/FbgemmEmbedding.h:41-49;
 * with a non-NULL compressed_indices_table the row-wise-sparse signature,
 * ...:205-222, whose third argument is the UNCOMPRESSED row count and whose
 * output is fp32 with dense strides).  Arithmetic follows
 * src/RefImplementations.cc:1290-1346 (8-bit), :1485-1541 (N-bit) and
 * :1746-1822 (pruned) operation for operation, so fp32 results are bit-equal.
 *
 * All pointers are device pointers valid on the context's device.  The call
 * enqueues work on `stream` and returns without synchronising; it allocates
 * nothing except, in lengths mode (cfg->use_offsets = 0), the scratch for the
 * scanned offsets: one grow-only buffer per stream the context has seen, so
 * lengths-mode calls on different streams may overlap; growing a buffer frees
 * and allocates device memory, which waits for the device - warm up with the
 * largest batch, or use offsets, where that matters.
 * Errors found by the kernel are recorded first-writer-wins in status slot
 * `slot` (0 <= slot < FBGEMM_B200_USER_SLOTS; the slots above belong to the
 * library); read it with fbgemm_b200_status_read once the stream has caught
 * up.  Calls that overlap on the GPU should use distinct slots.
 *
 * Returns 0 when enqueued, or a negative error code.
 */
FBGEMM_B200_API int fbgemm_b200_spmdm_launch(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets_or_lengths,
    const float* weights, /* NULL unless cfg->has_weight */
    void* out,
    const int32_t* compressed_indices_table, /* NULL = dense table */
    int slot,
    void* stream);

/*
 * Table-wise sharding over the GPUs of one box: the lookup of a table owned by
 * this GPU for the whole (global) batch, with the pooled rows written straight
 * to where the batch-wise layout wants them - bag b goes to row
 * b % bags_per_peer of peer_out[b / bags_per_peer], which may be a buffer in a
 * peer GPU's memory (mapped through CUDA IPC / symmetric memory, stores cross
 * NVLink).  This is the lookup and the all-to-all of the pooled outputs in one
 * kernel; there is no staging buffer and no separate collective.  The
 * reference has neither step (its callers loop over tables on one host,
 * fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:343-473);
 * the layout written is that caller's `output + D_start` with
 * output_stride = total_D, cut batch-wise.
 * Each peer_out[i] already includes the column offset of this table;
 * cfg->output_stride is the row pitch of the destination buffers.  Offsets
 * flavour only, dense tables only.  The caller orders the peers' reads after
 * this kernel (stream/event or barrier).  Returns 0 or a negative code.
 */
#define FBGEMM_B200_MAX_PEERS 8
FBGEMM_B200_API int fbgemm_b200_spmdm_launch_sharded(
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
    void* stream);

/*
 * Several tables in one call - what the reference's multi-table caller does
 * with a loop of functor calls, one per table, writing `output + D_start` with
 * output_stride = total_D
 * (fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:343-473;
 * the reference library itself has no multi-table entry point).  A plan is
 * built once for a fixed set of device pointers: the tables are grouped by
 * kernel variant and every group becomes ONE launch whose grid covers all bags
 * of all its tables.  Launching the plan again pools whatever the index,
 * offset and weight arrays hold by then.
 *
 * One fbgemm_b200_table_call per table: the arguments of
 * fbgemm_b200_spmdm_launch (offsets flavour only).  With num_peers > 0 the
 * pooled rows go to peer_out as in fbgemm_b200_spmdm_launch_sharded (`out` is
 * ignored, dense tables only).  All tables report into status slot `slot`.
 */
typedef struct fbgemm_b200_table_call {
  fbgemm_b200_spmdm_config cfg;
  int64_t output_size;
  int64_t index_size;
  int64_t data_size;
  const void* input;
  const void* indices;
  const void* offsets;
  const float* weights;                    /* NULL unless cfg.has_weight */
  void* out;
  const int32_t* compressed_indices_table; /* NULL = dense table */
  void* const* peer_out;                   /* num_peers pointers, or NULL */
} fbgemm_b200_table_call;

typedef struct fbgemm_b200_multi_plan fbgemm_b200_multi_plan;

FBGEMM_B200_API int fbgemm_b200_multi_plan_create(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_table_call* calls,
    int32_t num_tables,
    int32_t num_peers,
    int64_t bags_per_peer,
    int slot,
    fbgemm_b200_multi_plan** plan);
/* Enqueues the plan's launches on `stream` (no allocation, no copy: it can be
 * captured into a CUDA graph).  Returns 0 or a negative code. */
FBGEMM_B200_API int fbgemm_b200_multi_plan_launch(fbgemm_b200_multi_plan* plan, void* stream);
/* Kernel launches one fbgemm_b200_multi_plan_launch enqueues. */
FBGEMM_B200_API int fbgemm_b200_multi_plan_num_launches(const fbgemm_b200_multi_plan* plan);
FBGEMM_B200_API void fbgemm_b200_multi_plan_destroy(fbgemm_b200_multi_plan* plan);

/* Waits for `stream`, reads status slot `slot` into info[4] = {code, bag,
 * position in indices, offending value (low 32 bits)} and clears the slot.
 * Returns 1 if the code is 0 (functor result true), 0 otherwise, negative on
 * a CUDA error.  `info` may be NULL. */
FBGEMM_B200_API int fbgemm_b200_status_read(
    fbgemm_b200_ctx* ctx,
    int slot,
    void* stream,
    int32_t* info);

/* fbgemm_b200_spmdm_launch + fbgemm_b200_status_read on slot 0: the
 * synchronous functor call.  Returns 1 / 0 / negative. */
FBGEMM_B200_API int fbgemm_b200_spmdm(
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
    void* stream);

/*
 * The lengths flavour of the lookup (cfg->use_offsets == 0) for callers that
 * may not allocate device memory: programs whose own allocator owns the whole
 * device, or whose serving loop forbids cudaMalloc after start-up because an
 * allocation can stall the device or find the pool already taken.  It has no
 * counterpart in the reference (whose functors run on the CPU and need no
 * scratch); arguments and result are those of fbgemm_b200_spmdm without the
 * context, and the pooled rows are bit-equal to that call's.
 *
 * The scratch that holds the scanned offsets and the status record is a
 * fixed array in the library's device image (about 8.4 MB on every GPU that
 * loads the library, held until the process exits) instead of a buffer from
 * cudaMalloc; no allocating call is made, directly or indirectly.
 *   - output_size may not exceed FBGEMM_B200_NOALLOC_MAX_BAGS; larger calls
 *     are refused with FBGEMM_B200_EINVAL and an explanatory error text.
 *   - The first call on a device looks up the array's device address (with
 *     that device current); make that first call before any stream capture.
 *   - All calls on a GPU share the one array, which keeps the previous
 *     call's contents (the entry point clears what has to start at zero):
 *     calls that overlap on the GPU race.  Run them one after another, e.g.
 *     on one stream.
 *   - The call synchronises `stream` to read the status record.
 * All pointers are device pointers on the current device.
 * Returns 1 / 0 (the functor's bool) or a negative error code.
 */
#define FBGEMM_B200_NOALLOC_MAX_BAGS (1 << 20)
FBGEMM_B200_API int fbgemm_b200_spmdm_lengths_noalloc(
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
    void* stream);

/* ---- index remapping ahead of the lookup --------------------------------- */

/*
 * fbgemm::compressed_indices_remap<IndexType> (include/fbgemm/FbgemmEmbedding.h:393-401,
 * src/EmbeddingSpMDM.cc:1714-1770; scalar form src/RefImplementations.cc:2308-2333):
 * the other way to use a pruned table - rewrite (indices, offsets, weights)
 * so that pruned rows disappear and the rest address the compressed table,
 * then run a plain lookup.  Device pointers; offsets share the index type, as
 * in the reference.  Two arguments the reference does not have, because a
 * GPU must not follow a wild index and sizes its grid on the host:
 * index_size = entries in `indices` (at least offsets[offsets_len-1]) and
 * mapping_size = entries in the map.  out_indices / out_weights need room for
 * index_size entries, out_offsets for offsets_len.  Waits for `stream`.
 * Returns 1, or 0 if an index lay outside the map (that entry is dropped),
 * or a negative code.  One remap at a time per context.
 */
FBGEMM_B200_API int fbgemm_b200_compressed_indices_remap(
    fbgemm_b200_ctx* ctx,
    int32_t offsets_len,
    const void* indices,
    int32_t index_bytes,
    int64_t index_size,
    const int32_t* compressed_indices_mapping,
    int64_t mapping_size,
    const void* offsets,
    const float* weights, /* NULL: no per-sample weights */
    void* out_indices,
    void* out_offsets,
    float* out_weights,
    void* stream);

/*
 * Index remapping of table-batched pruned tables (the step a table-batched
 * caller runs before the lookup when rows were pruned):
 *   pruned_hashmap_lookup_{un}weighted_cpu and pruned_array_lookup_cpu,
 *   fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:524-601, :605-659
 *   (GPU forms: embedding_forward_quantized_split_lookup.cu:20-160).
 * `offsets` holds T*B+1 entries, table after table; position k of `indices`
 * belongs to the table t with offsets[t*B] <= k < offsets[(t+1)*B].
 *
 * hashmap: hash_table is [sum of capacities][2] integers of hash_bytes (4 or
 * 8) each, (sparse index, dense index), sparse index -1 = empty slot; table t
 * owns slots [hash_table_offsets[t], hash_table_offsets[t+1]).  The index is
 * hashed in its own width with the MurmurHash3 finaliser (:102-120), reduced
 * modulo the capacity and probed linearly; dense_indices[k] is the dense
 * index, or -1 when an empty slot is met first (a pruned row).  A table of
 * capacity 0 is not pruned: its indices are copied.  Unlike the reference,
 * whose probe loop has no end on a full table that lacks the key, a probe
 * sequence stops after `capacity` slots with -1.
 *
 * array: remappings is one array of remap_bytes-wide integers; table t owns
 * [remappings_offsets[t], remappings_offsets[t+1]) and dense_indices[k] =
 * remappings[start_t + indices[k]]; capacity 0 copies the indices.  An index
 * outside its table's array (the reference reads out of bounds) gives -1 and
 * a return value of 0.
 *
 * All pointers are device pointers; hash_table_offsets / remappings_offsets
 * are int64[T+1].  index_size = entries in `indices` and `dense_indices`;
 * positions the offsets do not cover are left untouched.  Asynchronous on
 * `stream`; a bad index shows in status slot `slot`.  Returns 0 or a negative
 * code.
 */
FBGEMM_B200_API int fbgemm_b200_pruned_hashmap_lookup(
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
    void* stream);

FBGEMM_B200_API int fbgemm_b200_pruned_array_lookup(
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
    void* stream);

/*
 * pruned_hashmap_insert on the device (the reference has no such form: its
 * GPU module fills the table on the host).  Device pointers; hash_table must
 * start as -1 everywhere.  Every position whose dense index is not -1 claims
 * the first free slot of its probe sequence with a compare-and-swap, so the
 * table may differ byte for byte from the one the host insert builds while
 * every lookup answers the same.  Asynchronous on `stream`; a table without a
 * free slot shows as FBGEMM_B200_STATUS_TABLE_FULL in status slot `slot`.
 * Returns 0 or a negative code.
 */
FBGEMM_B200_API int fbgemm_b200_pruned_hashmap_insert(
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
    void* stream);

/*
 * pruned_hashmap_insert_{un}weighted_cpu (same file, :124-204): fills the
 * hash table at model-load time.  HOST pointers and host code, as in the
 * reference (whose GPU module also inserts on the CPU and then moves the
 * table); positions whose dense index is -1 are not inserted.  Returns 1, or
 * 0 if a table was full (the reference would not return), or a negative code.
 */
FBGEMM_B200_API int fbgemm_b200_pruned_hashmap_insert_host(
    int32_t T,
    int32_t B,
    const void* indices,
    const void* dense_indices,
    const void* offsets,
    int32_t index_bytes,
    void* hash_table,
    int32_t hash_bytes,
    const int64_t* hash_table_offsets);

/* ---- sequence ("nobag") lookup over the tables of a table-batched call --- */

#define FBGEMM_B200_OUT_INT4 4 /* sequence lookup only: packed 4-bit rows copied whole */

/* One table of the call; an array of T of these lives in DEVICE memory.  type
 * is the SparseType code of fbgemm_gpu/include/fbgemm_gpu/embedding_common.h:20-32
 * (FP32 0, FP16 1, INT8 2, INT4 3, INT2 4, FP8 6). */
typedef struct fbgemm_b200_sequence_table {
  int64_t weight_offset; /* byte offset of the table's first row in dev_weights */
  int64_t rows;
  int32_t row_bytes;     /* padded row size (nbit::padded_row_size_in_bytes)   */
  int32_t type;
} fbgemm_b200_sequence_table;

/*
 * int_nbit_split_embedding_nobag_codegen_forward_unweighted_cpu
 * (fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:206-520,
 * the `nobag` branch): no pooling, one output row per index.  Position k of
 * `indices` belongs to the table t with offsets[t*B] <= k < offsets[(t+1)*B]
 * (offsets: T*B+1 entries of the index type); output row k starts at byte
 * k * out_row_bytes of `out` and holds
 *   F32/F16/BF16: the D dequantized columns of row indices[k] - what the
 *                 pooled kernel of the table's type gives for a bag of that one
 *                 row without weights (:391-395, :421-473); with scale and bias
 *                 first, index -1 is a pruned row and gives zeros;
 *   U8:           min(out_row_bytes, row_bytes) bytes of the row (8-bit tables;
 *                 the reference's out_row_bytes is D + 4);
 *   INT4:         the bytes of the row (4-bit tables; the caller makes
 *                 out_row_bytes = row_bytes = (D + 8 + 1) / 2; never more than
 *                 out_row_bytes are written).
 * All tables share D.  Everything is a device pointer; rows of positions that
 * no table covers, or whose index is out of range (reported in status slot
 * `slot`), are left as they were.  Asynchronous on `stream`; returns 0 or a
 * negative code.
 */
FBGEMM_B200_API int fbgemm_b200_sequence_lookup(
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
    void* stream);

/* ---- pooled lookup, host pointers -------------------------------------- */

/*
 * The reference functor is called with host pointers.  A caller that keeps
 * its buffers in host memory registers each table once (the table then lives
 * in HBM) and afterwards passes the same host address as `input`; indices,
 * offsets/lengths, weights and the output travel through pinned staging
 * buffers on every call.
 */

/* Copy `bytes` of a fused-row table (or of a compressed_indices_table) to the
 * device and remember it under its host address.  Registering the same
 * address again replaces the copy. */
FBGEMM_B200_API int fbgemm_b200_table_register(
    fbgemm_b200_ctx* ctx,
    const void* host_ptr,
    size_t bytes);
FBGEMM_B200_API int fbgemm_b200_table_unregister(fbgemm_b200_ctx* ctx, const void* host_ptr);
/* Device address of a registered table, NULL if unknown. */
FBGEMM_B200_API const void* fbgemm_b200_table_device_ptr(fbgemm_b200_ctx* ctx, const void* host_ptr);

/* Asynchronous host-pointer functor call on pipeline lane `lane`
 * (0 <= lane < FBGEMM_B200_HOST_LANES): host->device copies of indices,
 * offsets/lengths and weights, the lookup kernel, and the device->host copy
 * of the output rows into `out` are enqueued on the lane's own stream.
 * `input` (and compressed_indices_table, if any) must have been registered;
 * an unregistered table is registered on the spot using
 * data_size * input_stride bytes (for the compressed_indices_table:
 * data_size * 4 bytes).  The host buffers must stay valid until
 * fbgemm_b200_spmdm_host_wait(lane) returns.  Returns 0 or a negative code
 * (FBGEMM_B200_EBUSY if the lane has un-waited work). */
FBGEMM_B200_API int fbgemm_b200_spmdm_host_submit(
    fbgemm_b200_ctx* ctx,
    int lane,
    const fbgemm_b200_spmdm_config* cfg,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const void* input,
    const void* indices,
    const void* offsets_or_lengths,
    const float* weights,
    void* out,
    const int32_t* compressed_indices_table);

/* Wait for lane `lane`; returns the functor result 1 / 0, or negative. */
FBGEMM_B200_API int fbgemm_b200_spmdm_host_wait(fbgemm_b200_ctx* ctx, int lane);

/* submit on lane 0 + wait: the synchronous functor call with host pointers. */
FBGEMM_B200_API int fbgemm_b200_spmdm_host(
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
    const int32_t* compressed_indices_table);

/* ---- kernel choice (tests and comparisons) ---------------------------------- */

/* Quantized rows are pooled by one of two kernels with identical results: the
 * register-resident one (rows whose address, pitch and width allow 4- or
 * 8-byte loads) and a generic one that stages rows in shared memory and takes
 * every shape.  FBGEMM_B200_KERNEL_AUTO picks per call; _GENERIC sends every
 * call to the generic kernel, so that both can be compared on the same
 * inputs.  Process-wide.  Returns the previous choice, or a negative code.
 * No counterpart in the reference (whose ISA dispatch is by CPU feature,
 * src/EmbeddingSpMDM.cc:1012-1130). */
#define FBGEMM_B200_KERNEL_AUTO 0
#define FBGEMM_B200_KERNEL_GENERIC 1
FBGEMM_B200_API int fbgemm_b200_set_kernel_choice(int choice);

/* ---- ordering between the GPUs of a sharded lookup ---------------------- */

/*
 * fbgemm_b200_spmdm_launch_sharded stores pooled rows into peer GPUs' memory;
 * these two calls tell a GPU, on the device and per step, when it may read or
 * overwrite such a buffer.  A counter is an 8-byte word in some GPU's memory
 * (peer-mapped where another GPU writes it), starting at 0 and only growing.
 * The reference orders its peer copies with events between the streams of one
 * process (fbgemm_gpu/src/merge_pooled_embedding_ops/merge_pooled_embedding_ops_gpu.cpp:223-230,454-461);
 * with one process per GPU these counters take that role.
 *
 * fbgemm_b200_peer_signal enqueues, after everything already on `stream`, one
 * small kernel that writes `value` to the num_flags words flags[i] (release
 * stores at system scope: the stores of earlier kernels on the stream are
 * visible to whoever then reads the value).
 * fbgemm_b200_peer_wait enqueues one small kernel that returns when each of
 * the num_flags consecutive words at `flags` (this GPU's memory) has reached
 * `value`, or after timeout_us (1 us .. 60 s); in that case it records
 * {FBGEMM_B200_STATUS_PEER_TIMEOUT, word that lagged, its value, `value`} in
 * status slot `slot`, later work on the stream still runs and the context stays
 * usable - read the slot before trusting the buffer.  Plain loads and stores,
 * no multicast.  Both return 0 when enqueued or a negative code.
 */
FBGEMM_B200_API int fbgemm_b200_peer_signal(
    fbgemm_b200_ctx* ctx,
    void* const* flags,
    int num_flags,
    uint64_t value,
    void* stream);
FBGEMM_B200_API int fbgemm_b200_peer_wait(
    fbgemm_b200_ctx* ctx,
    const void* flags,
    int num_flags,
    uint64_t value,
    uint64_t timeout_us,
    int slot,
    void* stream);

/*
 * Buffers for the two calls above and for the peer_out of a sharded lookup,
 * for callers with one process per GPU and no framework to exchange addresses
 * for them: _alloc gives `bytes` of zeroed device memory on the context's
 * device and a 64-byte handle; the handle travels to the peer processes of the
 * same box over any channel (a file, a socket, MPI), where _open maps the
 * buffer (the address it returns is valid on that process's device; loads and
 * stores through it cross NVLink).  _close unmaps, _free releases the original
 * (after the peers have closed it).  CUDA IPC underneath; these calls allocate
 * and synchronise - set-up time only.  No counterpart in the reference, whose
 * multi-GPU operators live in one process.  Return 0 or a negative code.
 */
#define FBGEMM_B200_IPC_HANDLE_BYTES 64
FBGEMM_B200_API int fbgemm_b200_peer_buffer_alloc(
    fbgemm_b200_ctx* ctx,
    size_t bytes,
    void** ptr,
    unsigned char* handle /* [FBGEMM_B200_IPC_HANDLE_BYTES] */);
FBGEMM_B200_API int fbgemm_b200_peer_buffer_open(
    fbgemm_b200_ctx* ctx,
    const unsigned char* handle,
    void** ptr);
FBGEMM_B200_API int fbgemm_b200_peer_buffer_close(fbgemm_b200_ctx* ctx, void* ptr);
FBGEMM_B200_API int fbgemm_b200_peer_buffer_free(fbgemm_b200_ctx* ctx, void* ptr);

/* The counters of one rank of a table-wise sharded job, as
 * fbgemm_b200_multi_host_create takes them.  "ready": rank r writes
 * ready_flags[g] (a word in GPU g's memory, slot r of g's ready_local array)
 * once its rows for g's slice are stored; "ack": rank g writes ack_flags[r]
 * (slot g of r's ack_local array) once it has consumed its slice. */
typedef struct fbgemm_b200_peer_sync {
  int32_t num_peers;        /* G, the same as the lookups' num_peers */
  void* const* ready_flags; /* [G] words this rank writes, one per peer */
  const void* ready_local;  /* G consecutive words in this GPU's memory */
  void* const* ack_flags;   /* [G] words this rank writes, one per peer */
  const void* ack_local;    /* G consecutive words in this GPU's memory */
  uint64_t timeout_us;      /* per wait; 0 = 2 s */
} fbgemm_b200_peer_sync;

/* ---- several tables per call, host pointers ------------------------------ */

/*
 * The reference's multi-table caller on host tensors
 * (fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_template.cpp:208-280,343-473:
 * host indices/offsets/weights of T tables in, output[B, total_D] out) with the
 * tables resident in HBM.  A handle is built once per set of tables and output
 * buffer; each step
 *   1. copies every table's indices, offsets and weights from the caller's
 *      host arrays into the handle's device staging block,
 *   2. runs one lookup per table (offsets flavour), the pooled rows going to
 *      calls[t].out - or, with num_peers > 0, to calls[t].peer_out as in
 *      fbgemm_b200_spmdm_launch_sharded,
 *   3. with `sync`: publishes this rank's "ready" counters and waits for the
 *      peers' (fbgemm_b200_peer_signal / _wait),
 *   4. copies out_bytes from out_dev (the device buffer the rows of THIS rank's
 *      bags land in) to the caller's host buffer,
 *   5. with `sync`: publishes the "ack" counters; the next step on this handle
 *      first waits for all peers' acks, so no buffer is overwritten while a
 *      peer still reads it.
 * calls[t]: cfg, output_size, data_size, input (DEVICE pointer of the resident
 * table, e.g. fbgemm_b200_table_device_ptr), compressed_indices_table (device),
 * out / peer_out; its indices/offsets/weights/index_size fields are ignored.
 * index_capacity[t] bounds the indices a step may bring for table t.  Every
 * rank of a sharded job must submit the same number of steps on corresponding
 * handles.  submit enqueues on the handle's own stream and returns; wait
 * blocks until the rows are in the host buffer and returns 1 (every table's
 * functor result true), 0 (a lookup or a counter wait failed: info[4] as in
 * fbgemm_b200_status_read) or a negative code.  Pinned host arrays keep the
 * copies asynchronous.  Arrays that touch or overlap in host memory (per-table
 * views of one indices, one offsets, one weights array) go up as ONE copy; the
 * number of copies is what bounds a step beside another handle's download.
 * create allocates (staging, streams); submit and wait allocate nothing.
 * fbgemm_b200_multi_host_step_device: the same step for a caller whose index,
 * offset and weight arrays are already on the device: no upload, no download,
 * everything enqueued on the CALLER's `stream` (the handle's side streams fork
 * from it and join it): wait for the peers' acks, the lookups, publish "ready"
 * and wait for the peers'; when `stream` gets past it, out_dev holds this rank's
 * rows.  Returns the step number (> 0) or a negative code; errors of the lookups
 * and counter waits go to status slot `slot` (fbgemm_b200_status_read).  With
 * `release` != 0 the "ack" counters are published right away (the caller has no
 * use for the rows, e.g. a benchmark); otherwise call
 * fbgemm_b200_multi_host_release(handle, step, stream) after the work that
 * reads out_dev has been enqueued on `stream`.  One call from the host per
 * step instead of one per table and counter: with 8 tables per rank the host
 * needs 169-186 us per step through per-table calls from Python, as long as
 * the GPU needs for the lookups.  A handle is used either with host arrays
 * (submit / wait) or with device arrays, not both.
 * fbgemm_b200_multi_host_last_step_ms: device time of the three phases of the
 * step that the last wait returned - ms[0] from the step's first operation
 * (with `sync`: the wait for the peers' acks) to the end of the uploads, ms[1]
 * the lookups (with `sync`: and the ready counters), ms[2] the download.  The
 * phases of two handles overlap; each handle reports its own.
 */
typedef struct fbgemm_b200_multi_host fbgemm_b200_multi_host;

FBGEMM_B200_API int fbgemm_b200_multi_host_create(
    fbgemm_b200_ctx* ctx,
    const fbgemm_b200_table_call* calls,
    int32_t num_tables,
    const int64_t* index_capacity,
    int32_t num_peers,
    int64_t bags_per_peer,
    void* out_dev,
    size_t out_bytes,
    const fbgemm_b200_peer_sync* sync, /* NULL: no peers to wait for */
    int slot,
    fbgemm_b200_multi_host** handle);
FBGEMM_B200_API int fbgemm_b200_multi_host_submit(
    fbgemm_b200_multi_host* handle,
    const void* const* indices,   /* [T] host arrays */
    const void* const* offsets,   /* [T] host arrays of output_size + 1 */
    const float* const* weights,  /* [T] host arrays, or NULL when no table is weighted */
    const int64_t* index_sizes,   /* [T] */
    void* out_host);
FBGEMM_B200_API int fbgemm_b200_multi_host_wait(fbgemm_b200_multi_host* handle, int32_t* info);
FBGEMM_B200_API int64_t fbgemm_b200_multi_host_step_device(
    fbgemm_b200_multi_host* handle,
    const void* const* indices,   /* [T] device arrays */
    const void* const* offsets,   /* [T] device arrays of output_size + 1 */
    const float* const* weights,  /* [T] device arrays, or NULL when no table is weighted */
    const int64_t* index_sizes,   /* [T] */
    int release,
    void* stream);
FBGEMM_B200_API int fbgemm_b200_multi_host_release(fbgemm_b200_multi_host* handle, int64_t step, void* stream);
FBGEMM_B200_API int fbgemm_b200_multi_host_last_step_ms(fbgemm_b200_multi_host* handle, float* ms /* [3] */);
FBGEMM_B200_API void fbgemm_b200_multi_host_destroy(fbgemm_b200_multi_host* handle);

/* ---- row-wise quantizers, device pointers ------------------------------ */

/* fbgemm::FloatOrHalfToFused8BitRowwiseQuantizedSBFloat<float>
 * (include/fbgemm/QuantUtils.h:312; arithmetic of src/QuantUtils.cc:677-718):
 * fp32 [rows x cols] -> uint8 [rows x (cols + 8)].  Enqueued on `stream`. */
FBGEMM_B200_API int fbgemm_b200_float_to_fused_8bit_rowwise(
    const float* input,
    int64_t rows,
    int32_t cols,
    uint8_t* output,
    void* stream);

/* fbgemm::FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf<float>
 * (include/fbgemm/QuantUtils.h:277; arithmetic of src/QuantUtils.cc:534-611):
 * fp32 [rows x cols] -> uint8 [rows x (ceil(cols / (8/bit_rate)) + 4)].
 * bit_rate 2, 4 or 8; cols must be a multiple of 8/bit_rate, as in the
 * reference (src/QuantUtils.cc:624-627). */
FBGEMM_B200_API int fbgemm_b200_float_to_fused_nbit_rowwise(
    int32_t bit_rate,
    const float* input,
    int64_t rows,
    int32_t cols,
    uint8_t* output,
    void* stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* FBGEMM_B200_EMBEDDING_C_API_H_ */

/*
 * TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.
 *
 * A scalar, single-threaded CPU restatement (plain C) of the arithmetic of
 * FBGEMM's quantized embedding-bag path.  It exists only so that tests can
 * check the CUDA kernels, and so that the benchmark can time a CPU leg; the
 * library itself never links, loads or calls anything in this file.
 *
 * Parity status: PINNED.  This file is checked (a) against the quantizer
 * known-answer vectors of test/QuantUtilsTest.cc:550-667 of the reference,
 * and (b) bit-for-bit against the reference's own scalar functions compiled
 * from the reference tree (see ref_shim.cc / Makefile in this directory) on
 * seeded inputs; the outputs of that comparison are committed as fixtures.
 *
 * Every function names the reference lines it restates (paths are relative to
 * the FBGEMM source tree).
 *
 * Build: gcc -O2 -ffp-contract=off -mfma -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: `acc + bias` followed by fma() must stay two
 * roundings, exactly as in the reference.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__GNUC__)
#define ORACLE_API __attribute__((visibility("default")))
#else
#define ORACLE_API
#endif

/* ------------------------------------------------------------------------- */
/* fp16 <-> fp32, software, round-to-nearest-even.                            */
/* Restates include/fbgemm/FloatConversion.h:211-217 (cpu_float2half_rn) and  */
/* :229-291 (cpu_half2float_ref).                                             */
/* ------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

static inline float bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

ORACLE_API uint16_t oracle_float_to_half_rn(float f) {
  const uint32_t x = f32_bits(f);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t absx = x & 0x7fffffffu;
  if (absx >= 0x7f800000u) { /* inf / nan */
    if (absx > 0x7f800000u) {
      return (uint16_t)(sign | 0x7e00u | ((absx >> 13) & 0x3ffu));
    }
    return (uint16_t)(sign | 0x7c00u);
  }
  if (absx >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (absx < 0x33000001u) { /* <= 2^-25: rounds to zero (tie goes to even=0) */
    return (uint16_t)sign;
  }
  int32_t exp = (int32_t)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7fffffu) | 0x800000u; /* 24-bit significand */
  uint32_t shift;
  uint32_t half_exp;
  if (exp < -14) { /* subnormal half */
    shift = (uint32_t)(13 + (-14 - exp));
    half_exp = 0;
  } else {
    shift = 13;
    half_exp = (uint32_t)(exp + 15);
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) {
    ++q;
  }
  uint32_t out;
  if (half_exp == 0) {
    out = q; /* a carry into bit 10 lands on the smallest normal: correct */
  } else {
    out = ((half_exp - 1) << 10) + q; /* q carries the implicit 1 (bit 10) */
  }
  return (uint16_t)(sign | out);
}

ORACLE_API float oracle_half_to_float(uint16_t h) {
  const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = (uint32_t)(h & 0x3ffu) << 13;
  if (exp == 0x1fu) {
    if (man) {
      return bits_f32(0x7fffffffu); /* FloatConversion.h:262-266 */
    }
    return bits_f32(sign | 0x7f800000u);
  }
  if (exp == 0) {
    if (man == 0) {
      return bits_f32(sign);
    }
    exp = 127 - 15 + 1;
    uint32_t msb;
    do {
      msb = man & 0x400000u;
      man <<= 1;
      --exp;
    } while (!msb);
    man &= 0x7fffffu;
  } else {
    exp += 127 - 15;
  }
  return bits_f32(sign | (exp << 23) | man);
}

/* ------------------------------------------------------------------------- */
/* Index / offset accessors: the reference is templated on int32/int64; the  */
/* oracle takes the element width in bytes.                                   */
/* ------------------------------------------------------------------------- */

static inline int64_t load_int(const void* p, int64_t i, int width) {
  return width == 8 ? ((const int64_t*)p)[i] : (int64_t)((const int32_t*)p)[i];
}

static inline void store_out(void* out, int64_t i, float v, int out_is_half) {
  if (out_is_half) {
    ((uint16_t*)out)[i] = oracle_float_to_half_rn(v);
  } else {
    ((float*)out)[i] = v;
  }
}

/* ------------------------------------------------------------------------- */
/* Pooled lookup, 8-bit rows with trailing fp32 scale, bias.                  */
/* Restates src/RefImplementations.cc:1196-1346 (EmbeddingSpMDM_ref, the      */
/* uint8_t / scale_bias_last / bag branch).  Returns 1 for true, 0 for false. */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_embedding_spmdm_8bit(
    int64_t block_size,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const uint8_t* input,
    const void* indices,
    int index_bytes,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights, /* nullable */
    int normalize_by_lengths,
    void* out,
    int out_is_half,
    int is_weight_positional,
    int use_offsets,
    int64_t output_stride, /* -1: block_size */
    int64_t input_stride /* -1: block_size + 8 */) {
  if (output_stride == -1) {
    output_stride = block_size; /* RefImplementations.cc:1217-1219 */
  }
  if (input_stride == -1) {
    input_stride = block_size + 2 * (int64_t)sizeof(float); /* :1226-1232 */
  }
  float* buf = (float*)malloc(sizeof(float) * (size_t)(block_size > 0 ? block_size : 1));
  int64_t current = 0;
  int64_t out_base = 0;
  int ok = 1;
  for (int64_t m = 0; m < output_size; ++m) {
    memset(buf, 0, sizeof(float) * (size_t)block_size);
    /* `int len` in the reference: the difference is narrowed to 32 bits. */
    const int len = use_offsets
        ? (int)(load_int(offsets_or_lengths, m + 1, offset_bytes) -
                load_int(offsets_or_lengths, m, offset_bytes))
        : (int)load_int(offsets_or_lengths, m, offset_bytes);
    if (current + len > index_size) { /* :1294-1296 */
      ok = 0;
      goto done;
    }
    for (int i = 0; i < len; ++i, ++current) {
      const int64_t idx = load_int(indices, current, index_bytes);
      if (idx < 0 || idx >= data_size) { /* :1304-1306 */
        ok = 0;
        goto done;
      }
      const uint8_t* row = input + input_stride * idx;
      float sb[2];
      memcpy(sb, row + block_size, sizeof(sb)); /* :1308-1309 */
      float weight = 1.0f;
      if (weights) {
        weight = weights[is_weight_positional ? i : current]; /* :1311-1314 */
      }
      const float scale = weight * sb[0]; /* :1316-1318 */
      const float bias = weight * sb[1];
      for (int64_t j = 0; j < block_size; ++j) {
        /* :1326-1333: fma(scale, q, buf + bias) - two roundings. */
        const float t = buf[j] + bias;
        buf[j] = fmaf(scale, (float)row[j], t);
      }
    }
    if (normalize_by_lengths && len) { /* :1335-1340 */
      const float inv = 1.f / (float)len;
      for (int64_t j = 0; j < block_size; ++j) {
        buf[j] *= inv;
      }
    }
    for (int64_t j = 0; j < block_size; ++j) { /* :1341-1343 */
      store_out(out, out_base + j, buf[j], out_is_half);
    }
    out_base += output_stride;
  }
  ok = (current == index_size); /* :1346 */
done:
  free(buf);
  return ok;
}

/* ------------------------------------------------------------------------- */
/* Pooled lookup, 4-bit / 2-bit rows with trailing fp16 scale, bias.          */
/* Restates src/RefImplementations.cc:1427-1541 (EmbeddingSpMDMNBit_ref,      */
/* scale_bias_last, bag branch).                                              */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_embedding_spmdm_nbit(
    int bit_rate,
    int64_t block_size,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const uint8_t* input,
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
    int64_t output_stride,
    int64_t input_stride) {
  if (bit_rate != 2 && bit_rate != 4) {
    return 0;
  }
  const int epb = 8 / bit_rate; /* :1452 */
  const int64_t data_bytes = (block_size + epb - 1) / epb;
  if (output_stride == -1) {
    output_stride = block_size;
  }
  if (input_stride == -1) {
    input_stride = data_bytes + 2 * (int64_t)sizeof(uint16_t); /* :1460-1465 */
  }
  float* buf = (float*)malloc(sizeof(float) * (size_t)(block_size > 0 ? block_size : 1));
  int64_t current = 0;
  int64_t out_base = 0;
  int ok = 1;
  const unsigned mask = (1u << bit_rate) - 1u;
  for (int64_t m = 0; m < output_size; ++m) {
    memset(buf, 0, sizeof(float) * (size_t)block_size);
    const int len = use_offsets
        ? (int)(load_int(offsets_or_lengths, m + 1, offset_bytes) -
                load_int(offsets_or_lengths, m, offset_bytes))
        : (int)load_int(offsets_or_lengths, m, offset_bytes);
    if (current + len > index_size) { /* :1492-1494 */
      ok = 0;
      goto done;
    }
    for (int i = 0; i < len; ++i, ++current) {
      const int64_t idx = load_int(indices, current, index_bytes);
      if (idx < 0 || idx >= data_size) { /* :1502-1504 */
        ok = 0;
        goto done;
      }
      const uint8_t* row = input + input_stride * idx;
      uint16_t sb[2];
      memcpy(sb, row + data_bytes, sizeof(sb)); /* :1506-1510 */
      float weight = 1.0f;
      if (weights) {
        weight = weights[is_weight_positional ? i : current];
      }
      const float scale = weight * oracle_half_to_float(sb[0]); /* :1516 */
      const float bias = weight * oracle_half_to_float(sb[1]); /* :1517 */
      for (int64_t j = 0; j < block_size; ++j) {
        /* :1519-1526: element j sits in byte j/epb at bit (j%epb)*bit_rate. */
        unsigned q = row[j / epb];
        q >>= (unsigned)(j % epb) * (unsigned)bit_rate;
        q &= mask;
        const float t = buf[j] + bias;
        buf[j] = fmaf(scale, (float)q, t);
      }
    }
    if (normalize_by_lengths && len) {
      const float inv = 1.f / (float)len;
      for (int64_t j = 0; j < block_size; ++j) {
        buf[j] *= inv;
      }
    }
    for (int64_t j = 0; j < block_size; ++j) {
      store_out(out, out_base + j, buf[j], out_is_half);
    }
    out_base += output_stride;
  }
  ok = (current == index_size);
done:
  free(buf);
  return ok;
}

/* ------------------------------------------------------------------------- */
/* The same two lookups with the generators' remaining options:               */
/*  - scale_bias_last = 0: the row layout of table-batched embeddings - fp16  */
/*    scale and bias at the START of the row (for 8-bit rows too), payload    */
/*    after them, and an index of -1 is a pruned row: skipped, but it still   */
/*    consumes its index / weight slot (RefImplementations.cc:1223-1229,      */
/*    :1299-1303, :1316-1333 for 8-bit; :1496-1501, :1506-1523 for N-bit);    */
/*  - out_kind 2: bf16 output, (bits + 0x8000) >> 16 (cpu_float2bfloat16,     */
/*    include/fbgemm/FloatConversion.h:312-315), with 0 = fp32, 1 = fp16;     */
/*  - no_bag = 1 (8-bit rows only): output row m is the dequantized row       */
/*    indices[m] times weights[m]; no offsets, no normalisation, and no -1    */
/*    skipping (:1235-1288).                                                  */
/* ------------------------------------------------------------------------- */
static inline void store_out_kind(void* out, int64_t i, float v, int out_kind) {
  if (out_kind == 2) {
    uint32_t b;
    memcpy(&b, &v, sizeof(b));
    ((uint16_t*)out)[i] = (uint16_t)((b + (1u << 15)) >> 16);
  } else {
    store_out(out, i, v, out_kind == 1);
  }
}

ORACLE_API int oracle_embedding_spmdm_ex(
    int bit_rate, /* 8, 4 or 2 */
    int64_t block_size,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
    const uint8_t* input,
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
    int64_t output_stride,
    int64_t input_stride,
    int scale_bias_last,
    int no_bag) {
  if (bit_rate != 8 && bit_rate != 4 && bit_rate != 2) {
    return 0;
  }
  const int epb = 8 / bit_rate;
  const int64_t data_bytes = (block_size + epb - 1) / epb;
  const int half_sb = bit_rate != 8 || !scale_bias_last;
  const int64_t sb_bytes = half_sb ? 4 : 8;
  const int64_t data_at = scale_bias_last ? 0 : sb_bytes;
  const int64_t sb_at = scale_bias_last ? data_bytes : 0;
  const unsigned mask = (1u << bit_rate) - 1u;
  if (output_stride == -1) {
    output_stride = block_size;
  }
  if (input_stride == -1) {
    input_stride = data_bytes + sb_bytes;
  }
  if (no_bag && bit_rate != 8) {
    return 0; /* N-bit no_bag is an int4 -> int4 row copy, not restated here */
  }
  float* buf = (float*)malloc(sizeof(float) * (size_t)(block_size > 0 ? block_size : 1));
  int64_t current = 0;
  int64_t out_base = 0;
  int ok = 1;
  for (int64_t m = 0; m < output_size; ++m) {
    memset(buf, 0, sizeof(float) * (size_t)block_size);
    int len = 1;
    if (!no_bag) {
      len = use_offsets
          ? (int)(load_int(offsets_or_lengths, m + 1, offset_bytes) - load_int(offsets_or_lengths, m, offset_bytes))
          : (int)load_int(offsets_or_lengths, m, offset_bytes);
      if (current + len > index_size) {
        ok = 0;
        goto done;
      }
    }
    for (int i = 0; i < len; ++i, ++current) {
      const int64_t idx = load_int(indices, current, index_bytes);
      if (!no_bag && !scale_bias_last && idx == -1) {
        continue; /* pruned row of a table-batched embedding */
      }
      if (idx < 0 || idx >= data_size) {
        ok = 0;
        goto done;
      }
      const uint8_t* row = input + input_stride * idx;
      float s, b;
      if (half_sb) {
        uint16_t sb[2];
        memcpy(sb, row + sb_at, sizeof(sb));
        s = oracle_half_to_float(sb[0]);
        b = oracle_half_to_float(sb[1]);
      } else {
        float sb[2];
        memcpy(sb, row + sb_at, sizeof(sb));
        s = sb[0];
        b = sb[1];
      }
      float weight = 1.0f;
      if (weights) {
        weight = weights[no_bag ? m : (is_weight_positional ? i : current)];
      }
      const float scale = weight * s;
      const float bias = weight * b;
      for (int64_t j = 0; j < block_size; ++j) {
        unsigned q = row[data_at + j / epb];
        q >>= (unsigned)(j % epb) * (unsigned)bit_rate;
        q &= mask;
        const float t = buf[j] + bias;
        buf[j] = fmaf(scale, (float)q, t);
      }
    }
    if (!no_bag && normalize_by_lengths && len) {
      const float inv = 1.f / (float)len;
      for (int64_t j = 0; j < block_size; ++j) {
        buf[j] *= inv;
      }
    }
    for (int64_t j = 0; j < block_size; ++j) {
      store_out_kind(out, out_base + j, buf[j], out_kind);
    }
    out_base += output_stride;
  }
  ok = no_bag ? 1 : (current == index_size);
done:
  free(buf);
  return ok;
}

/* ------------------------------------------------------------------------- */
/* Pooled lookup on tables that are NOT row-wise quantized: fp32, fp16, bf16  */
/* rows (EmbeddingSpMDM_ref<float | float16>, the non-uint8 branch,           */
/* src/RefImplementations.cc:1347-1424) and FP8 rows (EmbeddingSpMDMFP8_ref,  */
/* :1543-1615, conversion Float8ToFloat_ref :184-215).  One rounding per row  */
/* and column: buf[j] = fma(w, float(row[j]), buf[j]).                        */
/* in_kind: 1 fp32, 2 fp16, 3 bf16, 4 fp8.  input_stride counts ELEMENTS, as  */
/* the reference's does.  scale_bias_last = 0 only makes -1 a pruned index    */
/* (not for fp8, whose reference has no such argument).                       */
/* ------------------------------------------------------------------------- */
static float oracle_fp8_to_float(uint8_t v, int exponent_bits, int exponent_bias) {
  const uint32_t sign = ((uint32_t)(v & 0x80)) << 24;
  float f = bits_f32(((uint32_t)(v & 0x7F)) << (24 - (8 - exponent_bits)));
  const float multiplier = bits_f32((uint32_t)(127 + (127 - exponent_bias)) << 23); /* 2^(127-bias) */
  f *= multiplier;
  return bits_f32(f32_bits(f) | sign);
}

ORACLE_API int oracle_embedding_spmdm_plain(
    int in_kind,
    int64_t block_size,
    int64_t output_size,
    int64_t index_size,
    int64_t data_size,
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
    int64_t output_stride,
    int64_t input_stride,
    int scale_bias_last,
    int no_bag,
    int exponent_bits,
    int exponent_bias) {
  if (in_kind < 1 || in_kind > 4 || (no_bag && in_kind == 4)) {
    return 0;
  }
  if (output_stride == -1) {
    output_stride = block_size;
  }
  if (input_stride == -1) {
    input_stride = block_size;
  }
  float* buf = (float*)malloc(sizeof(float) * (size_t)(block_size > 0 ? block_size : 1));
  int64_t current = 0;
  int64_t out_base = 0;
  int ok = 1;
  for (int64_t m = 0; m < output_size; ++m) {
    memset(buf, 0, sizeof(float) * (size_t)block_size);
    int len = 1;
    if (!no_bag) {
      len = use_offsets
          ? (int)(load_int(offsets_or_lengths, m + 1, offset_bytes) - load_int(offsets_or_lengths, m, offset_bytes))
          : (int)load_int(offsets_or_lengths, m, offset_bytes);
      if (current + len > index_size) {
        ok = 0;
        goto done;
      }
    }
    for (int i = 0; i < len; ++i, ++current) {
      const int64_t idx = load_int(indices, current, index_bytes);
      if (!no_bag && in_kind != 4 && !scale_bias_last && idx == -1) {
        continue;
      }
      if (idx < 0 || idx >= data_size) {
        ok = 0;
        goto done;
      }
      float w = 1.f;
      if (weights) {
        w = weights[no_bag ? m : (is_weight_positional ? i : current)];
      }
      for (int64_t j = 0; j < block_size; ++j) {
        const int64_t at = input_stride * idx + j;
        float x;
        if (in_kind == 1) {
          x = ((const float*)input)[at];
        } else if (in_kind == 2) {
          x = oracle_half_to_float(((const uint16_t*)input)[at]);
        } else if (in_kind == 3) {
          x = bits_f32(((uint32_t)((const uint16_t*)input)[at]) << 16);
        } else {
          x = oracle_fp8_to_float(((const uint8_t*)input)[at], exponent_bits, exponent_bias);
        }
        buf[j] = fmaf(w, x, buf[j]);
      }
    }
    if (!no_bag && normalize_by_lengths && len) {
      const float inv = 1.f / (float)len;
      for (int64_t j = 0; j < block_size; ++j) {
        buf[j] *= inv;
      }
    }
    for (int64_t j = 0; j < block_size; ++j) {
      store_out_kind(out, out_base + j, buf[j], out_kind);
    }
    out_base += output_stride;
  }
  ok = no_bag ? 1 : (current == index_size);
done:
  free(buf);
  return ok;
}

/* ------------------------------------------------------------------------- */
/* no_bag with 8-bit output: output row m is a byte copy of table row          */
/* indices[m] - no arithmetic.  bit_rate 8: min(output_stride, input_stride)   */
/* bytes per row, rows output_stride apart (EmbeddingSpMDM_ref<uint8_t, ...,   */
/* uint8_t>, src/RefImplementations.cc:1235-1254).  bit_rate 4: input_stride   */
/* bytes per row, rows input_stride apart (EmbeddingSpMDMNBit_ref, int4 to     */
/* int4 only, :1467-1485; that loop lets idx == data_size through - one row    */
/* past the table - which this restatement refuses like any other index out    */
/* of range).                                                                  */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_embedding_rows_copy(
    int bit_rate,
    int64_t output_size,
    int64_t data_size,
    const uint8_t* input,
    const void* indices,
    int index_bytes,
    uint8_t* out,
    int64_t output_stride,
    int64_t input_stride) {
  if (bit_rate != 8 && bit_rate != 4) {
    return 0;
  }
  const int64_t width = bit_rate == 8 ? (output_stride < input_stride ? output_stride : input_stride) : input_stride;
  const int64_t pitch = bit_rate == 8 ? output_stride : input_stride;
  for (int64_t m = 0; m < output_size; ++m) {
    const int64_t idx = load_int(indices, m, index_bytes);
    if (idx < 0 || idx >= data_size) {
      return 0;
    }
    memcpy(out + m * pitch, input + input_stride * idx, (size_t)width);
  }
  return 1;
}

/* ------------------------------------------------------------------------- */
/* Pruned (row-wise sparse) pooled lookup: indices address an uncompressed    */
/* row space and go through compressed_indices_table; -1 there means the row  */
/* was pruned: it contributes nothing but still consumes its index/weight     */
/* slot and counts towards the bag length.  fp32 output, dense strides.       */
/* bit_rate == 8 restates src/RefImplementations.cc:1617-1688                 */
/* (EmbeddingSpMDMRowWiseSparse_ref<uint8_t>); 4 and 2 restate :1746-1822     */
/* (EmbeddingSpMDMNBitRowWiseSparse_ref).                                     */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_embedding_spmdm_rowwise_sparse(
    int bit_rate,
    int64_t block_size,
    int64_t output_size,
    int64_t index_size,
    int64_t uncompressed_data_size,
    const uint8_t* input,
    const void* indices,
    int index_bytes,
    const int32_t* compressed_indices_table,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    float* out,
    int is_weight_positional,
    int use_offsets) {
  if (bit_rate != 2 && bit_rate != 4 && bit_rate != 8) {
    return 0;
  }
  const int epb = 8 / bit_rate;
  const int64_t data_bytes = (block_size + epb - 1) / epb;
  const int64_t sb_bytes = bit_rate == 8 ? 8 : 4;
  const int64_t fused = data_bytes + sb_bytes; /* :1637-1638 / :1769-1771 */
  const unsigned mask = (1u << bit_rate) - 1u;
  int64_t current = 0;
  for (int64_t m = 0; m < output_size; ++m) {
    memset(out, 0, sizeof(float) * (size_t)block_size); /* accumulates in out */
    const int len = use_offsets
        ? (int)(load_int(offsets_or_lengths, m + 1, offset_bytes) -
                load_int(offsets_or_lengths, m, offset_bytes))
        : (int)load_int(offsets_or_lengths, m, offset_bytes);
    if (current + len > index_size) {
      return 0;
    }
    for (int i = 0; i < len; ++i, ++current) {
      const int64_t uidx = load_int(indices, current, index_bytes);
      if (uidx < 0 || uidx >= uncompressed_data_size) { /* :1782-1784 */
        return 0;
      }
      const int64_t idx = compressed_indices_table[uidx];
      if (idx == -1) { /* :1786-1788: pruned, slot still consumed */
        continue;
      }
      /* the compressed index itself is not range-checked (:1789-1791) */
      const uint8_t* row = input + fused * idx;
      float weight = 1.0f;
      if (weights) {
        weight = weights[is_weight_positional ? i : current];
      }
      float scale, bias;
      if (bit_rate == 8) {
        float sb[2];
        memcpy(sb, row + data_bytes, sizeof(sb));
        scale = weight * sb[0];
        bias = weight * sb[1];
      } else {
        uint16_t sb[2];
        memcpy(sb, row + data_bytes, sizeof(sb));
        scale = weight * oracle_half_to_float(sb[0]);
        bias = weight * oracle_half_to_float(sb[1]);
      }
      for (int64_t j = 0; j < block_size; ++j) {
        unsigned q = row[j / epb];
        q >>= (unsigned)(j % epb) * (unsigned)bit_rate;
        q &= mask;
        const float t = out[j] + bias;
        out[j] = fmaf(scale, (float)q, t);
      }
    }
    if (normalize_by_lengths && len) {
      const float inv = 1.f / (float)len;
      for (int64_t j = 0; j < block_size; ++j) {
        out[j] *= inv;
      }
    }
    out += block_size;
  }
  return current == index_size;
}

/* ------------------------------------------------------------------------- */
/* Row-wise quantizers that produce the fused rows the lookups read.          */
/* ------------------------------------------------------------------------- */

/* Restates src/QuantUtils.cc:677-718                                        */
/* (FloatOrHalfToFused8BitRowwiseQuantizedSBFloatRef<float>).                 */
ORACLE_API void oracle_float_to_fused_8bit_rowwise_sbfloat(
    const float* input,
    int64_t input_rows,
    int input_columns,
    uint8_t* output) {
  const float kEpsilon = 1e-8f;
  if (input_rows == 0 || input_columns == 0) {
    return;
  }
  const int64_t output_columns = (int64_t)input_columns + 8;
  for (int64_t r = 0; r < input_rows; ++r) {
    const float* in = input + r * input_columns;
    uint8_t* o = output + r * output_columns;
    float mn = in[0], mx = in[0];
    for (int c = 1; c < input_columns; ++c) {
      if (in[c] < mn) mn = in[c];
      if (in[c] > mx) mx = in[c];
    }
    const float range = mx - mn;
    const float sb[2] = {range / 255.0f, mn};
    memcpy(o + input_columns, sb, sizeof(sb));
    const float inverse_scale = 255.0f / (range + kEpsilon);
    for (int c = 0; c < input_columns; ++c) {
      o[c] = (uint8_t)lrintf((in[c] - mn) * inverse_scale);
    }
  }
}

/* Restates src/QuantUtils.cc:534-611                                        */
/* (FloatOrHalfToFusedNBitRowwiseQuantizedSBHalfRef<float>); bit_rate may be  */
/* 2, 4 or 8 there.                                                           */
ORACLE_API void oracle_float_to_fused_nbit_rowwise_sbhalf(
    int bit_rate,
    const float* input,
    int64_t input_rows,
    int input_columns,
    uint8_t* output) {
  if (input_rows == 0 || input_columns == 0) {
    return;
  }
  const int epb = 8 / bit_rate;
  const int64_t data_bytes = ((int64_t)input_columns + epb - 1) / epb;
  const int64_t output_columns = data_bytes + 4;
  const int qmax = (1 << bit_rate) - 1;
  for (int64_t r = 0; r < input_rows; ++r) {
    const float* in = input + r * input_columns;
    uint8_t* o = output + r * output_columns;
    float mn = in[0], mx = in[0];
    for (int c = 1; c < input_columns; ++c) {
      if (in[c] < mn) mn = in[c];
      if (in[c] > mx) mx = in[c];
    }
    /* the bias is stored as fp16, so the minimum is rounded first (:572-575) */
    const uint16_t mn_h = oracle_float_to_half_rn(mn);
    mn = oracle_half_to_float(mn_h);
    const float range = mx - mn;
    float scale = range == 0 ? 1.0f : range / (float)qmax;
    const uint16_t scale_h = oracle_float_to_half_rn(scale);
    scale = oracle_half_to_float(scale_h);
    if (scale == 0) { /* :580-584 */
      scale = 1.0f;
    }
    float inverse_scale = 1.0f / scale;
    if (isinf(inverse_scale)) { /* :586-589 */
      scale = 1.0f;
      inverse_scale = 1.0f;
    }
    const uint16_t sb[2] = {oracle_float_to_half_rn(scale), mn_h};
    memcpy(o + data_bytes, sb, sizeof(sb));
    for (int c = 0; c < input_columns; ++c) {
      long q = lrintf((in[c] - mn) * inverse_scale);
      if (q > qmax) q = qmax;
      if (q < 0) q = 0;
      if (c % epb == 0) {
        o[c / epb] = (uint8_t)q;
      } else {
        o[c / epb] |= (uint8_t)(q << ((c % epb) * bit_rate));
      }
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Index remapping for pruned tables (drops pruned entries up front).         */
/* Restates src/RefImplementations.cc:2308-2333 (compressed_indices_remap_ref)*/
/* ------------------------------------------------------------------------- */
ORACLE_API void oracle_compressed_indices_remap(
    int32_t offsets_len,
    const void* indices,
    int index_bytes, /* offsets share the index type in the reference */
    const int32_t* compressed_indices_mapping,
    const void* offsets,
    const float* weights, /* nullable */
    void* out_indices,
    void* out_offsets,
    float* out_weights) {
  const int has_w = weights != NULL;
  int64_t k = 0;
  if (index_bytes == 8) {
    ((int64_t*)out_offsets)[0] = ((const int64_t*)offsets)[0];
  } else {
    ((int32_t*)out_offsets)[0] = ((const int32_t*)offsets)[0];
  }
  for (int32_t i = 1; i < offsets_len; ++i) {
    const int64_t lo = load_int(offsets, i - 1, index_bytes);
    const int64_t hi = load_int(offsets, i, index_bytes);
    for (int64_t j = lo; j < hi; ++j) {
      const int64_t idx = load_int(indices, j, index_bytes);
      const int32_t mapped = compressed_indices_mapping[idx];
      if (mapped != -1) {
        if (index_bytes == 8) {
          ((int64_t*)out_indices)[k] = mapped;
        } else {
          ((int32_t*)out_indices)[k] = mapped;
        }
        if (has_w) {
          out_weights[k] = weights[j];
        }
        ++k;
      }
    }
    if (index_bytes == 8) {
      ((int64_t*)out_offsets)[i] = k;
    } else {
      ((int32_t*)out_offsets)[i] = (int32_t)k;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Index remapping of table-batched pruned tables, before the lookup.         */
/* Restates fbgemm_gpu/codegen/inference/embedding_forward_quantized_cpu_     */
/* template.cpp: pruned_hash_function :102-120 (the MurmurHash3 32- and       */
/* 64-bit finalisers), pruned_hashmap_insert_*_cpu :124-204,                  */
/* pruned_hashmap_lookup_*_cpu :524-601 and pruned_array_lookup_cpu :605-659. */
/*                                                                            */
/* Parity status of THIS block: UNPINNED against reference output.  The       */
/* functions live in a Jinja template over ATen tensors, which cannot be      */
/* compiled from its own sources here, and the reference holds no golden      */
/* vectors for them; they are checked by the property the reference's own     */
/* test uses (fbgemm_gpu/test/tbe/utils/split_embeddings_utils_test.py:       */
/* 476-620: insert, then every inserted index looks up its dense index and    */
/* any other index looks up -1) and by the published MurmurHash3 finalisers.  */
/*                                                                            */
/* One deliberate difference: the reference probes `while (true)`, which      */
/* never ends on a full table that lacks the key; here a probe sequence ends  */
/* after `capacity` slots (lookup: -1; insert: returns 0).                    */
/* ------------------------------------------------------------------------- */

static inline uint32_t pruned_hash32(uint32_t h) {
  h ^= h >> 16;
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  h *= 0xc2b2ae35u;
  h ^= h >> 16;
  return h;
}

static inline uint64_t pruned_hash64(uint64_t k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return k;
}

ORACLE_API uint64_t oracle_pruned_hash(uint64_t key, int index_bytes) {
  return index_bytes == 8 ? pruned_hash64(key) : (uint64_t)pruned_hash32((uint32_t)key);
}

static inline void store_int(void* p, int64_t i, int64_t v, int width) {
  if (width == 8) {
    ((int64_t*)p)[i] = v;
  } else {
    ((int32_t*)p)[i] = (int32_t)v;
  }
}

static inline uint64_t first_slot(int64_t idx, int index_bytes, int64_t capacity) {
  /* the index is hashed in its own width (static_cast<uidx_t>(idx), :176,:573) */
  const uint64_t h = index_bytes == 8 ? pruned_hash64((uint64_t)idx) : (uint64_t)pruned_hash32((uint32_t)idx);
  return h % (uint64_t)capacity;
}

/* hash_table: [sum(capacity)][2] of hash_bytes-wide integers, (-1,-1) = empty. */
ORACLE_API int oracle_pruned_hashmap_insert(
    int64_t T, int64_t B, const void* indices, const void* dense_indices, const void* offsets, int index_bytes,
    void* hash_table, int hash_bytes, const int64_t* hash_table_offsets) {
  int ok = 1;
  for (int64_t t = 0; t < T; ++t) {
    const int64_t table_start = hash_table_offsets[t];
    const int64_t capacity = hash_table_offsets[t + 1] - table_start;
    if (capacity == 0) {
      continue;
    }
    const int64_t lo = load_int(offsets, t * B, index_bytes), hi = load_int(offsets, (t + 1) * B, index_bytes);
    for (int64_t k = lo; k < hi; ++k) {
      const int64_t idx = load_int(indices, k, index_bytes);
      const int64_t dense = load_int(dense_indices, k, index_bytes);
      if (dense == -1) {
        continue; /* a pruned row is not inserted (:171-174) */
      }
      uint64_t slot = first_slot(idx, index_bytes, capacity);
      int64_t probes = 0;
      for (; probes < capacity; ++probes) {
        const int64_t at = table_start + (int64_t)slot;
        const int64_t key = load_int(hash_table, 2 * at, hash_bytes);
        if (key == -1 || key == idx) {
          store_int(hash_table, 2 * at, idx, hash_bytes);
          store_int(hash_table, 2 * at + 1, dense, hash_bytes);
          break;
        }
        slot = (slot + 1) % (uint64_t)capacity;
      }
      if (probes == capacity) {
        ok = 0;
      }
    }
  }
  return ok;
}

ORACLE_API void oracle_pruned_hashmap_lookup(
    int64_t T, int64_t B, const void* indices, const void* offsets, int index_bytes, const void* hash_table,
    int hash_bytes, const int64_t* hash_table_offsets, void* dense_indices) {
  for (int64_t t = 0; t < T; ++t) {
    const int64_t table_start = hash_table_offsets[t];
    const int64_t capacity = hash_table_offsets[t + 1] - table_start;
    const int64_t lo = load_int(offsets, t * B, index_bytes), hi = load_int(offsets, (t + 1) * B, index_bytes);
    for (int64_t k = lo; k < hi; ++k) {
      const int64_t idx = load_int(indices, k, index_bytes);
      if (capacity == 0) {
        store_int(dense_indices, k, idx, index_bytes); /* table without pruning (:565-569) */
        continue;
      }
      uint64_t slot = first_slot(idx, index_bytes, capacity);
      int64_t found = -1;
      for (int64_t probes = 0; probes < capacity; ++probes) {
        const int64_t at = table_start + (int64_t)slot;
        const int64_t key = load_int(hash_table, 2 * at, hash_bytes);
        if (key == -1) {
          break;
        }
        if (key == idx) {
          found = load_int(hash_table, 2 * at + 1, hash_bytes);
          break;
        }
        slot = (slot + 1) % (uint64_t)capacity;
      }
      store_int(dense_indices, k, found, index_bytes);
    }
  }
}

/* Returns 0 if an index falls outside its table's remapping array (the
 * reference reads out of bounds there and leaves it to a bounds checker,
 * split_embeddings_utils_test.py:612-614); such a position gets -1. */
ORACLE_API int oracle_pruned_array_lookup(
    int64_t T, int64_t B, const void* indices, const void* offsets, int index_bytes, const void* remappings,
    int remap_bytes, const int64_t* remappings_offsets, void* dense_indices) {
  int ok = 1;
  for (int64_t t = 0; t < T; ++t) {
    const int64_t start = remappings_offsets[t];
    const int64_t capacity = remappings_offsets[t + 1] - start;
    const int64_t lo = load_int(offsets, t * B, index_bytes), hi = load_int(offsets, (t + 1) * B, index_bytes);
    for (int64_t k = lo; k < hi; ++k) {
      const int64_t idx = load_int(indices, k, index_bytes);
      if (capacity <= 0) {
        store_int(dense_indices, k, idx, index_bytes);
      } else if (idx < 0 || idx >= capacity) {
        ok = 0;
        store_int(dense_indices, k, -1, index_bytes);
      } else {
        store_int(dense_indices, k, load_int(remappings, start + idx, remap_bytes), index_bytes);
      }
    }
  }
  return ok;
}

/* ------------------------------------------------------------------------- */
/* Pruned (row-wise sparse) pooled lookup over a table that is not quantized: */
/* the non-8-bit branch of EmbeddingSpMDMRowWiseSparse_ref,                   */
/* src/RefImplementations.cc:1688-1743.  in_kind 1: float rows; 2: fp16 rows  */
/* (InType float16, and InType uint16_t, which that function also reads as    */
/* fp16, :1723-1726).  Rows are block_size elements apart, fp32 output.       */
/* Pinned bit-for-bit against the compiled reference like the rest.           */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_embedding_spmdm_plain_rowwise_sparse(
    int in_kind,
    int64_t block_size,
    int64_t output_size,
    int64_t index_size,
    int64_t uncompressed_data_size,
    const void* input,
    const void* indices,
    int index_bytes,
    const int32_t* compressed_indices_table,
    const void* offsets_or_lengths,
    int offset_bytes,
    const float* weights,
    int normalize_by_lengths,
    float* out,
    int is_weight_positional,
    int use_offsets) {
  if (in_kind != 1 && in_kind != 2) {
    return 0;
  }
  int64_t current = 0;
  for (int64_t m = 0; m < output_size; ++m) {
    memset(out, 0, sizeof(float) * (size_t)block_size);
    const int len = use_offsets
        ? (int)(load_int(offsets_or_lengths, m + 1, offset_bytes) - load_int(offsets_or_lengths, m, offset_bytes))
        : (int)load_int(offsets_or_lengths, m, offset_bytes);
    if (current + len > index_size) {
      return 0;
    }
    for (int i = 0; i < len; ++i, ++current) {
      const int64_t uidx = load_int(indices, current, index_bytes);
      if (uidx < 0 || uidx >= uncompressed_data_size) { /* :1701-1704 */
        return 0;
      }
      const int64_t idx = compressed_indices_table[uidx];
      if (idx == -1) { /* :1706-1709: pruned, slot still consumed */
        continue;
      }
      float w = 1.f;
      if (weights) {
        w = weights[is_weight_positional ? i : current];
      }
      for (int64_t j = 0; j < block_size; ++j) {
        const float x = in_kind == 1 ? ((const float*)input)[block_size * idx + j]
                                     : oracle_half_to_float(((const uint16_t*)input)[block_size * idx + j]);
        out[j] = fmaf(w, x, out[j]); /* :1729 */
      }
    }
    if (normalize_by_lengths && len) {
      const float inv = 1.f / (float)len;
      for (int64_t j = 0; j < block_size; ++j) {
        out[j] *= inv;
      }
    }
    out += block_size;
  }
  return current == index_size;
}

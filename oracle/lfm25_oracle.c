/*
 * CPU oracle for the LFM2.5 decode hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference runtime's
 * GPU kernels for the decode step.  It is the checker that the CUDA kernels
 * of this repository are compared with; it is never linked into, called from
 * or shipped with the product library.  Only the test-suite, the smoke check
 * and the CPU-baseline leg of the benchmark may load it.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle_*.py)
 * against the known-answer vectors that the reference's own tests hold, and
 * against fixtures under tests/golden/ that were produced by running the
 * reference's unmodified kernels (rebuilt for sm_100a) on a B200.
 *
 * Each function cites the reference file:line it follows.  Paths are relative
 * to the reference project's root.
 *
 * Layout constants of the model (src/config.rs:55-96, kernels/attention.cu:8-12):
 * 32 query heads, 8 KV heads, head_dim 64, GQA group 4, softmax scale 1/8.
 * Storage is bf16 (as uint16_t bit patterns) unless stated otherwise.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define Q_HEADS 32
#define KV_HEADS 8
#define HEAD_DIM 64
#define HALF_DIM 32
#define Q_PER_KV 4
#define PARTIAL_STRIDE 66
#define ATTN_SCALE 0.125

/* ---------------------------------------------------------------- bf16 --- */

static inline float bf16_to_f32(uint16_t bits) {
    uint32_t wide = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &wide, sizeof value);
    return value;
}

/* Round-to-nearest-even, NaN kept quiet: the behaviour of __float2bfloat16_rn. */
static inline uint16_t f32_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof bits);
    if ((bits & 0x7fffffffu) > 0x7f800000u) {
        return 0x7fffu;
    }
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

/* __hmul on two bf16 values: the exact product rounded once to bf16. */
static inline uint16_t bf16_mul(uint16_t a, uint16_t b) {
    /* 8-bit x 8-bit significands: the product is exact in fp32. */
    return f32_to_bf16(bf16_to_f32(a) * bf16_to_f32(b));
}

uint16_t oracle_f32_to_bf16(float value) { return f32_to_bf16(value); }
float oracle_bf16_to_f32(uint16_t bits) { return bf16_to_f32(bits); }

/* ---------------------------------------------------------------- E4M3 --- */

/*
 * float -> E4M3 (1-4-3, bias 7, no infinity, 0x7f = NaN), round to nearest
 * even, saturate to +-448.  Follows kernels/fp8_quantize.cu:25-37, whose
 * conversion is __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3):
 * magnitudes above 464 saturate to 0x7e, 448..464 round down to 0x7e,
 * magnitudes <= 2^-10 flush to zero (the tie at 2^-10 goes to even = 0).
 */
uint8_t oracle_e4m3_from_f32(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof bits);
    const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
    const uint32_t magnitude_bits = bits & 0x7fffffffu;
    if (magnitude_bits > 0x7f800000u) {
        return (uint8_t)(sign | 0x7fu);
    }
    float magnitude;
    memcpy(&magnitude, &magnitude_bits, sizeof magnitude);
    if (magnitude >= 448.0f) {
        return (uint8_t)(sign | 0x7eu);
    }
    if (magnitude < 0.015625f) {
        /* Subnormal range: step 2^-9.  rintf rounds ties to even; the value 8
         * is the encoding of the smallest normal, which is what it should be. */
        const float steps = rintf(magnitude * 512.0f);
        return (uint8_t)(sign | (uint8_t)steps);
    }
    int exponent;
    const float fraction = frexpf(magnitude, &exponent); /* [0.5, 1) */
    float mantissa = rintf((fraction * 2.0f - 1.0f) * 8.0f);
    exponent -= 1;
    if (mantissa == 8.0f) {
        mantissa = 0.0f;
        exponent += 1;
    }
    return (uint8_t)(sign | (uint8_t)((exponent + 7) << 3) | (uint8_t)mantissa);
}

float oracle_e4m3_to_f32(uint8_t code) {
    const uint32_t exponent = (code >> 3) & 0xfu;
    const uint32_t mantissa = code & 0x7u;
    float magnitude;
    if (exponent == 0xfu && mantissa == 0x7u) {
        magnitude = NAN;
    } else if (exponent == 0) {
        magnitude = ldexpf((float)mantissa, -9);
    } else {
        magnitude = ldexpf(1.0f + (float)mantissa / 8.0f, (int)exponent - 7);
    }
    return (code & 0x80u) ? -magnitude : magnitude;
}

/*
 * Per-tensor scale pair from an absolute maximum.
 * Follows src/model/quantization.rs:159-173: non-finite or non-positive amax
 * gives the identity pair; otherwise q = 448 / amax, d = amax / 448 (f32).
 */
void oracle_scalar_scale(float clip_amax, float* quantize_multiplier, float* dequantize_multiplier) {
    if (!isfinite(clip_amax) || clip_amax <= 0.0f) {
        *quantize_multiplier = 1.0f;
        *dequantize_multiplier = 1.0f;
        return;
    }
    *quantize_multiplier = 448.0f / clip_amax;
    *dequantize_multiplier = clip_amax / 448.0f;
}

/* kernels/fp8_quantize.cu:9-45: code[i] = e4m3(float(x[i]) * scale). */
void oracle_quantize_bf16_e4m3(const uint16_t* input, uint8_t* output, size_t numel, float scale) {
#pragma omp parallel for schedule(static)
    for (size_t index = 0; index < numel; ++index) {
        const float scaled = bf16_to_f32(input[index]) * scale;
        output[index] = oracle_e4m3_from_f32(scaled);
    }
}

/*
 * kernels/silu_mul.cu:7-9,95-111 (and :13-61 for the bf16 variant).
 * packed row = [gate(0..I) | up(0..I)]; h = bf16(silu(g) * u) with
 * silu(x) = x / (1 + exp(-x)); code = e4m3(float(h) * scale).
 * The reference evaluates exp with the GPU's fast __expf; this oracle uses
 * expf, so codes may differ by one step on a very small fraction of elements.
 * `hidden_out` (bf16, may be NULL) receives h; `codes_out` (may be NULL) the codes.
 */
void oracle_silu_mul_packed(const uint16_t* packed, uint16_t* hidden_out, uint8_t* codes_out,
                            size_t rows, size_t intermediate, float scale) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row) {
        const uint16_t* gate = packed + row * 2 * intermediate;
        const uint16_t* up = gate + intermediate;
        for (size_t column = 0; column < intermediate; ++column) {
            const float g = bf16_to_f32(gate[column]);
            const float u = bf16_to_f32(up[column]);
            const float silu = g / (1.0f + expf(-g));
            const uint16_t rounded = f32_to_bf16(silu * u);
            if (hidden_out) {
                hidden_out[row * intermediate + column] = rounded;
            }
            if (codes_out) {
                codes_out[row * intermediate + column] =
                    oracle_e4m3_from_f32(bf16_to_f32(rounded) * scale);
            }
        }
    }
}

/*
 * FP8 linear.  Follows src/ops/linear.rs:62-75, src/cuda/blaslt/mod.rs:274-295,
 * src/cuda/blaslt/fp8.rs:99-107,319-322:
 *   Y[m,n] = bf16( output_scale * sum_k e4m3(X[m,k]) * e4m3(W[n,k]) ),
 * X [M,K] and W [N,K] row-major E4M3 codes, fp32 accumulation inside cuBLASLt
 * (closed source; the order of summation is unspecified).  Every product of two
 * E4M3 values is exact in fp32, so this oracle sums in double, which bounds
 * the distance to any fp32 summation order.  `exact_out` (may be NULL)
 * receives the unrounded double result for tolerance checks.
 */
void oracle_linear_fp8(const uint8_t* x, const uint8_t* weight, uint16_t* out, double* exact_out,
                       size_t m, size_t n, size_t k, float output_scale) {
    float lut[256];
    for (int code = 0; code < 256; ++code) {
        lut[code] = oracle_e4m3_to_f32((uint8_t)code);
    }
#pragma omp parallel for schedule(static)
    for (size_t column = 0; column < n; ++column) {
        const uint8_t* w_row = weight + column * k;
        for (size_t row = 0; row < m; ++row) {
            const uint8_t* x_row = x + row * k;
            double sum = 0.0;
            for (size_t inner = 0; inner < k; ++inner) {
                sum += (double)(lut[x_row[inner]] * lut[w_row[inner]]);
            }
            const double scaled = sum * (double)output_scale;
            if (exact_out) {
                exact_out[row * n + column] = scaled;
            }
            out[row * n + column] = f32_to_bf16((float)scaled);
        }
    }
}

/* ------------------------------------------------------------ KV append --- */

/* Element index inside a paged cache tensor [pages, 8, page_size, 64]
 * (kernels/attention_async_fast.cu:39-48, kernels/kv_cache.cu:64-106). */
static inline size_t cache_index(size_t page, size_t head, size_t offset, size_t dim, size_t page_size) {
    return ((page * KV_HEADS + head) * page_size + offset) * HEAD_DIM + dim;
}

/*
 * Raw append.  Follows kernels/kv_cache.cu:30-120: token t goes to physical
 * slot slot_mapping[t]; page = slot / page_size, offset = slot % page_size;
 * a negative slot or page >= num_pages skips the token.  Pure bit copy.
 */
void oracle_kv_cache_write(const uint16_t* key, const uint16_t* value, uint16_t* key_cache,
                           uint16_t* value_cache, const int64_t* slot_mapping, size_t num_tokens,
                           size_t num_pages, size_t page_size) {
    for (size_t token = 0; token < num_tokens; ++token) {
        const int64_t slot = slot_mapping[token];
        if (slot < 0) {
            continue;
        }
        const size_t page = (size_t)slot / page_size;
        const size_t offset = (size_t)slot % page_size;
        if (page >= num_pages) {
            continue;
        }
        for (size_t head = 0; head < KV_HEADS; ++head) {
            const size_t source = (token * KV_HEADS + head) * HEAD_DIM;
            const size_t destination = cache_index(page, head, offset, 0, page_size);
            memcpy(key_cache + destination, key + source, HEAD_DIM * sizeof(uint16_t));
            memcpy(value_cache + destination, value + source, HEAD_DIM * sizeof(uint16_t));
        }
    }
}

/* Sum of 32 lane values in the order of a shuffle-down tree (deltas 16,8,4,2,1)
 * as read by lane 0: kernels/qk_postprocess.cu:13-19. */
static float warp_tree_sum(const float* lanes) {
    float work[32];
    memcpy(work, lanes, sizeof work);
    for (int delta = 16; delta > 0; delta >>= 1) {
        for (int lane = 0; lane < delta; ++lane) {
            work[lane] = work[lane] + work[lane + delta];
        }
    }
    return work[0];
}

/* One head of RMSNorm + RoPE, rounding points as kernels/qk_postprocess.cu:21-30,104-112:
 *   sum   = tree_sum( fma(x[l], x[l], x[l+32]*x[l+32]) )
 *   inv   = rsqrt_rn(sum/64 + eps)
 *   y     = float( bf16(x*inv) *bf16 weight )
 *   out[l]    = bf16( fma(-y[l+32], sin_l, y[l]*cos_l) )
 *   out[l+32] = bf16( fma( y[l],    sin_l, y[l+32]*cos_l) )
 */
static void norm_rope_head(const uint16_t* in, const uint16_t* weight, const float* sin_table,
                           const float* cos_table, float eps, uint16_t* out) {
    float lanes[32];
    for (int lane = 0; lane < HALF_DIM; ++lane) {
        const float raw0 = bf16_to_f32(in[lane]);
        const float raw1 = bf16_to_f32(in[lane + HALF_DIM]);
        lanes[lane] = fmaf(raw0, raw0, raw1 * raw1);
    }
    const float sum = warp_tree_sum(lanes);
    const float mean = sum * (1.0f / 64.0f) + eps;
    /* correctly rounded reciprocal square root */
    const float inv_rms = (float)(1.0 / sqrt((double)mean));
    for (int lane = 0; lane < HALF_DIM; ++lane) {
        const float raw0 = bf16_to_f32(in[lane]);
        const float raw1 = bf16_to_f32(in[lane + HALF_DIM]);
        const float x0 = bf16_to_f32(bf16_mul(f32_to_bf16(raw0 * inv_rms), weight[lane]));
        const float x1 = bf16_to_f32(bf16_mul(f32_to_bf16(raw1 * inv_rms), weight[lane + HALF_DIM]));
        const float s = sin_table[lane];
        const float c = cos_table[lane];
        out[lane] = f32_to_bf16(fmaf(-x1, s, x0 * c));
        out[lane + HALF_DIM] = f32_to_bf16(fmaf(x0, s, x1 * c));
    }
}

/*
 * Fused decode post-processing.  Follows kernels/qk_postprocess.cu:44-151:
 * a token whose slot is negative or beyond the pool is skipped entirely (its
 * query stays untouched); otherwise Q is normalised and rotated in place,
 * K is normalised and rotated straight into the paged cache, V is copied.
 * Angle = float(position) * inv_freq[l] evaluated with sincosf.
 */
void oracle_qk_norm_rope_kv_write_decode(uint16_t* query, const uint16_t* key, const uint16_t* value,
                                         const uint16_t* query_norm, const uint16_t* key_norm,
                                         const float* inv_freq, const uint32_t* position_ids,
                                         const int64_t* slot_mapping, uint16_t* key_cache,
                                         uint16_t* value_cache, size_t num_tokens, size_t num_pages,
                                         size_t page_size, float eps) {
    for (size_t token = 0; token < num_tokens; ++token) {
        const int64_t slot = slot_mapping[token];
        if (slot < 0) {
            continue;
        }
        const size_t page = (size_t)slot / page_size;
        const size_t offset = (size_t)slot % page_size;
        if (page >= num_pages) {
            continue;
        }
        float sin_table[HALF_DIM];
        float cos_table[HALF_DIM];
        for (int lane = 0; lane < HALF_DIM; ++lane) {
            const float angle = (float)position_ids[token] * inv_freq[lane];
            sin_table[lane] = sinf(angle);
            cos_table[lane] = cosf(angle);
        }
        for (size_t head = 0; head < Q_HEADS; ++head) {
            uint16_t rotated[HEAD_DIM];
            uint16_t* row = query + (token * Q_HEADS + head) * HEAD_DIM;
            norm_rope_head(row, query_norm, sin_table, cos_table, eps, rotated);
            memcpy(row, rotated, sizeof rotated);
        }
        for (size_t head = 0; head < KV_HEADS; ++head) {
            const size_t source = (token * KV_HEADS + head) * HEAD_DIM;
            const size_t destination = cache_index(page, head, offset, 0, page_size);
            norm_rope_head(key + source, key_norm, sin_table, cos_table, eps, key_cache + destination);
            memcpy(value_cache + destination, value + source, HEAD_DIM * sizeof(uint16_t));
        }
    }
}

/* ------------------------------------------------------------ attention --- */

/*
 * Exact softmax state of one (token, query head) over logical pages
 * [first_page, end_page), keys limited to positions <= position.
 * Returns 0 if a block-table entry is out of range (the reference CTA returns
 * silently in that case), 1 otherwise.  max/denominator/accumulator follow the
 * partial-record convention of kernels/attention_async_fast.cu:253-267,350-357:
 * an empty range yields (-inf, 0, 0...).
 * Scores: 0.125 * sum_d float(Q[d]) * float(K[d]) (kernels/attention.cu:232-246).
 * This is a two-pass evaluation in double precision, not the online recurrence.
 */
static int attention_range(const uint16_t* q_row, const uint16_t* key_cache, const uint16_t* value_cache,
                           const uint32_t* block_table, size_t kv_head, uint32_t position,
                           size_t first_page, size_t end_page, size_t num_pages, size_t page_size,
                           double* maximum_out, double* denominator_out, double* accumulator) {
    double q[HEAD_DIM];
    for (int dim = 0; dim < HEAD_DIM; ++dim) {
        q[dim] = (double)bf16_to_f32(q_row[dim]);
        accumulator[dim] = 0.0;
    }
    *maximum_out = -INFINITY;
    *denominator_out = 0.0;
    if (first_page >= end_page) {
        return 1;
    }
    const size_t first_token = first_page * page_size;
    size_t end_token = end_page * page_size;
    if (end_token > (size_t)position + 1) {
        end_token = (size_t)position + 1;
    }
    const size_t count = end_token - first_token;
    double* scores = (double*)malloc(count * sizeof(double));
    double maximum = -INFINITY;
    for (size_t token = first_token; token < end_token; ++token) {
        const size_t physical_page = block_table[token / page_size];
        if (physical_page >= num_pages) {
            free(scores);
            return 0;
        }
        const uint16_t* k_row = key_cache + cache_index(physical_page, kv_head, token % page_size, 0, page_size);
        double dot = 0.0;
        for (int dim = 0; dim < HEAD_DIM; ++dim) {
            dot += q[dim] * (double)bf16_to_f32(k_row[dim]);
        }
        dot *= ATTN_SCALE;
        scores[token - first_token] = dot;
        if (dot > maximum) {
            maximum = dot;
        }
    }
    double denominator = 0.0;
    for (size_t token = first_token; token < end_token; ++token) {
        const size_t physical_page = block_table[token / page_size];
        const uint16_t* v_row = value_cache + cache_index(physical_page, kv_head, token % page_size, 0, page_size);
        const double weight = exp(scores[token - first_token] - maximum);
        denominator += weight;
        for (int dim = 0; dim < HEAD_DIM; ++dim) {
            accumulator[dim] += weight * (double)bf16_to_f32(v_row[dim]);
        }
    }
    free(scores);
    *maximum_out = maximum;
    *denominator_out = denominator;
    return 1;
}

/*
 * Ragged paged GQA decode attention.
 * Follows kernels/attention.cu:144-270 (precise kernel) and
 * kernels/attention_async_fast.cu:72-205 (production kernel) for everything
 * but the order of floating-point operations:
 *   token t reads block_tables[request_slots[t]] (row 0 when request_slots is NULL),
 *   keys 0..=position_ids[t], kv head = q head / 4, O = bf16(acc / denominator).
 * A token is skipped, leaving its output rows untouched, when its request slot
 * is >= block_table_rows, its position is >= stride * page_size, or a needed
 * block-table entry is >= num_pages (attention_async_fast.cu:88-111,149-151).
 * `exact_out` (may be NULL) receives the unrounded result [T,32,64] as double.
 */
void oracle_paged_ragged_attention(const uint16_t* query, const uint16_t* key_cache,
                                   const uint16_t* value_cache, const uint32_t* block_tables,
                                   const uint32_t* request_slots, const uint32_t* position_ids,
                                   uint16_t* output, double* exact_out, size_t num_tokens,
                                   size_t num_pages, size_t block_table_stride,
                                   size_t block_table_rows, size_t page_size) {
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (size_t token = 0; token < num_tokens; ++token) {
        for (size_t kv_head = 0; kv_head < KV_HEADS; ++kv_head) {
            const size_t row = request_slots ? (size_t)request_slots[token] : 0;
            if (row >= block_table_rows || block_table_stride == 0) {
                continue;
            }
            const uint32_t position = position_ids[token];
            if ((size_t)position >= block_table_stride * page_size) {
                continue;
            }
            const uint32_t* table = block_tables + row * block_table_stride;
            const size_t total_pages = (size_t)position / page_size + 1;
            double results[Q_PER_KV][HEAD_DIM];
            double denominators[Q_PER_KV];
            int valid = 1;
            for (size_t offset = 0; offset < Q_PER_KV && valid; ++offset) {
                const size_t q_head = kv_head * Q_PER_KV + offset;
                double maximum;
                valid = attention_range(query + (token * Q_HEADS + q_head) * HEAD_DIM, key_cache,
                                        value_cache, table, kv_head, position, 0, total_pages,
                                        num_pages, page_size, &maximum, &denominators[offset],
                                        results[offset]);
            }
            if (!valid) {
                continue;
            }
            for (size_t offset = 0; offset < Q_PER_KV; ++offset) {
                const size_t q_head = kv_head * Q_PER_KV + offset;
                const size_t base = (token * Q_HEADS + q_head) * HEAD_DIM;
                for (int dim = 0; dim < HEAD_DIM; ++dim) {
                    const double value = results[offset][dim] / denominators[offset];
                    if (exact_out) {
                        exact_out[base + dim] = value;
                    }
                    output[base + dim] = f32_to_bf16((float)value);
                }
            }
        }
    }
}

/*
 * Split-K partial records.  Follows kernels/attention_async_fast.cu:211-358:
 * split s of S covers logical pages [P*s/S, P*(s+1)/S) with P = position/16 + 1;
 * record index ((t*32 + q)*S + s)*66 holds (max, denominator, acc[64]) in f32,
 * un-normalised, relative to the split's own maximum; an empty split holds
 * (-inf, 0, 0...).  Skipped tokens leave their records untouched.
 */
void oracle_paged_ragged_attention_splitk_partials(
    const uint16_t* query, const uint16_t* key_cache, const uint16_t* value_cache,
    const uint32_t* block_tables, const uint32_t* request_slots, const uint32_t* position_ids,
    float* partials, size_t num_tokens, size_t num_pages, size_t block_table_stride,
    size_t block_table_rows, size_t page_size, uint32_t num_splits) {
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (size_t token = 0; token < num_tokens; ++token) {
        for (size_t kv_head = 0; kv_head < KV_HEADS; ++kv_head) {
            const size_t row = (size_t)request_slots[token];
            if (row >= block_table_rows || block_table_stride == 0 || num_splits <= 1) {
                continue;
            }
            const uint32_t position = position_ids[token];
            if ((size_t)position >= block_table_stride * page_size) {
                continue;
            }
            const uint32_t* table = block_tables + row * block_table_stride;
            const size_t total_pages = (size_t)position / page_size + 1;
            for (size_t split = 0; split < num_splits; ++split) {
                const size_t first_page = total_pages * split / num_splits;
                const size_t end_page = total_pages * (split + 1) / num_splits;
                for (size_t offset = 0; offset < Q_PER_KV; ++offset) {
                    const size_t q_head = kv_head * Q_PER_KV + offset;
                    double maximum, denominator, accumulator[HEAD_DIM];
                    const int valid = attention_range(
                        query + (token * Q_HEADS + q_head) * HEAD_DIM, key_cache, value_cache, table,
                        kv_head, position, first_page, end_page, num_pages, page_size, &maximum,
                        &denominator, accumulator);
                    if (!valid) {
                        continue;
                    }
                    float* record = partials + ((token * Q_HEADS + q_head) * num_splits + split) * PARTIAL_STRIDE;
                    record[0] = (float)maximum;
                    record[1] = (float)denominator;
                    for (int dim = 0; dim < HEAD_DIM; ++dim) {
                        record[2 + dim] = (float)accumulator[dim];
                    }
                }
            }
        }
    }
}

/*
 * Merge of split-K records.  Follows kernels/attention_async_fast.cu:362-419:
 * M = max_s m_s; w_s = (l_s == 0) ? 0 : exp(m_s - M);
 * O = bf16( sum_s w_s*acc_s / sum_s w_s*l_s ).
 */
void oracle_merge_splitk(const float* partials, uint16_t* output, size_t num_tokens, uint32_t num_splits) {
#pragma omp parallel for schedule(static)
    for (size_t item = 0; item < num_tokens * Q_HEADS; ++item) {
        const float* records = partials + item * num_splits * PARTIAL_STRIDE;
        double maximum = -INFINITY;
        for (uint32_t split = 0; split < num_splits; ++split) {
            const double m = (double)records[split * PARTIAL_STRIDE];
            if (m > maximum) {
                maximum = m;
            }
        }
        double denominator = 0.0;
        double accumulator[HEAD_DIM] = {0.0};
        for (uint32_t split = 0; split < num_splits; ++split) {
            const float* record = records + split * PARTIAL_STRIDE;
            const double scale = record[1] == 0.0f ? 0.0 : exp((double)record[0] - maximum);
            denominator += (double)record[1] * scale;
            for (int dim = 0; dim < HEAD_DIM; ++dim) {
                accumulator[dim] += (double)record[2 + dim] * scale;
            }
        }
        for (int dim = 0; dim < HEAD_DIM; ++dim) {
            output[item * HEAD_DIM + dim] = f32_to_bf16((float)(accumulator[dim] / denominator));
        }
    }
}

/* ------------------------------------------------------- step metadata --- */

/*
 * Decode-step slot computation.  Follows src/model/lfm2_base.rs:371-378:
 * physical_slot = block_table[slot_row][pos / page_size] * page_size + pos % page_size.
 * An unassigned entry (0xffffffff) or out-of-range row gives -1, the value that
 * the append kernels skip.
 */
void oracle_physical_slots(const uint32_t* block_tables, const uint32_t* request_slots,
                           const uint32_t* position_ids, int64_t* physical_slots, size_t num_tokens,
                           size_t block_table_stride, size_t block_table_rows, size_t page_size) {
    for (size_t token = 0; token < num_tokens; ++token) {
        const size_t row = request_slots[token];
        const size_t position = position_ids[token];
        physical_slots[token] = -1;
        if (row >= block_table_rows || position / page_size >= block_table_stride) {
            continue;
        }
        const uint32_t page = block_tables[row * block_table_stride + position / page_size];
        if (page == 0xffffffffu) {
            continue;
        }
        physical_slots[token] = (int64_t)page * (int64_t)page_size + (int64_t)(position % page_size);
    }
}

/* ------------------------------------------------------- other step ops --- */

/*
 * RMSNorm of rows.  Follows kernels/rms_norm.cu:268-278: inv = rsqrt_rn(mean(x^2) + eps) with the sum in fp32
 * (here in double, which bounds every fp32 order), n = bf16(x * inv), out = n *bf16 weight.
 */
void oracle_rms_norm_bf16(const uint16_t* x, const uint16_t* weight, uint16_t* out, size_t rows, size_t hidden,
                          float eps) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row) {
        double sum = 0.0;
        for (size_t index = 0; index < hidden; ++index) {
            const double value = (double)bf16_to_f32(x[row * hidden + index]);
            sum += value * value;
        }
        const float inv_rms = (float)(1.0 / sqrt((double)((float)(sum / (double)hidden) + eps)));
        for (size_t index = 0; index < hidden; ++index) {
            const float value = bf16_to_f32(x[row * hidden + index]);
            out[row * hidden + index] = bf16_mul(f32_to_bf16(value * inv_rms), weight[index]);
        }
    }
}

/*
 * Residual add + RMSNorm.  Follows kernels/rms_norm.cu:394-453: r = bf16(residual + update) is stored; the
 * variance uses the unrounded fp32 sums; out = bf16(float(r) * inv * float(weight)).
 */
void oracle_residual_rms_norm_bf16(const uint16_t* residual, const uint16_t* update, const uint16_t* weight,
                                   uint16_t* residual_out, uint16_t* normalized_out, size_t rows, size_t hidden,
                                   float eps) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row) {
        double sum = 0.0;
        for (size_t index = 0; index < hidden; ++index) {
            const size_t offset = row * hidden + index;
            const float added = bf16_to_f32(residual[offset]) + bf16_to_f32(update[offset]);
            residual_out[offset] = f32_to_bf16(added);
            sum += (double)added * (double)added;
        }
        const float inv_rms = (float)(1.0 / sqrt((double)((float)(sum / (double)hidden) + eps)));
        for (size_t index = 0; index < hidden; ++index) {
            const size_t offset = row * hidden + index;
            const float value = bf16_to_f32(residual_out[offset]);
            normalized_out[offset] = f32_to_bf16(value * inv_rms * bf16_to_f32(weight[index]));
        }
    }
}

/*
 * Gated short convolution, decode step (one token per sequence).  Follows kernels/short_conv.cu:100-143:
 * projected[t] = (b | c | x); gated = b*x; y = c*(w0*s0 + w1*s1 + w2*gated) in fp32; state <- (s1, gated) as bf16.
 * A request slot beyond the state table skips the token.
 */
void oracle_short_conv_decode_bf16(const uint16_t* projected, const uint16_t* weight, uint16_t* states,
                                   const uint32_t* request_slots, uint16_t* output, size_t num_tokens, size_t hidden,
                                   size_t num_request_slots) {
    for (size_t token = 0; token < num_tokens; ++token) {
        const size_t slot = request_slots[token];
        if (slot >= num_request_slots) {
            continue;
        }
        for (size_t channel = 0; channel < hidden; ++channel) {
            uint16_t* state = states + (slot * hidden + channel) * 2;
            const float state0 = bf16_to_f32(state[0]);
            const float state1 = bf16_to_f32(state[1]);
            const float w0 = bf16_to_f32(weight[channel * 3]);
            const float w1 = bf16_to_f32(weight[channel * 3 + 1]);
            const float w2 = bf16_to_f32(weight[channel * 3 + 2]);
            const size_t base = token * hidden * 3;
            const float b = bf16_to_f32(projected[base + channel]);
            const float c = bf16_to_f32(projected[base + hidden + channel]);
            const float x = bf16_to_f32(projected[base + hidden * 2 + channel]);
            const float gated = b * x;
            const float convolved = w0 * state0 + w1 * state1 + w2 * gated;
            output[token * hidden + channel] = f32_to_bf16(c * convolved);
            state[0] = f32_to_bf16(state1);
            state[1] = f32_to_bf16(gated);
        }
    }
}

/*
 * Gated short convolution over token segments (prefill chunks and decode tokens in one batch).  Follows
 * kernels/short_conv.cu:100-143 (short_conv_segmented_lfm2_bf16): per (segment, channel) the two state values are
 * loaded once, carried in fp32 across the segment's tokens (state1 <- gated is NOT rounded between tokens) and
 * stored as bf16 at the end; y[token] = bf16(c * (w0*s0 + w1*s1 + w2*gated)).  A segment whose slot is beyond
 * the state table is skipped.
 */
void oracle_short_conv_segmented_bf16(const uint16_t* projected, const uint16_t* weight, uint16_t* states,
                                      const uint32_t* segment_offsets, const uint32_t* segment_slots,
                                      uint16_t* output, size_t num_segments, size_t hidden,
                                      size_t num_request_slots) {
#pragma omp parallel for schedule(static)
    for (size_t channel = 0; channel < hidden; ++channel) {
        for (size_t segment = 0; segment < num_segments; ++segment) {
            const size_t slot = segment_slots[segment];
            if (slot >= num_request_slots) {
                continue;
            }
            uint16_t* state = states + (slot * hidden + channel) * 2;
            float state0 = bf16_to_f32(state[0]);
            float state1 = bf16_to_f32(state[1]);
            const float w0 = bf16_to_f32(weight[channel * 3]);
            const float w1 = bf16_to_f32(weight[channel * 3 + 1]);
            const float w2 = bf16_to_f32(weight[channel * 3 + 2]);
            for (size_t token = segment_offsets[segment]; token < segment_offsets[segment + 1]; ++token) {
                const size_t base = token * hidden * 3;
                const float b = bf16_to_f32(projected[base + channel]);
                const float c = bf16_to_f32(projected[base + hidden + channel]);
                const float x = bf16_to_f32(projected[base + hidden * 2 + channel]);
                const float gated = b * x;
                const float convolved = w0 * state0 + w1 * state1 + w2 * gated;
                output[token * hidden + channel] = f32_to_bf16(c * convolved);
                state0 = state1;
                state1 = gated;
            }
            state[0] = f32_to_bf16(state0);
            state[1] = f32_to_bf16(state1);
        }
    }
}

/*
 * Hybrid ragged attention of a mixed prefill / decode step.  Follows kernels/attention.cu:389-558
 * (hybrid_ragged_gqa_lfm2_bf16_body) for everything but the order of floating-point operations: token t belongs
 * to the segment [segment_offsets[s], segment_offsets[s+1]) that contains it (segment 0's start if none does);
 * with current_offset = t - segment_begin and prefix = position_ids[t] - current_offset it attends to
 *   keys 0 .. prefix-1            of the paged cache, through block_tables[request_slots[t]], and
 *   tokens segment_begin .. t     of the contiguous current_key / current_value [T, 8, 64],
 * scale 0.125, kv head = q head / 4, exact two-pass softmax in double, O = bf16(acc / denominator).
 * A token whose position is smaller than its offset, or that meets a block-table entry >= num_pages, leaves
 * its output rows untouched.  `exact_out` (may be NULL) receives the unrounded result.
 */
void oracle_hybrid_ragged_attention(const uint16_t* query, const uint16_t* current_key,
                                    const uint16_t* current_value, const uint16_t* key_cache,
                                    const uint16_t* value_cache, const uint32_t* block_tables,
                                    const uint32_t* request_slots, const uint32_t* position_ids,
                                    const uint32_t* segment_offsets, uint16_t* output, double* exact_out,
                                    size_t num_tokens, size_t num_pages, size_t block_table_stride,
                                    size_t num_segments, size_t page_size) {
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (size_t token = 0; token < num_tokens; ++token) {
        for (size_t q_head = 0; q_head < Q_HEADS; ++q_head) {
            const size_t kv_head = q_head / Q_PER_KV;
            size_t segment_begin = 0;
            for (size_t segment = 0; segment < num_segments; ++segment) {
                if (token >= segment_offsets[segment] && token < segment_offsets[segment + 1]) {
                    segment_begin = segment_offsets[segment];
                    break;
                }
            }
            const size_t position = position_ids[token];
            const size_t current_offset = token - segment_begin;
            if (position < current_offset) {
                continue;
            }
            const size_t prefix = position - current_offset;
            const uint32_t* table = block_tables + (size_t)request_slots[token] * block_table_stride;
            const size_t count = prefix + current_offset + 1;
            double* scores = (double*)malloc(count * sizeof(double));
            const uint16_t** value_rows = (const uint16_t**)malloc(count * sizeof(const uint16_t*));
            const uint16_t* q_row = query + (token * Q_HEADS + q_head) * HEAD_DIM;
            double maximum = -INFINITY;
            int valid = 1;
            for (size_t index = 0; index < count && valid; ++index) {
                const uint16_t* k_row;
                if (index < prefix) {
                    const size_t physical_page = table[index / page_size];
                    if (physical_page >= num_pages) {
                        valid = 0;
                        break;
                    }
                    const size_t at = cache_index(physical_page, kv_head, index % page_size, 0, page_size);
                    k_row = key_cache + at;
                    value_rows[index] = value_cache + at;
                } else {
                    const size_t at = ((segment_begin + (index - prefix)) * KV_HEADS + kv_head) * HEAD_DIM;
                    k_row = current_key + at;
                    value_rows[index] = current_value + at;
                }
                double dot = 0.0;
                for (int dim = 0; dim < HEAD_DIM; ++dim) {
                    dot += (double)bf16_to_f32(q_row[dim]) * (double)bf16_to_f32(k_row[dim]);
                }
                scores[index] = dot * ATTN_SCALE;
                if (scores[index] > maximum) {
                    maximum = scores[index];
                }
            }
            if (valid) {
                double accumulator[HEAD_DIM] = {0.0};
                double denominator = 0.0;
                for (size_t index = 0; index < count; ++index) {
                    const double weight = exp(scores[index] - maximum);
                    denominator += weight;
                    for (int dim = 0; dim < HEAD_DIM; ++dim) {
                        accumulator[dim] += weight * (double)bf16_to_f32(value_rows[index][dim]);
                    }
                }
                const size_t base = (token * Q_HEADS + q_head) * HEAD_DIM;
                for (int dim = 0; dim < HEAD_DIM; ++dim) {
                    const double value = accumulator[dim] / denominator;
                    if (exact_out) {
                        exact_out[base + dim] = value;
                    }
                    output[base + dim] = f32_to_bf16((float)value);
                }
            }
            free(scores);
            free(value_rows);
        }
    }
}

/*
 * Greedy argmax per row with the legacy tie order.  Follows kernels/sampling.cu:53-134: the winner is the largest
 * value; among equal values the smaller (column % 256) wins, then the smaller (column / 256); NaN and -inf never
 * win (a row of only those answers 0); +0 and -0 are equal.
 */
void oracle_argmax_rows_bf16(const uint16_t* logits, uint32_t* sampled, size_t rows, size_t vocab) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row) {
        int found = 0;
        float best = 0.0f;
        uint32_t best_column = 0;
        for (size_t column = 0; column < vocab; ++column) {
            const uint16_t bits = logits[row * vocab + column];
            const float value = bf16_to_f32(bits);
            if (isnan(value) || (isinf(value) && value < 0.0f)) {
                continue;
            }
            int better = !found || value > best;
            if (found && value == best) {
                const uint32_t lane = (uint32_t)column & 0xffu, offset = (uint32_t)column >> 8;
                const uint32_t best_lane = best_column & 0xffu, best_offset = best_column >> 8;
                better = lane < best_lane || (lane == best_lane && offset < best_offset);
            }
            if (better) {
                found = 1;
                best = value;
                best_column = (uint32_t)column;
            }
        }
        sampled[row] = found ? best_column : 0u;
    }
}

/*
 * BF16 linear: Y[M,N] = bf16( sum_k X[m,k] * W[n,k] ).  Follows src/cuda/blaslt/mod.rs:113-186 (cuBLASLt, fp32
 * compute, order unspecified); products of two bf16 values are exact in fp32, the sum is taken in double.
 */
void oracle_linear_bf16(const uint16_t* x, const uint16_t* weight, uint16_t* out, size_t m, size_t n, size_t k) {
    float* x_f32 = (float*)malloc(m * k * sizeof(float));
    for (size_t index = 0; index < m * k; ++index) {
        x_f32[index] = bf16_to_f32(x[index]);
    }
#pragma omp parallel for schedule(static)
    for (size_t column = 0; column < n; ++column) {
        const uint16_t* w_row = weight + column * k;
        for (size_t row = 0; row < m; ++row) {
            const float* x_row = x_f32 + row * k;
            double sum = 0.0;
            for (size_t inner = 0; inner < k; ++inner) {
                sum += (double)(x_row[inner] * bf16_to_f32(w_row[inner]));
            }
            out[row * n + column] = f32_to_bf16((float)sum);
        }
    }
    free(x_f32);
}

/* Sets the OpenMP team size of the following calls (a launcher may have exported OMP_NUM_THREADS=1). */
void oracle_set_num_threads(int count) {
#ifdef _OPENMP
    if (count > 0) {
        omp_set_num_threads(count);
    }
#else
    (void)count;
#endif
}

int oracle_num_threads(void) {
    int count = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        count = omp_get_num_threads();
    }
#endif
    return count;
}

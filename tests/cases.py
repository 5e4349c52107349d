"""Input builders shared by the GPU parity tests, the golden-fixture generator and the oracle-vs-golden test.

The attention cases restate the inputs of the reference's own GPU tests (patterned tensors, block-table
orders, lengths); citations are file:line inside the reference project."""
import numpy as np

from lfm25_inference_b200 import workloads
from oracle import oracle


def write_cache(key, value, slots, pages, page_size=16):
    key_cache = np.zeros((pages, 8, page_size, 64), dtype=np.uint16)
    value_cache = np.zeros_like(key_cache)
    oracle.kv_cache_write(key, value, key_cache, value_cache, np.asarray(slots, dtype=np.int64), page_size)
    return key_cache, value_cache


def single_context_case(context):
    """src/ops/attention_async_fast_tests.rs:27-65 (one sequence, identity block table)."""
    key = workloads.patterned_bf16(context * 8 * 64, 13 + context, 89, 44.0, 64.0).reshape(context, 8, 64)
    value = workloads.patterned_bf16(context * 8 * 64, 7 + context, 79, 39.0, 32.0).reshape(context, 8, 64)
    query = workloads.patterned_bf16(32 * 64, 17 + context, 101, 50.0, 64.0).reshape(1, 32, 64)
    pages = (context + 15) // 16
    key_cache, value_cache = write_cache(key, value, list(range(context)), pages)
    return dict(query=query, key_cache=key_cache, value_cache=value_cache,
                block_tables=np.arange(pages, dtype=np.uint32).reshape(1, pages),
                request_slots=np.zeros(1, dtype=np.uint32), position_ids=np.array([context - 1], dtype=np.uint32))


SINGLE_CONTEXTS = [1, 16, 17, 33, 67, 128]


def ragged_reversed_case():
    """src/ops/attention_async_fast_tests.rs:67-146: 2 requests, context 2*PS+1, reversed page order per request."""
    requests, context = 2, 33
    pages_per_request = 3
    tables = np.zeros((requests, pages_per_request), dtype=np.uint32)
    for request in range(requests):
        for logical in range(pages_per_request):
            tables[request, logical] = request * pages_per_request + pages_per_request - 1 - logical
    slots = [int(tables[r, p // 16]) * 16 + p % 16 for r in range(requests) for p in range(context)]
    key = workloads.patterned_bf16(requests * context * 8 * 64, 13, 89, 44.0, 64.0).reshape(-1, 8, 64)
    value = workloads.patterned_bf16(requests * context * 8 * 64, 7, 79, 39.0, 32.0).reshape(-1, 8, 64)
    query = workloads.patterned_bf16(requests * 32 * 64, 17, 101, 50.0, 64.0).reshape(requests, 32, 64)
    key_cache, value_cache = write_cache(key, value, slots, requests * pages_per_request)
    return dict(query=query, key_cache=key_cache, value_cache=value_cache, block_tables=tables,
                request_slots=np.array([0, 1], dtype=np.uint32),
                position_ids=np.array([context - 1, context - 1], dtype=np.uint32))


def splitk_case():
    """src/ops/attention_splitk_tests.rs:21-132: lengths [257, 65], consecutive pages, unassigned tail entries."""
    lengths = [257, 65]
    pages = [(length + 15) // 16 for length in lengths]
    stride = max(pages)
    total_tokens = sum(lengths)
    index = np.arange(2 * 32 * 64, dtype=np.int64)
    query = oracle.f32_to_bf16(((index * 17 % 113).astype(np.float32) - 56.0) / 96.0).reshape(2, 32, 64)
    index = np.arange(total_tokens * 8 * 64, dtype=np.int64)
    key = oracle.f32_to_bf16(((index * 13 % 97).astype(np.float32) - 48.0) / 96.0).reshape(total_tokens, 8, 64)
    value = oracle.f32_to_bf16(((index * 7 % 89).astype(np.float32) - 44.0) / 48.0).reshape(total_tokens, 8, 64)
    tables = np.full((2, stride), 0xFFFFFFFF, dtype=np.uint32)
    slots = []
    base = 0
    for request, (length, count) in enumerate(zip(lengths, pages)):
        tables[request, :count] = base + np.arange(count)
        slots += [(base + p // 16) * 16 + p % 16 for p in range(length)]
        base += count
    key_cache, value_cache = write_cache(key, value, slots, base)
    return dict(query=query, key_cache=key_cache, value_cache=value_cache, block_tables=tables,
                request_slots=np.array([0, 1], dtype=np.uint32),
                position_ids=np.array([lengths[0] - 1, lengths[1] - 1], dtype=np.uint32))


def random_ragged_case(seed, sequences, low, high, pages):
    """Seeded N(0,1) ragged batch after its first append (positions = contexts)."""
    rng = np.random.default_rng(seed)
    batch = workloads.ragged_decode_batch(seed, sequences, low, high, pages, 1)
    key_cache, value_cache = workloads.fill_pool_for_batch(rng, batch)
    query = workloads.bf16_normal(rng, (sequences, 32, 64))
    return dict(query=query, key_cache=key_cache, value_cache=value_cache, block_tables=batch.block_tables,
                request_slots=batch.request_slots, position_ids=batch.positions(0))


def qk_postprocess_case(seed=11, tokens=6):
    """src/ops/qk_postprocess.rs:189-275: slots straddle a page boundary; one token is skipped (slot -1)."""
    rng = np.random.default_rng(seed)
    return dict(
        query=workloads.bf16_normal(rng, (tokens, 32, 64)), key=workloads.bf16_normal(rng, (tokens, 8, 64)),
        value=workloads.bf16_normal(rng, (tokens, 8, 64)),
        query_norm=oracle.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(64)),
        key_norm=oracle.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(64)), inv_freq=oracle.rope_inv_freq(),
        position_ids=np.array([0, 14, 15, 16, 4099, 33], dtype=np.uint32)[:tokens],
        slot_mapping=np.array([16, 30, 31, 0, 2 * 16 + 3, -1], dtype=np.int64)[:tokens], num_pages=3, eps=1e-5)


def fp8_inputs(seed=21, rows=5, width=1000):
    rng = np.random.default_rng(seed)
    values = workloads.bf16_normal(rng, (rows, width), std=1.5)
    values.reshape(-1)[:8] = oracle.f32_to_bf16(np.array([0.0, -0.0, 448.0, -1000.0, 1e-3, 2 ** -10, 3e38, -3e38],
                                                         dtype=np.float32))
    packed = workloads.bf16_normal(rng, (rows, 2 * width), std=2.0)
    return values, packed


def hybrid_known_answer_case():
    """src/ops/attention_regression_tests.rs:64-111: zero queries and keys, a prefix of two cached tokens with
    V = 2 and a current chunk of two tokens with V = 6; the outputs are the plain means 10/3 and 4."""
    prefix_value = oracle.f32_to_bf16(np.full((2, 8, 64), 2.0, dtype=np.float32))
    key_cache, value_cache = write_cache(np.zeros((2, 8, 64), dtype=np.uint16), prefix_value, [0, 1], 1)
    return dict(query=np.zeros((2, 32, 64), dtype=np.uint16), current_key=np.zeros((2, 8, 64), dtype=np.uint16),
                current_value=oracle.f32_to_bf16(np.full((2, 8, 64), 6.0, dtype=np.float32)),
                key_cache=key_cache, value_cache=value_cache, block_tables=np.zeros((1, 1), dtype=np.uint32),
                request_slots=np.zeros(2, dtype=np.uint32), position_ids=np.array([2, 3], dtype=np.uint32),
                segment_offsets=np.array([0, 2], dtype=np.uint32))


def mixed_step_case(seed, prefixes, chunks, pages):
    """Seeded N(0,1) mixed prefill / decode step: prefixes in the paged cache (NaN patterns everywhere else),
    the step's own K/V contiguous."""
    rng = np.random.default_rng(seed)
    batch = workloads.mixed_step_batch(seed, prefixes, chunks, pages)
    key_cache, value_cache = workloads.fill_prefixes(rng, batch)
    tokens = batch.num_tokens
    return dict(batch=batch, query=workloads.bf16_normal(rng, (tokens, 32, 64)),
                current_key=workloads.bf16_normal(rng, (tokens, 8, 64)),
                current_value=workloads.bf16_normal(rng, (tokens, 8, 64)), key_cache=key_cache,
                value_cache=value_cache, block_tables=batch.block_tables, request_slots=batch.request_slots,
                position_ids=batch.positions, segment_offsets=batch.segment_offsets)


# (prefixes, chunks): page-aligned and ragged prefixes, chunks shorter and longer than a page and than a query
# tile, decode tokens (chunk 1) among prefill chunks, an empty prefix
MIXED_SMALL = ([0, 16, 5, 40, 33, 7], [1, 16, 37, 1, 3, 70])


def short_conv_segmented_case(seed=31, hidden=256):
    rng = np.random.default_rng(seed)
    chunks = np.array([1, 5, 1, 12, 2], dtype=np.int64)
    tokens = int(chunks.sum())
    return dict(projected=workloads.bf16_normal(rng, (tokens, 3 * hidden)),
                weight=workloads.bf16_normal(rng, (hidden, 3), std=0.5),
                states=workloads.bf16_normal(rng, (7, hidden, 2)),
                segment_offsets=np.concatenate([[0], np.cumsum(chunks)]).astype(np.uint32),
                segment_slots=np.array([3, 0, 9, 6, 1], dtype=np.uint32))      # slot 9 is beyond the table: skipped


# The E4M3 decode GEMM sites at the batch sizes of the sweep (the reference's FP8 call sites,
# src/model/decode_executor.rs:35-76 with the shapes of src/model/lfm2.rs): 15 points.
FP8_GEMM_SITES = {"gate_up": (16384, 2048), "down": (2048, 8192), "lm_head": (65536, 2048)}
FP8_GEMM_BATCHES = (1, 8, 32, 128, 256)
FP8_GEMM_BLOCK = 512          # weight rows generated from one seed
FP8_GEMM_SAMPLE = 32          # rows sampled from the head of each of four blocks: 128 output columns
FP8_WEIGHT_CLIP = 0.1         # static weight scale c_w (5 sigma of N(0, 0.02)); values beyond it saturate
FP8_ACTIVATION_CLIP = 5.0     # static activation scale c_x


def fp8_gemm_weight_block(site, block):
    """E4M3 codes of weight rows [block * 512, block * 512 + 512) of a site: N(0, 0.02) quantised with c_w = 0.1.
    Every block has its own seed, so a test that checks a sample of the output columns only builds those rows."""
    n, k = FP8_GEMM_SITES[site]
    rng = np.random.default_rng([17, sorted(FP8_GEMM_SITES).index(site), block])
    weights = workloads.bf16_normal(rng, (min(FP8_GEMM_BLOCK, n - block * FP8_GEMM_BLOCK), k), std=0.02)
    return oracle.quantize_bf16_e4m3(weights, oracle.scalar_scale(FP8_WEIGHT_CLIP)[0])


def fp8_gemm_sample_blocks(site):
    blocks = FP8_GEMM_SITES[site][0] // FP8_GEMM_BLOCK
    return [0, blocks // 3, (2 * blocks) // 3, blocks - 1]


def fp8_gemm_point(site, m):
    """(activation codes [m, k], output scale d_x * d_w, sampled output columns) of one point of the sweep."""
    n, k = FP8_GEMM_SITES[site]
    rng = np.random.default_rng([19, sorted(FP8_GEMM_SITES).index(site), m])
    x_quantize, x_dequantize = oracle.scalar_scale(FP8_ACTIVATION_CLIP)
    x_codes = oracle.quantize_bf16_e4m3(workloads.bf16_normal(rng, (m, k)), x_quantize)
    columns = np.concatenate([np.arange(block * FP8_GEMM_BLOCK, block * FP8_GEMM_BLOCK + FP8_GEMM_SAMPLE)
                              for block in fp8_gemm_sample_blocks(site)])
    return x_codes, x_dequantize * oracle.scalar_scale(FP8_WEIGHT_CLIP)[1], columns


def fp8_gemm_sampled_weights(site):
    """The weight rows of the sampled output columns, [128, k]."""
    return np.concatenate([fp8_gemm_weight_block(site, block)[:FP8_GEMM_SAMPLE]
                           for block in fp8_gemm_sample_blocks(site)])

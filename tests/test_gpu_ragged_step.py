"""The mixed prefill / decode step of the executor (the reference's forward_prepared_batch on a ragged batch):
against the CPU step oracle, and the invariant a serving loop relies on -- prefilling a prompt in chunks and then
decoding gives what feeding the same tokens one by one through the decode step gives."""
import numpy as np
import pytest
import torch

from oracle import step_oracle
from conftest import bits_of
from lfm25_inference_b200 import model as lfm_model
from lfm25_inference_b200 import ops, workloads
from oracle import oracle

pytestmark = pytest.mark.gpu


def compare_logits(got_bits, want_bits, use_fp8):
    got = oracle.bf16_to_f32(got_bits).astype(np.float64)
    want = oracle.bf16_to_f32(want_bits).astype(np.float64)
    scale = np.abs(want).max()
    # the bounds of the decode-step test: 16 layers of bf16 round-offs; one E4M3 code flip upstream is a 6 % step
    assert np.abs(got - want).max() <= (0.15 if use_fp8 else 0.05) * scale
    cosine = (got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want))
    assert cosine >= (0.99 if use_fp8 else 0.999)


@pytest.mark.parametrize("prefixes,chunks", [([0, 20, 7, 33], [19, 1, 5, 1]),       # all segments in the hybrid kernel
                                             ([20, 33, 0, 7], [1, 1, 19, 5])])      # decode segments first: routed
@pytest.mark.parametrize("use_fp8", [False, True])
def test_mixed_step_against_the_oracle(device, use_fp8, prefixes, chunks):
    pages = 32
    batch = workloads.mixed_step_batch(3, prefixes, chunks, pages)
    assert lfm_model.leading_decode_segments(batch)[0] == (2 if chunks[0] == 1 else 0)
    model = lfm_model.RandomModel(3, device, pages, batch.num_segments)
    model.fill_caches(4)
    rng = np.random.default_rng(3)
    token_ids = rng.integers(0, lfm_model.VOCAB, size=batch.num_tokens).astype(np.uint32)
    host = step_oracle.HostModel(model)
    blaslt = ops.BlasLt()
    executor = lfm_model.DecodeExecutor(blaslt, 64, maximum_segments=8)
    device_batch = lfm_model.RaggedBatch(device, batch, token_ids)
    executor.forward_ragged(model, device_batch, use_fp8=use_fp8)
    got_logits = executor.logits(batch.num_segments)
    got_sampled = executor.sampled(batch.num_segments)
    want_logits, _ = step_oracle.ragged_step(host, token_ids, batch, use_fp8)
    compare_logits(got_logits, want_logits, use_fp8)
    assert np.array_equal(got_sampled, oracle.argmax_rows_bf16(got_logits))
    assert np.array_equal(device_batch.physical_slots.cpu().numpy(), batch.physical_slots)
    # every token of the step was appended at its slot, nothing else in the pools changed
    for index, layer in enumerate(model.layers):
        if not layer.is_attention:
            continue
        got = oracle.bf16_to_f32(bits_of(layer.tensors["key_cache"])).astype(np.float64)
        want = oracle.bf16_to_f32(host.layers[index]["key_cache"]).astype(np.float64)
        assert np.abs(got - want).max() <= (0.15 if use_fp8 else 0.05) * max(1.0, np.abs(want).max())
    for index, layer in enumerate(model.layers):
        if layer.is_attention:
            continue
        got = oracle.bf16_to_f32(bits_of(layer.tensors["conv_state"])).astype(np.float64)
        want = oracle.bf16_to_f32(host.layers[index]["conv_state"]).astype(np.float64)
        assert np.abs(got - want).max() <= (0.15 if use_fp8 else 0.05) * max(1.0, np.abs(want).max())
    assert ops.device_status()[0] == 0
    executor.close()
    blaslt.close()


def test_chunked_prefill_then_decode_equals_token_by_token_decode(device):
    """One sequence of 45 prompt tokens: (a) prefill in chunks of 16, 16, 13, then 3 greedy decode steps;
    (b) the same prompt fed one token per decode step.  Logits within bf16 noise, interchangeable greedy ids
    (the chunked route carries the conv state unrounded inside a chunk and uses other GEMM shapes)."""
    pages, prompt_length, decode_steps = 8, 45, 3
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, lfm_model.VOCAB, size=prompt_length).astype(np.uint32)
    table = np.arange(pages, dtype=np.uint32).reshape(1, pages)[:, ::-1].copy()

    def fresh():
        model = lfm_model.RandomModel(7, device, pages, 1)
        for layer in model.layers:                      # empty sequence: zero conv state, pools of NaN patterns
            for name in ("key_cache", "value_cache"):
                if name in layer.tensors:
                    layer.tensors[name].view(torch.int16).fill_(0x7FC1)
        blaslt = ops.BlasLt()
        return model, blaslt, lfm_model.DecodeExecutor(blaslt, 32, maximum_segments=4)

    def decode_one(model, executor, token, position):
        batch = lfm_model.DecodeBatch(device, table, np.zeros(1, np.uint32), np.array([position], np.uint32),
                                      np.array([token], np.uint32), position + 1)
        executor.forward(model, batch, use_fp8=False, advance=False)
        return executor.logits(1).copy(), int(executor.sampled(1)[0])

    # (b) token by token
    model, blaslt, executor = fresh()
    for position, token in enumerate(prompt):
        logits, sampled = decode_one(model, executor, int(token), position)
    serial_logits, serial_ids = [logits], [sampled]
    for step in range(decode_steps):
        logits, sampled = decode_one(model, executor, serial_ids[-1], prompt_length + step)
        serial_logits.append(logits)
        serial_ids.append(sampled)
    serial_cache = bits_of(model.layers[2].tensors["key_cache"])
    executor.close()
    blaslt.close()

    # (a) chunked prefill, then decode steps fed with route (b)'s ids so that both routes see the same tokens
    model, blaslt, executor = fresh()
    start = 0
    for chunk in (16, 16, 13):
        batch = workloads.MixedStepBatch(pages, table, np.array([start]), np.array([chunk]), np.zeros(1, np.uint32))
        executor.forward_ragged(model, lfm_model.RaggedBatch(device, batch, prompt[start:start + chunk]),
                                use_fp8=False)
        start += chunk
    chunked_logits = [executor.logits(1).copy()]
    chunked_ids = [int(executor.sampled(1)[0])]
    for step in range(decode_steps):
        logits, sampled = decode_one(model, executor, serial_ids[step], prompt_length + step)
        chunked_logits.append(logits)
        chunked_ids.append(sampled)
    chunked_cache = bits_of(model.layers[2].tensors["key_cache"])
    executor.close()
    blaslt.close()

    # the greedy choice of one route is (within the noise) a maximum of the other route's logits
    for chosen, logits in zip(chunked_ids, serial_logits):
        values = oracle.bf16_to_f32(logits[0]).astype(np.float64)
        assert values[chosen] >= values.max() - 0.05 * np.abs(values).max()
    for a, b in zip(chunked_logits, serial_logits):
        compare_logits(a, b, False)
    live = slice(0, prompt_length + decode_steps)      # the first attention layer's keys, position by position
    rows = [(int(table[0, position // 16]), position % 16) for position in range(live.stop)]
    a = np.stack([oracle.bf16_to_f32(chunked_cache[page, :, offset, :]) for page, offset in rows])
    b = np.stack([oracle.bf16_to_f32(serial_cache[page, :, offset, :]) for page, offset in rows])
    assert np.abs(a - b).max() <= 0.05 * max(1.0, np.abs(b).max())
    assert ops.device_status()[0] == 0


def test_ragged_step_argument_checks(device):
    pages = 8
    batch = workloads.mixed_step_batch(3, [0, 4], [9, 1], pages)
    model = lfm_model.RandomModel(3, device, pages, 2)
    blaslt = ops.BlasLt()
    executor = lfm_model.DecodeExecutor(blaslt, 8, maximum_segments=1)
    tokens = np.zeros(batch.num_tokens, dtype=np.uint32)
    with pytest.raises(ops.Lfm25Error, match="token count exceeds workspace"):
        executor.forward_ragged(model, lfm_model.RaggedBatch(device, batch, tokens))
    executor.close()
    executor = lfm_model.DecodeExecutor(blaslt, 16, maximum_segments=1)
    with pytest.raises(ops.Lfm25Error, match="segment count exceeds workspace"):
        executor.forward_ragged(model, lfm_model.RaggedBatch(device, batch, tokens))
    executor.close()
    with pytest.raises(ops.Lfm25Error, match="up to 8192 tokens"):
        lfm_model.DecodeExecutor(blaslt, 9000, maximum_segments=4)
    blaslt.close()


def test_prefix_reuse_through_radix_index_and_conv_checkpoints(device):
    """The reuse path of the serving loop (src/engine/serving/radix_owner.rs:464-547): request A prefills a prompt
    in two chunks and publishes the page-aligned first chunk (radix index + convolution checkpoint); request B with
    the same prompt finds it, shares the KV pages, restores the convolution states and prefills only the rest.
    Same chunk, same inputs: B's logits must be A's, bit for bit."""
    from lfm25_inference_b200 import cache

    pages, prompt_length, shared = 16, 45, 32
    rng = np.random.default_rng(21)
    prompt = rng.integers(0, lfm_model.VOCAB, size=prompt_length).astype(np.uint32)
    model = lfm_model.RandomModel(9, device, pages, 2)
    conv_layers = [layer for layer in model.layers if not layer.is_attention]
    allocator = cache.KvPageAllocator(pages)
    tables = cache.FixedBlockTables(2, 4)
    radix = cache.PageRadixCache(16, 8)
    checkpoints = cache.ConvCheckpointPool(len(conv_layers), 4)
    blaslt = ops.BlasLt()
    executor = lfm_model.DecodeExecutor(blaslt, 64, maximum_segments=2)
    stream = torch.cuda.current_stream().cuda_stream

    def prefill(slot, start, stop):
        batch = workloads.MixedStepBatch(pages, tables.as_array().copy(), np.array([start]), np.array([stop - start]),
                                         np.array([slot], dtype=np.uint32))
        executor.forward_ragged(model, lfm_model.RaggedBatch(device, batch, prompt[start:stop]), use_fp8=False)

    # request A, slot 0
    allocator.try_reserve_tokens(prompt_length)
    allocator.grow_sequence(0, prompt_length, tables.slot(0))
    prefill(0, 0, shared)
    slot = checkpoints.acquire()
    for index, layer in enumerate(conv_layers):
        checkpoints.capture_layer(stream, slot, index, layer.tensors["conv_state"], 0)
    assert radix.can_publish(prompt, shared)
    allocator.pin_cached_pages(radix.insert_checkpoint(prompt, shared, tables.slot(0)[:shared // 16], slot))
    prefill(0, shared, prompt_length)
    logits_a = executor.logits(1).copy()

    # request B, slot 1: the admission lookup leaves at least one prompt token to compute
    matched, found_slot, shared_pages = radix.longest_checkpoint(prompt, prompt_length - 1)
    assert (matched, found_slot) == (shared, slot) and list(shared_pages) == list(tables.slot(0)[:2])
    allocator.retain_pages(shared_pages)
    tables.slot(1)[:len(shared_pages)] = shared_pages
    allocator.try_reserve_tokens(prompt_length - matched)
    allocator.grow_sequence(matched, prompt_length, tables.slot(1))
    assert tables.slot(1)[2] != tables.slot(0)[2]                     # the unshared tail has its own page
    for index, layer in enumerate(conv_layers):
        checkpoints.restore_layer(stream, found_slot, index, layer.tensors["conv_state"], 1)
    prefill(1, matched, prompt_length)
    logits_b = executor.logits(1).copy()

    assert np.array_equal(logits_a, logits_b)
    assert radix.snapshot()["hits"] == 1 and checkpoints.available() == 3
    assert ops.device_status()[0] == 0
    executor.close()
    blaslt.close()
    checkpoints.close()
    radix.close()

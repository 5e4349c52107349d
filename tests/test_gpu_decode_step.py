"""The decode executor (C ABI): one full 16-layer step against the CPU restatement of the same op sequence, and
the device-advanced, graph-replayed step against the eager one."""
import numpy as np
import pytest
import torch

from conftest import bits_of
from lfm25_inference_b200 import model as lfm_model
from lfm25_inference_b200 import ops, workloads
from oracle import oracle
from oracle import step_oracle

pytestmark = pytest.mark.gpu


def small_batch(device, seed, tokens, pages, steps):
    batch = workloads.ragged_decode_batch(seed, tokens, 3, 70, pages, steps + 1)
    rng = np.random.default_rng(seed)
    token_ids = rng.integers(0, lfm_model.VOCAB, size=tokens).astype(np.uint32)
    return batch, token_ids


@pytest.mark.parametrize("route", [0, 1], ids=["two_launches", "one_kernel"])
@pytest.mark.parametrize("pack_qkv", [True, False])
@pytest.mark.parametrize("use_fp8", [False, True])
def test_one_step_against_the_oracle(device, library_option, use_fp8, pack_qkv, route):
    """Both routes of an attention layer (QK-norm + RoPE + append as a kernel of their own, or inside attention),
    with the three projections packed into one GEMM or apart."""
    library_option("fused_append", route)
    tokens, pages = 3, 32
    model = lfm_model.RandomModel(3, device, pages, 4, pack_qkv=pack_qkv)
    model.fill_caches(4)
    batch, token_ids = small_batch(device, 3, tokens, pages, 2)
    host = step_oracle.HostModel(model)
    blaslt = ops.BlasLt()
    executor = lfm_model.DecodeExecutor(blaslt, 8)
    device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0), token_ids,
                                         int(batch.contexts.max()) + 4)
    before = {index: bits_of(layer.tensors["key_cache"]) for index, layer in enumerate(model.layers)
              if layer.is_attention}
    executor.forward(model, device_batch, use_fp8=use_fp8, advance=False)
    got_logits = oracle.bf16_to_f32(executor.logits(tokens)).astype(np.float64)
    got_sampled = executor.sampled(tokens)
    want_logits_bits, _ = step_oracle.decode_step(host, token_ids, batch.positions(0), batch.request_slots,
                                                  batch.block_tables, use_fp8)
    want_logits = oracle.bf16_to_f32(want_logits_bits).astype(np.float64)
    # 16 layers of bf16 round-offs: compare on the scale of the logits.  With FP8 sites a one-bit difference
    # upstream can move an activation to the neighbouring E4M3 code (a 6 % step), so the end-to-end bound is
    # wider there; each FP8 op by itself is checked exactly in test_gpu_fp8_linear.py / test_gpu_fp8_elementwise.py.
    scale = np.abs(want_logits).max()
    assert np.abs(got_logits - want_logits).max() <= (0.15 if use_fp8 else 0.05) * scale
    cosine = (got_logits * want_logits).sum() / (np.linalg.norm(got_logits) * np.linalg.norm(want_logits))
    assert cosine >= (0.99 if use_fp8 else 0.999)
    # the sampled ids are the argmax of the executor's own logits, with the legacy tie order
    assert np.array_equal(got_sampled, oracle.argmax_rows_bf16(executor.logits(tokens)))
    # the step appended exactly one K/V row per sequence and layer, at the slots of the block tables
    slots = batch.physical_slots(0)
    for index, layer in enumerate(model.layers):
        if not layer.is_attention:
            continue
        want = host.layers[index]["key_cache"]
        got = bits_of(layer.tensors["key_cache"])
        changed = np.argwhere((got != before[index]).any(axis=(1, 3)))
        pages_touched = {(int(page), int(offset)) for page, offset in changed}
        assert pages_touched == {(int(slot) // 16, int(slot) % 16) for slot in slots}
        for slot in slots:
            page, offset = int(slot) // 16, int(slot) % 16
            a = oracle.bf16_to_f32(got[page, :, offset, :]).astype(np.float64)
            b = oracle.bf16_to_f32(want[page, :, offset, :]).astype(np.float64)
            assert np.abs(a - b).max() <= (0.15 if use_fp8 else 0.05) * max(1.0, np.abs(b).max())
    assert ops.device_status()[0] == 0
    executor.close()
    blaslt.close()


def test_graph_replay_matches_eager_steps(device):
    tokens, pages, steps = 5, 64, 6
    batch, token_ids = small_batch(device, 9, tokens, pages, steps)

    def run(use_graph):
        with torch.cuda.stream(torch.cuda.Stream()):      # graph capture needs a non-default stream
            return run_on_current_stream(use_graph)

    def run_on_current_stream(use_graph):
        model = lfm_model.RandomModel(5, device, pages, 8)
        model.fill_caches(6)
        blaslt = ops.BlasLt()
        executor = lfm_model.DecodeExecutor(blaslt, 8)
        device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0),
                                             token_ids, int(batch.contexts.max()) + steps + 1)
        history = []
        executor.forward(model, device_batch, use_fp8=True, advance=False)
        history.append(executor.sampled(tokens))
        for _ in range(steps):
            if use_graph:
                executor.step_graph(model, device_batch, use_fp8=True)
            else:
                executor.forward(model, device_batch, use_fp8=True, advance=True)
            history.append(executor.sampled(tokens))
        logits = executor.logits(tokens)
        positions = device_batch.positions.cpu().numpy().view(np.uint32)
        caches = [bits_of(layer.tensors["key_cache"]) for layer in model.layers if layer.is_attention]
        torch.cuda.current_stream().synchronize()
        executor.close()
        blaslt.close()
        return history, logits, positions, caches

    eager = run(False)
    graph = run(True)
    for a, b in zip(eager[0], graph[0]):
        assert np.array_equal(a, b)
    assert np.array_equal(eager[1], graph[1])
    assert np.array_equal(eager[2], batch.positions(0) + steps) and np.array_equal(graph[2], eager[2])
    for a, b in zip(eager[3], graph[3]):
        assert np.array_equal(a, b)
    # each step feeds the previous step's sampled ids: the histories must not be constant by construction
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("use_fp8", [False, True])
def test_one_step_against_the_reference_kernels(device, use_fp8):
    """The same step assembled from the reference's own kernels (compiled for this GPU) and cuBLASLt, on a second
    model with the same seed: logits within the end-to-end bound used against the CPU restatement, the appended
    K rows within the reference's own tolerance for its fast path."""
    from oracle import refkernels, refstep
    if not refkernels.available():
        pytest.skip("oracle/_ref holds no compiled reference kernels")
    tokens, pages = 16, 128                                # cuBLASLt's FP8 GEMM wants the batch in multiples of 16
    batch = workloads.ragged_decode_batch(11, tokens, 5, 90, pages, 3)
    token_ids = np.random.default_rng(11).integers(0, lfm_model.VOCAB, size=tokens).astype(np.uint32)
    ours, theirs = (lfm_model.RandomModel(7, device, pages, tokens) for _ in range(2))
    ours.fill_caches(8)
    theirs.fill_caches(8)
    blaslt = ops.BlasLt()
    executor = lfm_model.DecodeExecutor(blaslt, tokens)
    device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0), token_ids,
                                         int(batch.contexts.max()) + 4)
    executor.forward(ours, device_batch, use_fp8=use_fp8, advance=False)
    got = oracle.bf16_to_f32(executor.logits(tokens)).astype(np.float64)
    got_sampled = executor.sampled(tokens)

    reference = refstep.ReferenceKernelStep(theirs, tokens, use_fp8=use_fp8)
    slots = torch.from_numpy(batch.physical_slots(0).astype(np.int64)).to(device)
    reference.forward(device_batch.token_ids, device_batch.positions, device_batch.request_slots, slots,
                      device_batch.block_tables)
    torch.cuda.synchronize()
    want = oracle.bf16_to_f32(bits_of(reference.logits)).astype(np.float64)
    want_sampled = reference.sampled.cpu().numpy().view(np.uint32)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= (0.15 if use_fp8 else 0.05) * scale
    cosine = (got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want))
    assert cosine >= (0.99 if use_fp8 else 0.999)
    # greedy ids agree wherever the reference's top two logits are further apart than the bound
    ordered = np.sort(want, axis=1)
    decided = ordered[:, -1] - ordered[:, -2] > 2 * np.abs(got - want).max(axis=1)
    assert np.array_equal(got_sampled[decided], want_sampled[decided])
    for mine, other in zip(ours.layers, theirs.layers):
        if mine.is_attention:
            a = oracle.bf16_to_f32(bits_of(mine.tensors["key_cache"])).astype(np.float64)
            b = oracle.bf16_to_f32(bits_of(other.tensors["key_cache"])).astype(np.float64)
            assert np.abs(a - b).max() <= (0.15 if use_fp8 else 0.05) * max(1.0, np.abs(b).max())
        else:
            a = oracle.bf16_to_f32(bits_of(mine.tensors["conv_state"])).astype(np.float64)
            b = oracle.bf16_to_f32(bits_of(other.tensors["conv_state"])).astype(np.float64)
            assert np.abs(a - b).max() <= (0.15 if use_fp8 else 0.05) * max(1.0, np.abs(b).max())
    assert ops.device_status()[0] == 0
    executor.close()
    blaslt.close()


def test_served_step_equals_upload_replay_download(device):
    """lfm25_decode_executor_serve_step is upload + captured step + download + synchronise in one call."""
    tokens, pages, steps = 6, 64, 4
    batch, token_ids = small_batch(device, 21, tokens, pages, steps)

    def run(served):
        with torch.cuda.stream(torch.cuda.Stream()):
            model = lfm_model.RandomModel(5, device, pages, 8)
            model.fill_caches(6)
            blaslt = ops.BlasLt()
            executor = lfm_model.DecodeExecutor(blaslt, 8)
            device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0),
                                                 token_ids, int(batch.contexts.max()) + steps + 1)
            host_block = device_batch.step_metadata.cpu().pin_memory()
            host_sampled = torch.zeros(tokens, dtype=torch.int32).pin_memory()
            history = []
            for _ in range(steps):
                if served:
                    executor.serve_step(model, device_batch, host_block, host_sampled)
                else:
                    device_batch.step_metadata.copy_(host_block, non_blocking=True)
                    executor.forward(model, device_batch, use_fp8=True, advance=False)
                    executor.download_sampled(host_sampled)
                    torch.cuda.current_stream().synchronize()
                history.append(host_sampled.numpy().copy())
                host_block[:tokens].copy_(host_sampled)
                host_block[tokens:2 * tokens] += 1
            executor.close()
            blaslt.close()
            return history

    for a, b in zip(run(False), run(True)):
        assert np.array_equal(a, b)
    assert ops.device_status()[0] == 0


HEADLINE_ROWS = 128


def headline_batch(seed, steps):
    """128 sequences with contexts of a few hundred tokens in a small page pool: the batch size of the benchmark's
    headline configuration, where the step takes other branches than at 3 or 16 rows (cuBLASLt for the BF16 sites,
    the gated Gate/Up in the batch-major tcgen05 kernel, unsplit attention in the device-built token order)."""
    pages = 6144
    batch = workloads.ragged_decode_batch(seed, HEADLINE_ROWS, 100, 500, pages, steps + 1)
    token_ids = np.random.default_rng(seed).integers(0, lfm_model.VOCAB, size=HEADLINE_ROWS).astype(np.uint32)
    return batch, token_ids, pages


@pytest.mark.parametrize("use_fp8", [True, False])
def test_headline_batch_against_the_reference_kernels(device, use_fp8):
    """One eager step at 128 rows against the same step assembled from the reference's own kernels and cuBLASLt
    (src/model/decode_executor.rs:183-443) on a twin model: logits within the end-to-end bound of the smaller cases,
    greedy ids equal wherever the reference's top two logits are further apart than that bound, appended K rows and
    convolution states within the same bound, no bounded wait expired."""
    from oracle import refkernels, refstep
    if not refkernels.available():
        pytest.skip("oracle/_ref holds no compiled reference kernels")
    batch, token_ids, pages = headline_batch(31, 2)
    ours, theirs = (lfm_model.RandomModel(17, device, pages, HEADLINE_ROWS) for _ in range(2))
    ours.fill_caches(18)
    theirs.fill_caches(18)
    blaslt = ops.BlasLt()
    executor = lfm_model.DecodeExecutor(blaslt, HEADLINE_ROWS)
    device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0), token_ids,
                                         int(batch.contexts.max()) + 4)
    executor.forward(ours, device_batch, use_fp8=use_fp8, advance=False)
    got = oracle.bf16_to_f32(executor.logits(HEADLINE_ROWS)).astype(np.float64)
    got_sampled = executor.sampled(HEADLINE_ROWS)
    reference = refstep.ReferenceKernelStep(theirs, HEADLINE_ROWS, use_fp8=use_fp8)
    slots = torch.from_numpy(batch.physical_slots(0).astype(np.int64)).to(device)
    reference.forward(device_batch.token_ids, device_batch.positions, device_batch.request_slots, slots,
                      device_batch.block_tables)
    torch.cuda.synchronize()
    want = oracle.bf16_to_f32(bits_of(reference.logits)).astype(np.float64)
    want_sampled = reference.sampled.cpu().numpy().view(np.uint32)
    bound = 0.15 if use_fp8 else 0.05
    assert np.abs(got - want).max() <= bound * np.abs(want).max()
    cosine = (got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want))
    assert cosine >= (0.99 if use_fp8 else 0.999)
    assert np.array_equal(got_sampled, oracle.argmax_rows_bf16(executor.logits(HEADLINE_ROWS)))
    ordered = np.sort(want, axis=1)
    decided = ordered[:, -1] - ordered[:, -2] > 2 * np.abs(got - want).max(axis=1)
    assert decided.any()
    assert np.array_equal(got_sampled[decided], want_sampled[decided])
    for mine, other in zip(ours.layers, theirs.layers):
        name = "key_cache" if mine.is_attention else "conv_state"
        a = oracle.bf16_to_f32(bits_of(mine.tensors[name])).astype(np.float64)
        b = oracle.bf16_to_f32(bits_of(other.tensors[name])).astype(np.float64)
        assert np.abs(a - b).max() <= bound * max(1.0, np.abs(b).max())
    assert ops.device_status()[0] == 0
    executor.close()
    blaslt.close()


def test_headline_batch_graph_replay_matches_eager_steps(device):
    """Three self-feeding steps at 128 rows from the captured graph against the same steps launched eagerly on a twin
    model: sampled ids of every step, final logits, positions, K caches and convolution states bit for bit."""
    steps = 3
    batch, token_ids, pages = headline_batch(33, steps)

    def run(use_graph):
        with torch.cuda.stream(torch.cuda.Stream()):
            model = lfm_model.RandomModel(19, device, pages, HEADLINE_ROWS)
            model.fill_caches(20)
            blaslt = ops.BlasLt()
            executor = lfm_model.DecodeExecutor(blaslt, HEADLINE_ROWS)
            device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0),
                                                 token_ids, int(batch.contexts.max()) + steps + 1)
            history = []
            executor.forward(model, device_batch, use_fp8=True, advance=False)
            history.append(executor.sampled(HEADLINE_ROWS))
            for _ in range(steps):
                if use_graph:
                    executor.step_graph(model, device_batch, use_fp8=True)
                else:
                    executor.forward(model, device_batch, use_fp8=True, advance=True)
                history.append(executor.sampled(HEADLINE_ROWS))
            captures = executor.graph_captures()
            state = [executor.logits(HEADLINE_ROWS), device_batch.positions.cpu().numpy().view(np.uint32)]
            state += [bits_of(layer.tensors["key_cache" if layer.is_attention else "conv_state"])
                      for layer in model.layers]
            torch.cuda.current_stream().synchronize()
            executor.close()
            blaslt.close()
            return history, state, captures

    eager_history, eager_state, _ = run(False)
    graph_history, graph_state, captures = run(True)
    assert captures == 1
    for a, b in zip(eager_history, graph_history):
        assert np.array_equal(a, b)
    for a, b in zip(eager_state, graph_state):
        assert np.array_equal(a, b)
    assert np.array_equal(eager_state[1], batch.positions(0) + steps)
    assert ops.device_status()[0] == 0


def test_changed_batch_buffers_capture_again(device):
    """A captured step bakes in every pointer and stride of the batch: after the block tables move to a wider
    allocation (same contents, larger stride) under the same token-id buffer, the next calls run eagerly once and
    capture again instead of replaying the stale graph, and the results stay those of the eager step."""
    tokens, pages, steps = 6, 64, 8
    batch, token_ids = small_batch(device, 41, tokens, pages, steps)
    with torch.cuda.stream(torch.cuda.Stream()):
        model = lfm_model.RandomModel(5, device, pages, 8)
        model.fill_caches(6)
        twin = lfm_model.RandomModel(5, device, pages, 8)
        twin.fill_caches(6)
        blaslt = ops.BlasLt()
        executor = lfm_model.DecodeExecutor(blaslt, 8)
        reference = lfm_model.DecodeExecutor(blaslt, 8)
        context = int(batch.contexts.max()) + steps + 1
        device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0),
                                             token_ids, context)
        twin_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0),
                                           token_ids, context)
        for _ in range(3):                                   # eager warm-up, capture, replay
            executor.step_graph(model, device_batch, use_fp8=True)
            reference.forward(twin, twin_batch, use_fp8=True, advance=True)
        assert executor.graph_captures() == 1
        assert np.array_equal(executor.sampled(tokens), reference.sampled(tokens))
        # the tables move: twice the stride, unassigned tail entries, a new allocation
        wide = np.full((batch.block_tables.shape[0], 2 * batch.block_tables.shape[1]), 0xFFFFFFFF, dtype=np.uint32)
        wide[:, :batch.block_tables.shape[1]] = batch.block_tables
        moved = torch.from_numpy(wide.view(np.int32).copy()).to(device)
        device_batch.block_tables = moved
        device_batch.struct.block_tables = moved.data_ptr()
        device_batch.struct.block_table_stride = wide.shape[1]
        for _ in range(3):
            executor.step_graph(model, device_batch, use_fp8=True)
            reference.forward(twin, twin_batch, use_fp8=True, advance=True)
        assert executor.graph_captures() == 2
        assert np.array_equal(executor.sampled(tokens), reference.sampled(tokens))
        assert np.array_equal(device_batch.positions.cpu().numpy(), twin_batch.positions.cpu().numpy())
        torch.cuda.current_stream().synchronize()
        assert ops.device_status()[0] == 0
        executor.close()
        reference.close()
        blaslt.close()


@pytest.mark.parametrize("rows,low,high", [(8, 1500, 3000), (40, 600, 2500)])
def test_split_merge_inside_the_kernel_changes_no_bit_of_a_step(device, library_option, rows, low, high):
    """Small batches of long contexts split the KV axis (8 splits at 8 rows, 2 at 40); the executor then merges the
    splits inside the attention kernel (a cluster per token and KV head) instead of through records and the merge
    kernel.  Two self-feeding steps, eagerly and from the graph, with the switch on and off: sampled ids, logits and
    caches bit for bit."""
    steps = 2
    pages = 8192
    batch = workloads.ragged_decode_batch(41, rows, low, high, pages, steps + 1)
    token_ids = np.random.default_rng(41).integers(0, lfm_model.VOCAB, size=rows).astype(np.uint32)
    assert ops.splitk_decode_splits(rows, int(batch.contexts.max()) + steps + 1, 16) in (2, 4, 8)

    def run(in_kernel, use_graph):
        library_option("splitk_cluster_merge", in_kernel)
        with torch.cuda.stream(torch.cuda.Stream()):
            model = lfm_model.RandomModel(23, device, pages, rows)
            model.fill_caches(24)
            blaslt = ops.BlasLt()
            executor = lfm_model.DecodeExecutor(blaslt, rows)
            device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0),
                                                 token_ids, int(batch.contexts.max()) + steps + 1)
            executor.forward(model, device_batch, use_fp8=True, advance=False)
            history = [executor.sampled(rows)]
            for _ in range(steps):
                if use_graph:
                    executor.step_graph(model, device_batch, use_fp8=True)
                else:
                    executor.forward(model, device_batch, use_fp8=True, advance=True)
                history.append(executor.sampled(rows))
            state = [executor.logits(rows)]
            state += [bits_of(layer.tensors["key_cache" if layer.is_attention else "conv_state"])
                      for layer in model.layers]
            kernels = executor.graph_kernels()
            torch.cuda.current_stream().synchronize()
            executor.close()
            blaslt.close()
            return history, state, kernels

    want_history, want_state, _ = run(0, False)
    for in_kernel, use_graph in ((1, False), (1, True), (0, True)):
        history, state, kernels = run(in_kernel, use_graph)
        assert all(np.array_equal(a, b) for a, b in zip(history, want_history))
        assert all(np.array_equal(a, b) for a, b in zip(state, want_state))
        if use_graph and in_kernel:
            merged_inside = kernels
        if use_graph and not in_kernel:
            assert merged_inside == kernels - 6          # one merge kernel per attention layer fewer
    assert ops.device_status()[0] == 0

"""Parity of the remaining ops of the decode step (C ABI) with the CPU oracle: embedding and the device-side step
metadata are bit-exact; RMSNorm variants, the short convolution and the cuBLASLt BF16 linear are within one bf16
step of the oracle (fp32 sums in a different order); the greedy argmax reproduces the legacy tie order exactly."""
import numpy as np
import pytest
import torch

from conftest import BF16_GEMM_PATHS, assert_close_bf16, bits_of, to_bf16, to_u32
from lfm25_inference_b200 import _abi, ops, workloads
from lfm25_inference_b200._abi import check, library
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_embedding(device):
    rng = np.random.default_rng(0)
    table = workloads.bf16_normal(rng, (1000, 2048))
    ids = np.array([0, 999, 5, 5, 1000, 77], dtype=np.uint32)         # 1000 is out of range: row stays untouched
    out = torch.full((6, 2048), 7.0, dtype=torch.bfloat16, device=device)
    ops.embedding_bf16_into(to_u32(ids, device), to_bf16(table, device), out)
    got = bits_of(out)
    for row, token in enumerate(ids):
        if token < 1000:
            assert np.array_equal(got[row], table[token])
        else:
            assert np.all(got[row] == 0x40E0)


@pytest.mark.parametrize("rows,hidden", [(1, 2048), (128, 2048), (5, 64), (3, 6144)])
def test_rms_norms(device, rows, hidden):
    rng = np.random.default_rng(rows + hidden)
    x = workloads.bf16_normal(rng, (rows, hidden), std=3.0)
    update = workloads.bf16_normal(rng, (rows, hidden), std=0.5)
    weight = oracle.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(hidden))
    out = torch.zeros((rows, hidden), dtype=torch.bfloat16, device=device)
    ops.rms_norm_bf16_into(to_bf16(x, device), to_bf16(weight, device), 1e-5, out)
    want = oracle.rms_norm_bf16(x, weight, 1e-5)
    assert_close_bf16(bits_of(out), want, 1e-6, 2 ** -7)
    assert (bits_of(out) != want).mean() < 0.01
    residual_out = torch.zeros_like(out)
    normalized = torch.zeros_like(out)
    ops.residual_rms_norm_bf16_into(to_bf16(x, device), to_bf16(update, device), to_bf16(weight, device), 1e-5,
                                    residual_out, normalized)
    want_residual, want_normalized = oracle.residual_rms_norm_bf16(x, update, weight, 1e-5)
    assert np.array_equal(bits_of(residual_out), want_residual)
    assert_close_bf16(bits_of(normalized), want_normalized, 1e-6, 2 ** -7)
    assert (bits_of(normalized) != want_normalized).mean() < 0.01
    # the variant that also emits E4M3 codes: same bf16 outputs, and the codes of quantising them afterwards
    scale = 448.0 / 6.0
    residual_fused, normalized_fused = torch.zeros_like(out), torch.zeros_like(out)
    codes = torch.zeros((rows, hidden), dtype=torch.uint8, device=device)
    ops.residual_rms_norm_bf16_e4m3_into(to_bf16(x, device), to_bf16(update, device), to_bf16(weight, device), 1e-5,
                                         residual_fused, normalized_fused, codes, scale)
    assert np.array_equal(bits_of(residual_fused), bits_of(residual_out))
    assert np.array_equal(bits_of(normalized_fused), bits_of(normalized))
    assert np.array_equal(codes.cpu().numpy(), oracle.quantize_bf16_e4m3(bits_of(normalized), scale))


def test_short_conv_decode(device):
    rng = np.random.default_rng(4)
    tokens, hidden, slots = 5, 2048, 8
    projected = workloads.bf16_normal(rng, (tokens, 3 * hidden))
    weight = workloads.bf16_normal(rng, (hidden, 3), std=0.5)
    states = workloads.bf16_normal(rng, (slots, hidden, 2))
    request_slots = np.array([3, 0, 7, 9, 1], dtype=np.uint32)      # 9 is beyond the state table: skipped
    states_device = to_bf16(states, device)
    output = torch.full((tokens, hidden), 7.0, dtype=torch.bfloat16, device=device)
    for _ in range(2):   # two steps in a row exercise the state hand-over
        ops.short_conv_decode_bf16_into(to_bf16(projected, device), to_bf16(weight, device), states_device,
                                        to_u32(request_slots, device), output)
    want_states = states.copy()
    for _ in range(2):
        want = oracle.short_conv_decode_bf16(projected, weight, want_states, request_slots)
    got = bits_of(output)
    assert np.all(got[3] == 0x40E0)
    live = [0, 1, 2, 4]
    assert_close_bf16(got[live], want[live], 1e-6, 2 ** -7)
    assert np.array_equal(bits_of(states_device), want_states)       # products of two bf16 values round identically


def test_short_conv_segmented(device):
    """Segments of 1..12 tokens, one slot beyond the state table; bit-exact against the oracle, and a segment of
    one token equals the decode kernel."""
    import cases
    case = cases.short_conv_segmented_case(hidden=2048)
    want_states = case["states"].copy()
    want = oracle.short_conv_segmented_bf16(case["projected"], case["weight"], want_states, case["segment_offsets"],
                                            case["segment_slots"])
    states = to_bf16(case["states"], device)
    output = torch.zeros((case["projected"].shape[0], 2048), dtype=torch.bfloat16, device=device)
    ops.short_conv_segmented_lfm2_bf16_into(to_bf16(case["projected"], device), to_bf16(case["weight"], device),
                                            states, to_u32(case["segment_offsets"], device),
                                            to_u32(case["segment_slots"], device), output)
    assert np.array_equal(bits_of(output), want)
    assert np.array_equal(bits_of(states), want_states)


def test_gather_rows(device):
    rng = np.random.default_rng(9)
    values = workloads.bf16_normal(rng, (11, 2048))
    rows = np.array([10, 0, 3, 99, 3], dtype=np.uint32)              # 99 is beyond the input: row left as is
    output = torch.full((5, 2048), 7.0, dtype=torch.bfloat16, device=device)
    ops.gather_rows_bf16_into(to_bf16(values, device), to_u32(rows, device), output)
    got = bits_of(output)
    for row, source in enumerate(rows):
        if source < 11:
            assert np.array_equal(got[row], values[source])
        else:
            assert (got[row] == bits_of(torch.tensor([7.0], dtype=torch.bfloat16))[0]).all()


def test_argmax_tie_order(device):
    # src/ops/sampling.rs:105-182: ties, NaN, -inf, +-0, low-cardinality rows over the full vocabulary
    rng = np.random.default_rng(6)
    vocab = 65536
    rows = []
    rows.append(oracle.f32_to_bf16(rng.integers(-3, 4, size=vocab).astype(np.float32)))         # many ties
    row = np.full(vocab, 0xFF80, dtype=np.uint16)                                               # all -inf
    rows.append(row)
    row = np.full(vocab, 0x7FC0, dtype=np.uint16)                                               # all NaN
    rows.append(row)
    row = np.full(vocab, 0x8000, dtype=np.uint16); row[513] = 0x0000                            # -0 everywhere, one +0
    rows.append(row)
    row = oracle.f32_to_bf16(np.full(vocab, -5.0, dtype=np.float32)); row[[70000 % vocab, 300, 44]] = 0x4000
    rows.append(row)
    row = workloads.bf16_normal(rng, (vocab,)); row[100] = 0x7F80; row[99] = 0x7FC0             # +inf wins, NaN ignored
    rows.append(row)
    row = oracle.f32_to_bf16(np.full(vocab, -3.0e38, dtype=np.float32))                         # all equal, very negative
    rows.append(row)
    row = np.where(np.arange(vocab) % 2 == 0, 0x7FC0, 0xFF80).astype(np.uint16)                 # only NaN and -inf
    rows.append(row)
    row = np.full(vocab, 0xFFC0, dtype=np.uint16); row[40000] = 0xC2C8                          # one finite value among NaN
    rows.append(row)
    logits = np.stack(rows)
    sampled = torch.zeros(len(rows), dtype=torch.int32, device=device)
    ops.argmax_rows_bf16_into(to_bf16(logits, device), sampled)
    got = sampled.cpu().numpy().view(np.uint32)
    want = oracle.argmax_rows_bf16(logits)
    assert np.array_equal(got, want)
    assert want[1] == 0 and want[2] == 0 and want[3] == 0 and want[5] == 100 and want[6] == 0
    assert want[7] == 0 and want[8] == 40000
    # a vocabulary that is a multiple of 8 but not the register-resident length: the row is read twice
    short = oracle.f32_to_bf16(rng.integers(-2, 3, size=(5, 4096)).astype(np.float32))
    sampled = torch.zeros(5, dtype=torch.int32, device=device)
    ops.argmax_rows_bf16_into(to_bf16(short, device), sampled)
    assert np.array_equal(sampled.cpu().numpy().view(np.uint32), oracle.argmax_rows_bf16(short))
    odd = workloads.bf16_normal(rng, (3, 1001))
    sampled = torch.zeros(3, dtype=torch.int32, device=device)
    ops.argmax_rows_bf16_into(to_bf16(odd, device), sampled)
    assert np.array_equal(sampled.cpu().numpy().view(np.uint32), oracle.argmax_rows_bf16(odd))


def test_step_metadata_on_device(device):
    batch = workloads.ragged_decode_batch(5, 9, 1, 300, 512, 4)
    tables = batch.block_tables.copy()
    tables[4, :] = 0xFFFFFFFF                                         # an unmapped sequence -> slot -1
    positions = batch.positions(0)
    request_slots = batch.request_slots.copy()
    request_slots[7] = 100                                            # row beyond the table -> slot -1
    token_ids = np.arange(9, dtype=np.uint32)
    sampled = np.arange(100, 109, dtype=np.uint32)
    state = dict(token_ids=to_u32(token_ids, device), positions=to_u32(positions, device),
                 request_slots=to_u32(request_slots, device), tables=to_u32(tables, device),
                 slots=torch.zeros(9, dtype=torch.int64, device=device), sampled=to_u32(sampled, device))
    struct = _abi.DecodeBatch(state["token_ids"].data_ptr(), state["positions"].data_ptr(),
                              state["request_slots"].data_ptr(), state["slots"].data_ptr(), state["tables"].data_ptr(),
                              tables.shape[1], tables.shape[0], 9, 512)
    stream = torch.cuda.current_stream().cuda_stream
    check(library().lfm25_decode_step_metadata(stream, struct, ops._slice(state["sampled"]), 512, 0))
    assert np.array_equal(state["slots"].cpu().numpy(), oracle.physical_slots(tables, request_slots, positions))
    assert np.array_equal(state["token_ids"].cpu().numpy().view(np.uint32), token_ids)
    for step in (1, 2):
        check(library().lfm25_decode_step_metadata(stream, struct, ops._slice(state["sampled"]), 512, 1))
        assert np.array_equal(state["positions"].cpu().numpy().view(np.uint32), positions + step)
        assert np.array_equal(state["slots"].cpu().numpy(),
                              oracle.physical_slots(tables, request_slots, positions + step))
        assert np.array_equal(state["token_ids"].cpu().numpy().view(np.uint32), sampled)


@pytest.mark.parametrize("m,n,k", [(1, 2048, 2048), (128, 512, 2048), (7, 6144, 2048), (128, 2048, 8192)])
def test_bf16_linear_through_cublaslt(device, library_option, m, n, k):
    library_option("bf16_gemm", BF16_GEMM_PATHS["cublaslt"])
    rng = np.random.default_rng(m + n)
    x = workloads.bf16_normal(rng, (m, k))
    weight = workloads.bf16_normal(rng, (n, k), std=0.02)
    blaslt = ops.BlasLt()
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
    blaslt.linear_bf16(to_bf16(x, device), to_bf16(weight, device), out)
    assert_close_bf16(bits_of(out), oracle.linear_bf16(x, weight), 2e-3, 2 ** -7)
    blaslt.close()


@pytest.mark.parametrize("kernel", ["umma", "rows"])
@pytest.mark.parametrize("m,n,k", [(1, 2048, 2048), (128, 512, 2048), (7, 6144, 2048), (128, 2048, 8192),
                                   (33, 16384, 2048), (256, 2048, 2048), (128, 65536, 2048), (33, 3072, 2048),
                                   (128, 6144, 2048), (128, 16384, 2048), (128, 3072, 2048), (128, 2048, 2048)])
def test_bf16_linear_through_tcgen05(device, library_option, kernel, m, n, k):
    """The BF16 sites of the step through this library's tcgen05 kernels (fp32 accumulation, one rounding): the
    weight-major one and the batch-major one, at the batch sizes of the headline step (33 and 128 rows) too."""
    library_option("bf16_gemm", BF16_GEMM_PATHS[kernel])
    rng = np.random.default_rng(m + n + 1)
    x = workloads.bf16_normal(rng, (m, k))
    weight = workloads.bf16_normal(rng, (n, k), std=0.02)
    blaslt = ops.BlasLt()
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
    blaslt.linear_bf16(to_bf16(x, device), to_bf16(weight, device), out)
    torch.cuda.synchronize()
    assert_close_bf16(bits_of(out), oracle.linear_bf16(x, weight), 2e-3, 2 ** -7)
    assert not ops.device_status()[0]
    blaslt.close()

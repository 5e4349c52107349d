"""The bounded device-side waits, made to run out without any fault: with the option ``wait_selftest_drop`` the
kernels that feed a ring through TMA arm one barrier whose copy they never issue, and with ``wait_limit_ns`` set to a
few milliseconds the wait on that barrier gives up quickly.  Contract (the silent-return rule of the reference's
kernels, kernels/attention_async_fast.cu:88-111, applied to a wait that cannot complete): the kernel returns
normally, stores nothing, records the event in the device status words (count, kernel tag), frees what it holds
(TMEM), and the next ordinary launch on the same context is clean and correct."""
import numpy as np
import pytest
import torch

import cases
from conftest import assert_within_oracle, bits_of, to_bf16, to_u32
from lfm25_inference_b200 import _abi, ops, workloads
from oracle import oracle

pytestmark = pytest.mark.gpu

TAG_ATTENTION, TAG_GEMM_UMMA, TAG_GEMM_ROWS = 1, 3, 5
LIMIT_NS = 3_000_000


def fp8_problem(m, n, k):
    rng = np.random.default_rng(m + n + k)
    w = workloads.bf16_normal(rng, (n, k), std=0.02)
    x = workloads.bf16_normal(rng, (m, k))
    wq, wd = oracle.scalar_scale(float(np.abs(oracle.bf16_to_f32(w)).max()))
    xq, xd = oracle.scalar_scale(float(np.abs(oracle.bf16_to_f32(x)).max()))
    return oracle.quantize_bf16_e4m3(x, xq), oracle.quantize_bf16_e4m3(w, wq), xd * wd


@pytest.mark.parametrize("kernel,tag,m,n,k", [
    (_abi.GEMM_KERNEL_WEIGHT_MAJOR, TAG_GEMM_UMMA, 16, 512, 1024),      # four tiles, K split over a cluster
    (_abi.GEMM_KERNEL_WEIGHT_MAJOR, TAG_GEMM_UMMA, 64, 16384, 256),     # one tile per CTA, no split
    (_abi.GEMM_KERNEL_BATCH_MAJOR, TAG_GEMM_ROWS, 16, 512, 1024),
    (_abi.GEMM_KERNEL_BATCH_MAJOR, TAG_GEMM_ROWS, 200, 4096, 256)])
def test_gemm_wait_runs_out_and_the_next_launch_is_clean(device, library_option, kernel, tag, m, n, k):
    x_codes, w_codes, scale = fp8_problem(m, n, k)
    x = torch.from_numpy(x_codes).to(device)
    w = torch.from_numpy(w_codes).to(device)
    blaslt = ops.BlasLt()
    blaslt.set_gemm_tuning(kernel=kernel)
    assert ops.device_status()[0] == 0
    out = torch.full((m, n), 3.0, dtype=torch.bfloat16, device=device)
    library_option("wait_limit_ns", LIMIT_NS)
    library_option("wait_selftest_drop", 1)
    blaslt.linear_fp8_scaled(x, w, out, scale)
    torch.cuda.synchronize()                      # returns: nothing hangs, nothing faults
    count, last_tag, _, _ = ops.device_status()
    assert count >= 1 and last_tag == tag
    assert torch.all(out == 3.0)                  # no CTA stored a sum with a term missing
    library_option("wait_selftest_drop", 0)
    library_option("wait_limit_ns", 1_000_000_000)
    blaslt.linear_fp8_scaled(x, w, out, scale)    # TMEM was freed: the same kernel runs again at once
    _, exact = oracle.linear_fp8(x_codes, w_codes, scale, want_exact=True)
    assert_within_oracle(bits_of(out), exact)
    assert ops.device_status()[0] == 0
    blaslt.close()


def test_attention_wait_runs_out_and_the_next_launch_is_clean(device, library_option):
    case = cases.single_context_case(128)
    arena = ops.PagedKvArena(to_bf16(case["key_cache"], device), to_bf16(case["value_cache"], device))
    inputs = ops.FastRaggedAttentionInput(
        query=to_bf16(case["query"], device), arena=arena, block_tables=to_u32(case["block_tables"], device),
        block_table_stride=case["block_tables"].shape[1], request_slots=to_u32(case["request_slots"], device),
        position_ids=to_u32(case["position_ids"], device))
    assert ops.device_status()[0] == 0
    output = torch.full_like(inputs.query, 5.0)
    library_option("wait_limit_ns", LIMIT_NS)
    library_option("wait_selftest_drop", 1)
    ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, output)
    torch.cuda.synchronize()
    count, last_tag, _, _ = ops.device_status()
    assert count == 8 and last_tag == TAG_ATTENTION          # one CTA per KV head, each gave up once
    assert torch.all(output == 5.0)
    library_option("wait_selftest_drop", 0)
    library_option("wait_limit_ns", 1_000_000_000)
    ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, output)
    _, exact = oracle.paged_ragged_attention(case["query"], case["key_cache"], case["value_cache"],
                                             case["block_tables"], case["request_slots"], case["position_ids"],
                                             want_exact=True)
    assert_within_oracle(bits_of(output), exact)
    assert ops.device_status()[0] == 0


def test_options_are_validated():
    from lfm25_inference_b200 import Lfm25Error
    with pytest.raises(Lfm25Error):
        ops.set_option("no_such_option", 1)
    with pytest.raises(Lfm25Error):
        ops.set_option("wait_limit_ns", 0)
    with pytest.raises(Lfm25Error):
        ops.set_option("fp8_gemm_path", 9)
    assert ops.get_option("wait_selftest_drop") == 0

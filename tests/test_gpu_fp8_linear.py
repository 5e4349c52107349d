"""Parity of the FP8 (E4M3) linear (C ABI) with the CPU oracle.

The op is Y = bf16(output_scale * Xq Wq^T) on E4M3 codes with fp32 accumulation.  Every product of two E4M3
values is exact in fp32 and only the order of the fp32 sum differs between implementations, so the tolerance
against the fp64 oracle on the same codes is |y - y*| <= 2e-2 + 1e-2 |y*| and cosine >= 0.9999."""
import os

import numpy as np
import pytest
import torch

import cases

from conftest import FP8_GEMM_PATHS, assert_close_bf16, assert_within_oracle, bits_of, to_bf16
from lfm25_inference_b200 import Lfm25Error, ops, workloads
from oracle import oracle

pytestmark = pytest.mark.gpu


def codes_tensor(codes, device):
    return torch.from_numpy(np.ascontiguousarray(codes)).to(device)


def run_linear(x_codes, w_codes, scale, device):
    m, n = x_codes.shape[0], w_codes.shape[0]
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
    ops.linear_fp8_scaled_into(codes_tensor(x_codes, device), codes_tensor(w_codes, device), out, scale)
    return bits_of(out)


def test_exact_32(device):
    # src/cuda/tests/blaslt_fp8.rs:25-57: +-1.0 codes, M=1, N=16, K=32 -> every output exactly 32.0
    x = np.array([0x38 if i % 2 == 0 else 0xB8 for i in range(32)], dtype=np.uint8).reshape(1, 32)
    w = np.array([0x38 if i % 2 == 0 else 0xB8 for i in range(16 * 32)], dtype=np.uint8).reshape(16, 32)
    assert np.all(oracle.bf16_to_f32(run_linear(x, w, 1.0, device)) == 32.0)
    # the same identity on a shape that takes the tensor-core path
    x = np.tile(x, (3, 8))
    w = np.tile(w, (4, 8))
    assert np.all(oracle.bf16_to_f32(run_linear(x, w, 1.0, device)) == 256.0)


def quantised_problem(seed, m, n, k):
    """Weights ~ N(0, 0.02) and activations ~ N(0, 1), each quantised per tensor with scale amax / 448."""
    rng = np.random.default_rng(seed)
    w = workloads.bf16_normal(rng, (n, k), std=0.02)
    x = workloads.bf16_normal(rng, (m, k))
    wq, wd = oracle.scalar_scale(float(np.abs(oracle.bf16_to_f32(w)).max()))
    xq, xd = oracle.scalar_scale(float(np.abs(oracle.bf16_to_f32(x)).max()))
    return x, oracle.quantize_bf16_e4m3(x, xq), oracle.quantize_bf16_e4m3(w, wq), (xq, xd), (wq, wd)


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k", [(2048, 2048), (512, 8192), (1024, 128), (16, 256)])
def test_stream_path_against_oracle(device, m, n, k):
    _, x_codes, w_codes, (_, xd), (_, wd) = quantised_problem(m * 1000 + n + k, m, n, k)
    got = run_linear(x_codes, w_codes, xd * wd, device)
    _, exact = oracle.linear_fp8(x_codes, w_codes, xd * wd, want_exact=True)
    assert_within_oracle(got, exact)
    # tighter: the only differences are fp32 summation order and the final rounding
    want = oracle.bf16_to_f32(oracle.f32_to_bf16(exact.astype(np.float32))).astype(np.float64)
    assert np.abs(oracle.bf16_to_f32(got) - want).max() <= np.abs(exact).max() * 2 ** -7


@pytest.mark.parametrize("path", ["umma", "stream", "rows"])
@pytest.mark.parametrize("m", [1, 9, 16, 17, 31, 32, 48, 64, 100, 128, 129, 200, 256])
@pytest.mark.parametrize("n,k", [(128, 128), (256, 1024), (2048, 2048), (512, 8192)])
def test_kernel_paths_against_oracle(device, library_option, path, m, n, k):
    """The fast kernels on the shapes they accept (the option only selects among valid paths)."""
    if path == "stream" and m > 8:
        pytest.skip("the streaming kernel covers M <= 8")
    library_option("fp8_gemm_path", FP8_GEMM_PATHS[path])
    _, x_codes, w_codes, (_, xd), (_, wd) = quantised_problem(m * 31 + n + k, m, n, k)
    got = run_linear(x_codes, w_codes, xd * wd, device)
    _, exact = oracle.linear_fp8(x_codes, w_codes, xd * wd, want_exact=True)
    assert_within_oracle(got, exact)
    want = oracle.bf16_to_f32(oracle.f32_to_bf16(exact.astype(np.float32))).astype(np.float64)
    assert np.abs(oracle.bf16_to_f32(got) - want).max() <= np.abs(exact).max() * 2 ** -7
    assert ops.device_status()[0] == 0


def test_paths_agree_bit_for_bit_on_exact_sums(device, library_option):
    """With +-1.0 / +-0.5 codes every partial sum is exact in fp32, so all kernels must return identical bits."""
    rng = np.random.default_rng(4)
    choices = np.array([0x38, 0xB8, 0x30, 0xB0, 0x00], dtype=np.uint8)
    x = choices[rng.integers(0, 5, size=(24, 1024))]
    w = choices[rng.integers(0, 5, size=(256, 1024))]
    results = []
    for path in ("generic", "stream", "umma", "rows"):
        library_option("fp8_gemm_path", FP8_GEMM_PATHS[path])
        results.append(run_linear(x, w, 0.25, device))
    assert all(np.array_equal(results[0], other) for other in results[1:])
    assert np.array_equal(results[0], oracle.linear_fp8(x, w, 0.25))


@pytest.mark.parametrize("path", ["umma", "rows"])
def test_weight_stream_hint_does_not_change_a_bit(device, library_option, path):
    """The L2 evict-first hint on the weight tiles (switch `weights_evict_first`) is a cache policy: the same launch
    with and without it returns identical bits, through a handle (K split over a cluster) and without one."""
    library_option("fp8_gemm_path", FP8_GEMM_PATHS[path])
    _, x_codes, w_codes, (_, xd), (_, wd) = quantised_problem(77, 96, 2048, 4096)
    x_t, w_t = codes_tensor(x_codes, device), codes_tensor(w_codes, device)
    blaslt = ops.BlasLt()
    results = []
    for hint in (1, 0):
        library_option("weights_evict_first", hint)
        out = torch.zeros((96, 2048), dtype=torch.bfloat16, device=device)
        blaslt.linear_fp8_scaled(x_t, w_t, out, xd * wd)
        results.append((bits_of(out), run_linear(x_codes, w_codes, xd * wd, device)))
    assert np.array_equal(results[0][0], results[1][0]) and np.array_equal(results[0][1], results[1][1])
    assert ops.device_status()[0] == 0
    blaslt.close()


@pytest.mark.parametrize("m", [1, 8, 16, 100, 128, 256])
@pytest.mark.parametrize("n,k", [(2048, 8192), (256, 4096), (16384, 2048), (6144, 2048)])
def test_blaslt_handle_split_k(device, m, n, k):
    """The handle's exchange buffer lets problems with few weight tiles split K over a cluster of CTAs; calling
    repeatedly (and then the handle-free entry point, which never splits) has to keep giving the right answer."""
    blaslt = ops.BlasLt()
    assert blaslt.workspace_size() == 32 * 1024 * 1024
    _, x_codes, w_codes, (_, xd), (_, wd) = quantised_problem(m + n + k, m, n, k)
    _, exact = oracle.linear_fp8(x_codes, w_codes, xd * wd, want_exact=True)
    x_t, w_t = codes_tensor(x_codes, device), codes_tensor(w_codes, device)
    for _ in range(3):
        out = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
        blaslt.linear_fp8_scaled(x_t, w_t, out, xd * wd)
        assert_within_oracle(bits_of(out), exact)
    stateless = run_linear(x_codes, w_codes, xd * wd, device)
    assert_within_oracle(stateless, exact)
    assert ops.device_status()[0] == 0
    blaslt.close()


@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (4, 64, 128), (3, 17, 100), (5, 40, 2048 + 16), (128, 256, 512),
                                   (300, 128, 256)])
def test_other_shapes_against_oracle(device, m, n, k):
    _, x_codes, w_codes, (_, xd), (_, wd) = quantised_problem(n * 7 + k, m, n, k)
    got = run_linear(x_codes, w_codes, xd * wd, device)
    _, exact = oracle.linear_fp8(x_codes, w_codes, xd * wd, want_exact=True)
    assert_within_oracle(got, exact)


def test_quantise_then_linear_error_is_bounded(device):
    # src/cuda/tests/blaslt_fp8.rs:85-167: NRMSE < 0.08 and cosine > 0.995 against the bf16 product
    m, n, k = 4, 64, 128
    x, x_codes, w_codes, x_scale, w_scale = quantised_problem(3, m, n, k)
    out = ops.linear_fp8_e4m3(to_bf16(x, device), codes_tensor(w_codes, device), x_scale, w_scale)
    got = oracle.bf16_to_f32(bits_of(out)).astype(np.float64)
    table = oracle.e4m3_decode_table().astype(np.float64)
    dense = oracle.bf16_to_f32(x).astype(np.float64) @ (table[w_codes] * w_scale[1]).T
    nrmse = np.sqrt(np.mean((got - dense) ** 2)) / np.sqrt(np.mean(dense ** 2))
    cosine = float((got * dense).sum() / (np.linalg.norm(got) * np.linalg.norm(dense)))
    assert nrmse < 0.08 and cosine > 0.995


@pytest.mark.parametrize("name,n,k", [("gate_up", 16384, 2048), ("down", 2048, 8192), ("lm_head", 65536, 2048)])
@pytest.mark.parametrize("m", [1, 8, 32, 128, 256])
def test_model_shapes(device, name, n, k, m):
    """The three decode GEMM sites at full size; the oracle checks every batch row on a sample of output
    columns, and independence of the batch rows ties the rest: a row computed inside a batch of M must agree
    with the same row computed alone (another kernel may serve M = 1, so agreement is to one bf16 step)."""
    _, x_codes, w_codes, (_, xd), (_, wd) = quantised_problem(n + m, m, n, k)
    got = run_linear(x_codes, w_codes, xd * wd, device)
    columns = np.random.default_rng(0).choice(n, size=512, replace=False)
    _, exact = oracle.linear_fp8(x_codes, np.ascontiguousarray(w_codes[columns]), xd * wd, want_exact=True)
    assert_within_oracle(got[:, columns], exact)
    single = run_linear(x_codes[m - 1:m], w_codes, xd * wd, device)
    assert_close_bf16(single[0], got[m - 1], 1e-3, 2 ** -7)


def test_shape_checks(device):
    x = torch.zeros((2, 128), dtype=torch.uint8, device=device)
    w = torch.zeros((16, 128), dtype=torch.uint8, device=device)
    out = torch.zeros((2, 16), dtype=torch.bfloat16, device=device)
    with pytest.raises(Lfm25Error, match="K mismatch"):
        ops.linear_fp8_scaled_into(x, torch.zeros((16, 64), dtype=torch.uint8, device=device), out, 1.0)
    with pytest.raises(Lfm25Error, match="output storage too small"):
        ops.linear_fp8_scaled_into(x, w, out[:1], 1.0)
    with pytest.raises(Lfm25Error, match="finite and positive"):
        ops.linear_fp8_scaled_into(x, w, out, 0.0)
    with pytest.raises(Lfm25Error, match="Block32"):
        ops.linear_fp8_scaled_into(x, w, out, 1.0, scale_mode=1)


@pytest.mark.parametrize("e4m3_output", [True, False])
@pytest.mark.parametrize("m", [1, 5, 16, 33, 128, 200, 256])
@pytest.mark.parametrize("intermediate,k", [(8192, 2048), (256, 512), (64, 128)])
@pytest.mark.parametrize("kernel", ["umma", "rows"])
def test_gated_linear_equals_linear_then_silu_mul(device, library_option, kernel, m, intermediate, k, e4m3_output):
    """The packed Gate/Up linear with SiLU(gate) * up in its epilogue: bit for bit what the same GEMM kernel followed
    by the SiLU * Up kernel produces (src/model/decode_executor.rs:378-402 as two launches), and within the FP8
    tolerance of the oracle's restatement of those two ops."""
    library_option("fp8_gemm_path", FP8_GEMM_PATHS[kernel])    # the two-launch route through the same GEMM kernel
    _, x_codes, w_codes, (_, xd), (_, wd) = quantised_problem(m * 7 + intermediate + k, m, 2 * intermediate, k)
    x_device, w_device = codes_tensor(x_codes, device), codes_tensor(w_codes, device)
    activation_scale = 448.0 / 6.0
    blaslt = ops.BlasLt()
    packed = torch.zeros((m, 2 * intermediate), dtype=torch.bfloat16, device=device)
    ops.linear_fp8_scaled_into(x_device, w_device, packed, xd * wd)
    if e4m3_output:
        want = torch.zeros((m, intermediate), dtype=torch.uint8, device=device)
        ops.silu_mul_packed_bf16_to_e4m3_into(packed, want, activation_scale)
        got = torch.full((m, intermediate), 0x55, dtype=torch.uint8, device=device)
        blaslt.linear_fp8_silu_mul(x_device, w_device, got, xd * wd, activation_scale)
        assert np.array_equal(got.cpu().numpy(), want.cpu().numpy())
    else:
        want = torch.zeros((m, intermediate), dtype=torch.bfloat16, device=device)
        ops.silu_mul_packed_bf16_into(packed, want)
        got = torch.zeros((m, intermediate), dtype=torch.bfloat16, device=device)
        blaslt.linear_fp8_silu_mul(x_device, w_device, got, xd * wd)
        assert np.array_equal(bits_of(got), bits_of(want))
        # against the oracle: projections from the same codes, then its SiLU * Up
        projected = oracle.linear_fp8(x_codes, w_codes, xd * wd)
        activated, _ = oracle.silu_mul_packed(projected, 1.0)
        assert_close_bf16(bits_of(got), activated, atol=2e-2, rtol=2e-2)
    assert ops.device_status()[0] == 0
    blaslt.close()


def test_gated_linear_shape_checks(device):
    blaslt = ops.BlasLt()
    x = torch.zeros((4, 128), dtype=torch.uint8, device=device)
    weight = torch.zeros((2 * 100, 128), dtype=torch.uint8, device=device)     # 100 outputs: not a multiple of 8
    out = torch.zeros((4, 100), dtype=torch.uint8, device=device)
    with pytest.raises(Lfm25Error):
        blaslt.linear_fp8_silu_mul(x, weight, out, 1.0, 1.0)
    weight = torch.zeros((2 * 64, 128), dtype=torch.uint8, device=device)
    small = torch.zeros((4, 32), dtype=torch.uint8, device=device)             # output storage too small
    with pytest.raises(Lfm25Error):
        blaslt.linear_fp8_silu_mul(x, weight, small, 1.0, 1.0)
    blaslt.close()


@pytest.fixture(scope="module")
def sweep_weights(device):
    """Full weight matrices of the three sites (built block by block from their seeds), kept on the device."""
    cache = {}

    def get(site):
        if site not in cache:
            blocks = cases.FP8_GEMM_SITES[site][0] // cases.FP8_GEMM_BLOCK
            host = np.concatenate([cases.fp8_gemm_weight_block(site, block) for block in range(blocks)])
            cache[site] = codes_tensor(host, device)
        return cache[site]

    return get


@pytest.mark.parametrize("m", cases.FP8_GEMM_BATCHES)
@pytest.mark.parametrize("site", sorted(cases.FP8_GEMM_SITES))
def test_sweep_points_against_cublaslt(device, sweep_weights, site, m):
    """All 15 points of the decode GEMM sweep through a handle (the kernel the library picks for each) against
    cuBLASLt's E4M3 GEMM -- the reference's BlasLt::linear_fp8_scaled (src/cuda/blaslt/mod.rs:212-298) -- (a) live,
    on the same device buffers, every output element, and (b) from the committed fixture on a sample of columns.
    Both sides round one fp32 sum of exact products to bf16, in different orders: |a - b| <= 2^-7 |b| (one bf16
    step) + 2^-10 max|b| (the fp32 rounding of partial sums is relative to the largest terms, not to a result that
    cancels to almost nothing)."""
    x_codes, scale, columns = cases.fp8_gemm_point(site, m)
    weights = sweep_weights(site)
    n = weights.shape[0]
    blaslt = ops.BlasLt()
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
    blaslt.linear_fp8_scaled(codes_tensor(x_codes, device), weights, out, scale)
    got = bits_of(out)
    padded = np.zeros(((m + 15) // 16 * 16, x_codes.shape[1]), dtype=np.uint8)
    padded[:m] = x_codes
    one = torch.ones((), device=device)
    library = torch._scaled_mm(codes_tensor(padded, device).view(torch.float8_e4m3fn),
                               weights.view(torch.float8_e4m3fn).t(), scale_a=one * scale, scale_b=one,
                               out_dtype=torch.bfloat16)
    want = bits_of(library[:m])
    atol = float(np.abs(oracle.bf16_to_f32(want)).max()) * 2 ** -10
    assert_close_bf16(got, want, atol, 2 ** -7)
    golden_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_b200.npz")
    golden = np.load(golden_path)
    if f"fp8_{site}_{m}" in golden.files:
        assert_close_bf16(got[:, columns], golden[f"fp8_{site}_{m}"], atol, 2 ** -7)
    assert ops.device_status()[0] == 0
    blaslt.close()

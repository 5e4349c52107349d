"""Parity of the FP8 (E4M3) linear (C ABI) with the CPU oracle.

The op is Y = bf16(output_scale * Xq Wq^T) on E4M3 codes with fp32 accumulation.  Every product of two E4M3
values is exact in fp32 and only the order of the fp32 sum differs between implementations, so the tolerance
against the fp64 oracle on the same codes is |y - y*| <= 2e-2 + 1e-2 |y*| and cosine >= 0.9999."""
import numpy as np
import pytest
import torch

from conftest import assert_within_oracle, bits_of, to_bf16
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


@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (4, 64, 128), (3, 17, 100), (5, 40, 2048 + 16), (128, 256, 512)])
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
@pytest.mark.parametrize("m", [1, 8, 32])
def test_model_shapes(device, name, n, k, m):
    """The three decode GEMM sites at full size; the oracle checks every batch row on a sample of output
    columns, and linearity in the batch dimension ties the rest: rows computed at M must equal M = 1."""
    _, x_codes, w_codes, (_, xd), (_, wd) = quantised_problem(n + m, m, n, k)
    got = run_linear(x_codes, w_codes, xd * wd, device)
    columns = np.random.default_rng(0).choice(n, size=512, replace=False)
    _, exact = oracle.linear_fp8(x_codes, np.ascontiguousarray(w_codes[columns]), xd * wd, want_exact=True)
    assert_within_oracle(got[:, columns], exact)
    single = run_linear(x_codes[m - 1:m], w_codes, xd * wd, device)
    assert np.array_equal(single[0], got[m - 1])


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

"""Parity of the E4M3 producers (C ABI): quantisation codes are bit-exact against the CPU oracle and the
reference's kernel; SiLU*Up -> E4M3 is byte-equal to the reference's kernel (same fast exp on the same GPU)
and within one code step of the CPU oracle on at most 0.1 % of the elements."""
import numpy as np
import pytest
import torch

import cases
from conftest import bits_of, to_bf16
from lfm25_inference_b200 import ops, workloads
from oracle import oracle, refkernels

pytestmark = pytest.mark.gpu


def test_known_codes(device):
    # src/cuda/tests/blaslt_fp8.rs:60-82
    values = to_bf16(oracle.f32_to_bf16(np.array([1.0, -1.0, 0.5, -0.5], dtype=np.float32)), device)
    codes = torch.zeros(4, dtype=torch.uint8, device=device)
    ops.quantize_bf16_e4m3_into(values, codes, 1.0)
    assert codes.cpu().tolist() == [0x38, 0xB8, 0x30, 0xB0]


def test_every_bf16_value_quantises_like_the_oracle(device):
    bits = np.arange(65536, dtype=np.uint16)
    finite = np.isfinite(oracle.bf16_to_f32(bits))
    for scale in (1.0, 0.37, 448.0 / 3.0, 9.75):
        codes = torch.zeros(65536, dtype=torch.uint8, device=device)
        ops.quantize_bf16_e4m3_into(to_bf16(bits, device), codes, scale)
        got = codes.cpu().numpy()
        want = oracle.quantize_bf16_e4m3(bits, scale)
        assert np.array_equal(got[finite], want[finite])
        assert np.all((got[~finite] & 0x7F) >= 0x7E)


@pytest.mark.parametrize("shape", [(5, 1000), (1, 7), (3, 2049), (128, 2048), (256, 8192)])
def test_quantize_shapes(device, shape):
    rng = np.random.default_rng(shape[1])
    values = workloads.bf16_normal(rng, shape, std=1.5)
    amax = float(np.abs(oracle.bf16_to_f32(values)).max())
    scale, _ = oracle.scalar_scale(amax)
    # an odd element offset exercises the unaligned path as well
    for offset in (0, 1):
        flat = to_bf16(values, device).reshape(-1)[offset:]
        codes = torch.zeros(flat.numel(), dtype=torch.uint8, device=device)
        ops.quantize_bf16_e4m3_into(flat, codes, scale)
        assert np.array_equal(codes.cpu().numpy(), oracle.quantize_bf16_e4m3(values.reshape(-1)[offset:], scale))
        if refkernels.available() and offset == 0:
            reference = torch.zeros_like(codes)
            refkernels.quantize_bf16_e4m3(flat, reference, scale)
            assert torch.equal(codes, reference)


@pytest.mark.parametrize("rows,width", [(5, 1000), (2, 7), (1, 8192), (128, 8192)])
def test_silu_mul(device, rows, width):
    rng = np.random.default_rng(width)
    packed_bits = workloads.bf16_normal(rng, (rows, 2 * width), std=2.0)
    packed = to_bf16(packed_bits, device)
    hidden = torch.zeros((rows, width), dtype=torch.bfloat16, device=device)
    ops.silu_mul_packed_bf16_into(packed, hidden)
    codes = torch.zeros((rows, width), dtype=torch.uint8, device=device)
    ops.silu_mul_packed_bf16_to_e4m3_into(packed, codes, 9.75)
    # src/ops/silu_mul.rs:177-205: fused == unfused pipeline byte for byte
    unfused = torch.zeros_like(codes)
    ops.quantize_bf16_e4m3_into(hidden, unfused, 9.75)
    assert torch.equal(codes, unfused)
    want_hidden, want_codes = oracle.silu_mul_packed(packed_bits, 9.75)
    differing = bits_of(hidden) != want_hidden
    assert differing.mean() <= 1e-3
    table = oracle.e4m3_decode_table()
    got_codes = codes.cpu().numpy()
    mismatch = got_codes != want_codes
    assert mismatch.mean() <= 1e-3
    if mismatch.any():
        step = np.abs(table[got_codes[mismatch]] - table[want_codes[mismatch]])
        assert np.all(step <= np.abs(table[want_codes[mismatch]]) * 0.126 + 2 ** -9)
    if refkernels.available():
        ref_hidden = torch.zeros_like(hidden)
        refkernels.silu_mul_packed_bf16(packed, ref_hidden)
        ref_codes = torch.zeros_like(codes)
        refkernels.silu_mul_packed_bf16_to_e4m3(packed, ref_codes, 9.75)
        assert torch.equal(hidden, ref_hidden) and torch.equal(codes, ref_codes)

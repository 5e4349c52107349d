"""Parity of the batch-major tcgen05 GEMM (the batch on the TMEM lanes, n_tile weight rows per CTA) with the CPU
oracle, under the tile choices its policy can make: every n_tile granularity, ragged last tiles, split K through
the exchange buffer, one and two batch tiles, batch slices, one to four issuing warps, shallow and deep rings, E4M3 and BF16, plain and gated epilogues.

Tolerances are the repository's: against the fp64 oracle on the same inputs |y - y*| <= 2e-2 + 1e-2 |y*| and
cosine >= 0.9999 (E4M3: every product is exact in fp32, only the order of the sum differs); BF16 against the
oracle's fp32 linear to one bf16 step (atol 2e-3, rtol 2^-7); gated outputs bit for bit against the two-launch
route through the same kernel."""
import numpy as np
import pytest
import torch

from conftest import BF16_GEMM_PATHS, FP8_GEMM_PATHS, assert_close_bf16, assert_within_oracle, bits_of, to_bf16
from lfm25_inference_b200 import _abi, ops, workloads
from oracle import oracle

pytestmark = pytest.mark.gpu


def codes(array, device):
    return torch.from_numpy(np.ascontiguousarray(array)).to(device)


def fp8_problem(seed, m, n, k):
    rng = np.random.default_rng(seed)
    w = workloads.bf16_normal(rng, (n, k), std=0.02)
    x = workloads.bf16_normal(rng, (m, k))
    wq, wd = oracle.scalar_scale(float(np.abs(oracle.bf16_to_f32(w)).max()))
    xq, xd = oracle.scalar_scale(float(np.abs(oracle.bf16_to_f32(x)).max()))
    return oracle.quantize_bf16_e4m3(x, xq), oracle.quantize_bf16_e4m3(w, wq), xd * wd


@pytest.fixture
def blaslt():
    handle = ops.BlasLt()
    yield handle
    handle.close()


TILINGS = [dict(n_tile=16), dict(n_tile=64, issuers=1), dict(n_tile=112, issuers=2), dict(n_tile=256),
           dict(n_tile=128, splits=2), dict(n_tile=128, splits=5, issuers=4, shared_memory_bytes=200 * 1024),
           dict(n_tile=64, splits=8), dict(n_tile=112, splits=3, stages=2),
           dict(n_tile=128, stages=12, shared_memory_bytes=200 * 1024), dict(n_tile=96, stages=1, issuers=4),
           dict(n_tile=64, batch_slices=4), dict(n_tile=128, splits=2, batch_slices=2, issuers=4),
           dict(n_tile=224, batch_slices=3, stages=4), dict(n_tile=48, batch_slices=8, splits=4)]


@pytest.mark.parametrize("tiling", TILINGS, ids=lambda t: "-".join(f"{k}{v}" for k, v in t.items()))
@pytest.mark.parametrize("m", [1, 33, 128, 129, 256])
@pytest.mark.parametrize("n,k", [(2048, 2048), (1040, 1024), (512, 8192)])
def test_fp8_tilings_against_oracle(device, blaslt, tiling, m, n, k):
    """n = 1040 = 65 * 16 leaves a ragged last tile for every n_tile but 16; k = 8192 makes uneven K splits."""
    x_codes, w_codes, scale = fp8_problem(m * 13 + n + k, m, n, k)
    _, exact = oracle.linear_fp8(x_codes, w_codes, scale, want_exact=True)
    blaslt.set_gemm_tuning(kernel=_abi.GEMM_KERNEL_BATCH_MAJOR, **tiling)
    out = torch.full((m + 1, n), 7.0, dtype=torch.bfloat16, device=device)      # one guard row behind the output
    for _ in range(2):       # twice: the exchange buffer is reused
        blaslt.linear_fp8_scaled(codes(x_codes, device), codes(w_codes, device), out[:m], scale)
    assert_within_oracle(bits_of(out[:m]), exact)
    want = oracle.bf16_to_f32(oracle.f32_to_bf16(exact.astype(np.float32))).astype(np.float64)
    assert np.abs(oracle.bf16_to_f32(bits_of(out[:m])) - want).max() <= np.abs(exact).max() * 2 ** -7
    assert torch.all(out[m] == 7.0)
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("splits", [1, 4, 8])
def test_fp8_exact_sums_are_bit_identical_to_the_other_kernels(device, blaslt, library_option, splits):
    """With +-1.0 / +-0.5 codes every partial sum is exact in fp32: any tiling and any K split returns the same bits."""
    rng = np.random.default_rng(splits)
    choices = np.array([0x38, 0xB8, 0x30, 0xB0, 0x00], dtype=np.uint8)
    x = choices[rng.integers(0, 5, size=(150, 2048))]
    w = choices[rng.integers(0, 5, size=(256, 2048))]
    want = oracle.linear_fp8(x, w, 0.25)
    blaslt.set_gemm_tuning(kernel=_abi.GEMM_KERNEL_BATCH_MAJOR, n_tile=128, splits=splits)
    out = torch.zeros((150, 256), dtype=torch.bfloat16, device=device)
    blaslt.linear_fp8_scaled(codes(x, device), codes(w, device), out, 0.25)
    assert np.array_equal(bits_of(out), want)


@pytest.mark.parametrize("m", [1, 8, 32, 128, 256])
@pytest.mark.parametrize("name,n,k", [("gate_up", 16384, 2048), ("down", 2048, 8192), ("lm_head", 65536, 2048)])
def test_fp8_model_shapes_with_the_default_policy(device, blaslt, name, n, k, m):
    """The three E4M3 sites of the decode step at full size under the kernel's own tile policy; the oracle checks
    every batch row on a sample of output columns, including the ragged last tile."""
    x_codes, w_codes, scale = fp8_problem(n + m, m, n, k)
    blaslt.set_gemm_tuning(kernel=_abi.GEMM_KERNEL_BATCH_MAJOR)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
    blaslt.linear_fp8_scaled(codes(x_codes, device), codes(w_codes, device), out, scale)
    columns = np.concatenate([np.random.default_rng(0).choice(n, size=480, replace=False), np.arange(n - 32, n)])
    _, exact = oracle.linear_fp8(x_codes, np.ascontiguousarray(w_codes[columns]), scale, want_exact=True)
    assert_within_oracle(bits_of(out)[:, columns], exact)
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("tiling", [dict(), dict(n_tile=48), dict(n_tile=128, splits=4), dict(n_tile=240)],
                         ids=lambda t: "-".join(f"{k}{v}" for k, v in t.items()) or "policy")
@pytest.mark.parametrize("m,n,k", [(1, 2048, 2048), (33, 3072, 2048), (128, 2048, 2048), (128, 6144, 2048),
                                   (128, 2048, 8192), (200, 1040, 512), (256, 16384, 2048)])
def test_bf16_against_oracle(device, blaslt, tiling, m, n, k):
    rng = np.random.default_rng(m + n + k)
    x = workloads.bf16_normal(rng, (m, k))
    weight = workloads.bf16_normal(rng, (n, k), std=0.02)
    blaslt.set_gemm_tuning(kernel=_abi.GEMM_KERNEL_BATCH_MAJOR, **tiling)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
    blaslt.linear_bf16(to_bf16(x, device), to_bf16(weight, device), out)
    assert_close_bf16(bits_of(out), oracle.linear_bf16(x, weight), 2e-3, 2 ** -7)
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("e4m3_output", [True, False])
@pytest.mark.parametrize("m", [1, 33, 128, 200, 256])
@pytest.mark.parametrize("intermediate,k,n_tile", [(8192, 2048, 0), (8192, 2048, 128), (272, 512, 48), (64, 128, 0)])
def test_bf16_gated_equals_linear_then_silu_mul(device, blaslt, library_option, m, intermediate, k, n_tile,
                                                e4m3_output):
    """The BF16 packed Gate/Up linear with SiLU(gate) * up in its epilogue: bit for bit the same kernel's plain GEMM
    followed by the SiLU * Up kernel (src/model/decode_executor.rs:378-402 as two launches).  intermediate = 272
    with tiles of 24 gate + 24 up rows leaves a ragged last tile."""
    library_option("bf16_gemm", BF16_GEMM_PATHS["rows"])
    rng = np.random.default_rng(m + intermediate + k)
    x = to_bf16(workloads.bf16_normal(rng, (m, k)), device)
    weight = to_bf16(workloads.bf16_normal(rng, (2 * intermediate, k), std=0.02), device)
    # splits=1: the gated form never splits K, and only the same order of the fp32 sum gives the same bits
    blaslt.set_gemm_tuning(kernel=_abi.GEMM_KERNEL_BATCH_MAJOR, n_tile=n_tile, splits=1)
    packed = torch.zeros((m, 2 * intermediate), dtype=torch.bfloat16, device=device)
    blaslt.linear_bf16(x, weight, packed)
    scale = 448.0 / 6.0
    if e4m3_output:
        want = torch.zeros((m, intermediate), dtype=torch.uint8, device=device)
        ops.silu_mul_packed_bf16_to_e4m3_into(packed, want, scale)
        got = torch.full((m, intermediate), 0x55, dtype=torch.uint8, device=device)
        blaslt.linear_bf16_silu_mul(x, weight, got, scale)
        assert np.array_equal(got.cpu().numpy(), want.cpu().numpy())
    else:
        want = torch.zeros((m, intermediate), dtype=torch.bfloat16, device=device)
        ops.silu_mul_packed_bf16_into(packed, want)
        got = torch.zeros((m, intermediate), dtype=torch.bfloat16, device=device)
        blaslt.linear_bf16_silu_mul(x, weight, got)
        assert np.array_equal(bits_of(got), bits_of(want))
    assert ops.device_status()[0] == 0


def test_plan_fills_the_machine(device, blaslt):
    """The tile policy on the model's shapes: Gate/Up (plain and gated) in one wave of 147 CTAs -- the gated one at
    64..128 rows with six ring slots and two issuing warps, the tiling that measured best inside the step; every
    plan keeps the ring a multiple of the issuing warps; the 2048-row sites split K over clusters."""
    assert blaslt.gemm_plan(32, 16384, 2048)["tiles"] == 147
    gated = blaslt.gemm_plan(32, 8192, 2048, gated=True)
    assert (gated["n_tile"], gated["tiles"], gated["splits"]) == (112, 147, 1)
    for m in (64, 96, 128):
        wide = blaslt.gemm_plan(m, 8192, 2048, gated=True)
        assert (wide["n_tile"], wide["tiles"], wide["stages"], wide["issuers"], wide["ctas_per_sm"]) == (112, 147, 6, 2, 1)
        assert wide["smem_bytes"] <= 200 * 1024 + 16 * 1024
    for m in (1, 32, 128, 256):
        for n, k_bytes in ((16384, 2048), (65536, 2048), (2048, 8192), (2048, 4096), (6144, 4096)):
            plan = blaslt.gemm_plan(m, n, k_bytes)
            assert plan["stages"] % plan["issuers"] == 0 and plan["tiles"] * plan["n_tile"] >= n
    down = blaslt.gemm_plan(128, 2048, 8192)
    assert down["splits"] > 1 and down["tiles"] * down["splits"] <= 296


def test_tuning_is_validated(device, blaslt):
    from lfm25_inference_b200 import Lfm25Error
    with pytest.raises(Lfm25Error):
        blaslt.set_gemm_tuning(n_tile=100)
    with pytest.raises(Lfm25Error):
        blaslt.set_gemm_tuning(splits=9)
    with pytest.raises(Lfm25Error):
        blaslt.set_gemm_tuning(kernel=9)
    blaslt.set_gemm_tuning()

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

entry.load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture
def library_option():
    """Sets process-wide switches of the library (lfm25_set_option) for one test and restores them afterwards."""
    from lfm25_inference_b200 import ops
    before = {}

    def set_option(name: str, value: int) -> None:
        before.setdefault(name, ops.get_option(name))
        ops.set_option(name, value)

    yield set_option
    for name, value in before.items():
        ops.set_option(name, value)


FP8_GEMM_PATHS = {"auto": 0, "stream": 1, "umma": 2, "generic": 3, "rows": 4}
BF16_GEMM_PATHS = {"auto": 0, "umma": 1, "cublaslt": 2, "rows": 3}
HYBRID_ATTENTION_KERNELS = {"auto": 0, "umma": 1, "mma": 2}


def to_bf16(bits: np.ndarray, device):
    """uint16 bit patterns -> torch.bfloat16 tensor on `device`."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).to(device).view(torch.bfloat16)


def to_u32(values: np.ndarray, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(values, dtype=np.uint32).view(np.int32).copy()).to(device)


def to_i64(values: np.ndarray, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(values, dtype=np.int64).copy()).to(device)


def bits_of(tensor) -> np.ndarray:
    """torch.bfloat16 tensor -> uint16 bit patterns on the host."""
    import torch
    return tensor.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def assert_close_bf16(actual_bits, expected_bits, atol, rtol):
    """|a - e| <= atol + rtol * |e| element-wise (the reference's src/cuda/testing.rs:23-47)."""
    from oracle import oracle
    actual = oracle.bf16_to_f32(actual_bits).astype(np.float64)
    expected = oracle.bf16_to_f32(expected_bits).astype(np.float64)
    error = np.abs(actual - expected)
    bound = atol + rtol * np.abs(expected)
    worst = int(np.argmax(error - bound))
    assert np.all(error <= bound), (
        f"max violation at flat index {worst}: actual {actual.flat[worst]}, expected {expected.flat[worst]}")


def assert_within_oracle(actual_bits, exact, atol=2e-2, rtol=1e-2, min_cosine=0.9999):
    """Tolerance of this repository against the fp64 oracle: |y - y*| <= 2e-2 + 1e-2 |y*| and cosine >= 0.9999."""
    from oracle import oracle
    actual = oracle.bf16_to_f32(actual_bits).astype(np.float64).reshape(-1)
    exact = np.asarray(exact, dtype=np.float64).reshape(-1)
    error = np.abs(actual - exact)
    assert np.all(error <= atol + rtol * np.abs(exact)), f"max abs error {error.max()}"
    cosine = float(actual @ exact / (np.linalg.norm(actual) * np.linalg.norm(exact) + 1e-300))
    assert cosine >= min_cosine, f"cosine {cosine}"

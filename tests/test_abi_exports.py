"""The C-ABI library loads without a GPU, exports every symbol that include/lfm25_b200.h declares, and
rejects bad arguments on the host before touching the device (the reference's `ensure!` behaviour)."""
import ctypes
import os
import re

import pytest

from lfm25_inference_b200 import _abi
from lfm25_inference_b200._abi import Slice

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    with open(os.path.join(ROOT, "include", "lfm25_b200.h")) as handle:
        text = handle.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lfm25_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    library = _abi.library()
    symbols = declared_symbols()
    assert len(symbols) >= 13
    for name in symbols:
        assert hasattr(library, name), f"{name} is declared but not exported"
        assert name in _abi.PROTOTYPES, f"{name} has no ctypes prototype"
    assert set(_abi.PROTOTYPES) == set(symbols)
    assert b"sm_100a" in library.lfm25_version()


def fake(elements):
    """A non-null 'device pointer' that is never dereferenced: validation fails before any launch."""
    return Slice(0x1000, elements)


def call(function, *arguments):
    code = function(*arguments)
    return code, _abi.library().lfm25_last_error().decode()


def test_kv_write_validation():
    library = _abi.library()
    good = dict(page_size=16, key=fake(512), value=fake(512), key_cache=fake(8192), value_cache=fake(8192),
                slot_mapping=fake(1), num_tokens=1, num_pages=1)

    def launch(**changes):
        fields = {**good, **changes}
        return call(library.lfm25_kv_cache_write_lfm2_bf16, None, _abi.KvCacheWriteLaunch(*fields.values()))

    assert launch(num_tokens=0) == (_abi.ERR_INVALID_ARGUMENT, "KV cache write requires at least one token")
    assert launch(num_pages=0)[0] == _abi.ERR_INVALID_ARGUMENT
    assert launch(key=fake(511)) == (_abi.ERR_BUFFER_TOO_SMALL, "K storage too small")
    assert launch(value_cache=fake(8191)) == (_abi.ERR_BUFFER_TOO_SMALL, "V cache storage too small")
    assert launch(slot_mapping=fake(0))[0] == _abi.ERR_BUFFER_TOO_SMALL
    assert launch(page_size=8, key_cache=fake(1 << 20), value_cache=fake(1 << 20)) == (
        _abi.ERR_INVALID_ARGUMENT, "unsupported KV page size 8")
    assert launch(page_size=32, key_cache=fake(1 << 20), value_cache=fake(1 << 20))[0] == _abi.ERR_UNSUPPORTED
    assert launch(num_tokens=2 ** 62)[0] == _abi.ERR_OVERFLOW
    assert launch(key=Slice(None, 512))[0] == _abi.ERR_NULL_POINTER


def test_attention_validation():
    library = _abi.library()
    good = dict(page_size=16, query=fake(2048), key_cache=fake(8192), value_cache=fake(8192), block_tables=fake(4),
                request_slots=fake(1), position_ids=fake(1), output=fake(2048), num_tokens=1, num_pages=1,
                block_table_stride=4)

    def launch(**changes):
        fields = {**good, **changes}
        return call(library.lfm25_paged_ragged_attention_fast_lfm2_bf16, None,
                    _abi.FastRaggedAttentionLaunch(*fields.values()))

    assert launch(num_tokens=0) == (_abi.ERR_INVALID_ARGUMENT, "fast-exp ragged attention requires tokens")
    assert launch(block_table_stride=0)[0] == _abi.ERR_INVALID_ARGUMENT
    assert launch(block_tables=fake(3)) == (_abi.ERR_BUFFER_TOO_SMALL, "fast-exp ragged block tables too small")
    assert launch(block_tables=fake(6)) == (_abi.ERR_INVALID_ARGUMENT, "fast-exp ragged block tables not row aligned")
    assert launch(output=fake(2047)) == (_abi.ERR_BUFFER_TOO_SMALL, "fast-exp ragged output storage too small")
    assert launch(page_size=32)[0] == _abi.ERR_UNSUPPORTED

    split = dict(page_size=16, query=fake(2048), key_cache=fake(8192), value_cache=fake(8192), block_tables=fake(4),
                 request_slots=fake(1), position_ids=fake(1), partials=fake(32 * 8 * 66), output=fake(2048),
                 num_tokens=1, num_pages=1, block_table_stride=4, num_splits=8)

    def launch_split(**changes):
        fields = {**split, **changes}
        return call(library.lfm25_paged_ragged_attention_splitk_lfm2_bf16, None,
                    _abi.SplitKRaggedAttentionLaunch(*fields.values()))

    assert launch_split(num_splits=1) == (_abi.ERR_INVALID_ARGUMENT, "split-K ragged attention requires 2..=8 splits")
    assert launch_split(num_splits=9)[0] == _abi.ERR_INVALID_ARGUMENT
    code, message = launch_split(partials=fake(32 * 8 * 66 - 1))
    assert code == _abi.ERR_BUFFER_TOO_SMALL and "need 16896, have 16895" in message


def test_fp8_producer_validation():
    library = _abi.library()
    quantize = library.lfm25_quantize_bf16_e4m3
    assert call(quantize, None, fake(4), fake(4), 0, 1.0)[0] == _abi.ERR_INVALID_ARGUMENT
    assert call(quantize, None, fake(3), fake(4), 4, 1.0)[0] == _abi.ERR_BUFFER_TOO_SMALL
    for scale in (0.0, -1.0, float("inf"), float("nan")):
        assert call(quantize, None, fake(4), fake(4), 4, scale) == (
            _abi.ERR_INVALID_ARGUMENT, "invalid FP8 quantization scale")
    fused = library.lfm25_silu_mul_packed_bf16_to_e4m3
    assert call(fused, None, fake(16), fake(8), 0, 8, 1.0)[0] == _abi.ERR_INVALID_ARGUMENT
    assert call(fused, None, fake(15), fake(8), 1, 8, 1.0)[0] == _abi.ERR_BUFFER_TOO_SMALL
    assert call(fused, None, fake(16), fake(8), 1, 8, float("nan"))[0] == _abi.ERR_INVALID_ARGUMENT


def test_fp8_linear_validation():
    library = _abi.library()
    linear = library.lfm25_linear_fp8_scaled

    def launch(m=2, n=16, k=128, mode=0, scale=1.0, x=256, w=2048, out=32):
        return call(linear, None, fake(x), fake(w), fake(out), _abi.Fp8LinearConfig(m, n, k, mode, scale))

    assert launch(m=0) == (_abi.ERR_INVALID_ARGUMENT, "FP8 matmul M must be > 0")
    assert launch(n=0)[0] == _abi.ERR_INVALID_ARGUMENT and launch(k=0)[0] == _abi.ERR_INVALID_ARGUMENT
    assert launch(scale=float("inf")) == (_abi.ERR_INVALID_ARGUMENT, "FP8 output scale must be finite and positive")
    assert launch(mode=1)[0] == _abi.ERR_UNSUPPORTED
    assert launch(mode=1, k=100)[0] == _abi.ERR_INVALID_ARGUMENT      # MXFP8 wants K % 32 == 0
    assert launch(mode=7)[0] == _abi.ERR_INVALID_ARGUMENT
    assert launch(x=255) == (_abi.ERR_BUFFER_TOO_SMALL, "FP8 linear input storage too small: required=256, actual=255")
    assert launch(w=2047)[0] == _abi.ERR_BUFFER_TOO_SMALL and launch(out=31)[0] == _abi.ERR_BUFFER_TOO_SMALL
    assert launch(m=2 ** 40, n=2 ** 40)[0] == _abi.ERR_OVERFLOW


def test_workspace_and_split_policy():
    library = _abi.library()
    # src/ops/attention_async_fast.rs:203-207  splitk_workspace_is_bounded_for_serving_capacity
    assert library.lfm25_splitk_workspace_elements(64) == 64 * 32 * 8 * 66
    assert library.lfm25_splitk_workspace_elements(2 ** 62) == 0
    splits = library.lfm25_splitk_decode_splits
    assert splits(0, 8192, 16) == 1            # src/ops/splitk_policy.rs:20-22
    assert splits(1, 100, 16) == 1             # short contexts never split
    assert splits(1, 8192, 16) == 8            # one long sequence: as many splits as allowed
    assert splits(64, 8192, 16) == 4           # 512 items of up to 8192 tokens: four splits
    assert splits(64, 4096, 16) == 2
    assert splits(32, 4096, 16) == 2
    assert splits(16, 4096, 16) == 4
    assert splits(128, 4096, 16) == 1          # 1024 items, handed out longest first: no split
    assert splits(256, 8192, 16) == 1          # enough items without splitting
    assert splits(8, 256, 16) == 2             # never below 8 pages per split
    assert splits(4, 8192, 32) == 1            # page size 32 is not built
    for tokens in (1, 2, 8, 16, 32, 64, 128):
        for context in (16, 512, 2048, 8192):
            assert splits(tokens, context, 16) in (1, 2, 4, 8)


def test_one_kernel_dispatch_and_options():
    """The one-kernel / two-launch choice (the reference's table: src/ops/mok_dispatch.rs:7-27, tests :29-54) and
    the option table: unknown names and values out of range are refused, a set value reads back."""
    library = _abi.library()
    prefers = library.lfm25_decode_one_kernel_preferred
    assert library.lfm25_set_option(b"pdl", 1) == _abi.OK
    assert prefers(16, 64, 16) == 1 and prefers(16, 128, 32) == 1 and prefers(16, 4096, 32) == 1
    assert prefers(16, 4096, 128) == 1               # a long maximum context in a large batch: a ragged batch
    assert prefers(16, 40, 1) == 0                   # the dependent launch hides the boundary: two launches
    assert prefers(16, 16, 128) == 0 and prefers(16, 2048, 128) == 0 and prefers(16, 4096, 64) == 0
    assert prefers(16, 512, 16) == 0 and prefers(16, 64, 8) == 0
    assert prefers(32, 16, 8) == 0 and prefers(16, 16, 0) == 0
    try:
        assert library.lfm25_set_option(b"pdl", 0) == _abi.OK
        # without it, the reference's own thresholds
        assert prefers(16, 16, 128) == 1 and prefers(16, 32, 32) == 1 and prefers(16, 64, 8) == 1
        assert prefers(16, 32, 33) == 0 and prefers(16, 64, 9) == 0 and prefers(16, 65, 1) == 0
    finally:
        assert library.lfm25_set_option(b"pdl", 1) == _abi.OK
    value = ctypes.c_int64(-1)
    assert library.lfm25_get_option(b"fused_append", ctypes.byref(value)) == _abi.OK and value.value == 2
    assert library.lfm25_set_option(b"fused_append", 3) == _abi.ERR_INVALID_ARGUMENT
    assert library.lfm25_set_option(b"no_such_switch", 1) == _abi.ERR_INVALID_ARGUMENT
    assert library.lfm25_get_option(b"no_such_switch", ctypes.byref(value)) == _abi.ERR_INVALID_ARGUMENT
    assert library.lfm25_set_option(None, 1) == _abi.ERR_NULL_POINTER
    assert library.lfm25_set_option(b"decode_splits", 4) == _abi.OK
    assert library.lfm25_splitk_decode_splits(128, 4096, 16) == 4
    assert library.lfm25_set_option(b"decode_splits", 0) == _abi.OK
    assert library.lfm25_splitk_decode_splits(128, 4096, 16) == 1


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_abi, "_library", None)
    monkeypatch.setattr(_abi, "LIBRARY_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _abi.library()

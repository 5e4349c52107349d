"""Launcher for the reference's own CUDA kernels (``oracle/_ref/*.cubin``).  TEST INFRASTRUCTURE ONLY.

``make -C oracle ref`` compiles the reference project's unmodified ``kernels/*.cu`` for sm_100a.  This
module loads those images with the CUDA driver API and launches them with the grid and block sizes of
the reference's Rust wrappers, so that the new kernels can be compared with the reference's results
on the same device buffers (and timed next to them).  It needs a GPU; nothing in the product imports it.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")
_BLOCK = 256

_driver = None
_modules: dict[str, ctypes.c_void_p] = {}
_functions: dict[tuple[str, str], ctypes.c_void_p] = {}


def available() -> bool:
    return os.path.exists(os.path.join(_REF, "attention_async_fast.cubin"))


def _cuda():
    global _driver
    if _driver is None:
        _driver = ctypes.CDLL("libcuda.so.1")
        _driver.cuLaunchKernel.argtypes = [ctypes.c_void_p] + [ctypes.c_uint] * 6 + [
            ctypes.c_uint, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
    return _driver


def _check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with CUDA driver error {code}")


def _function(module: str, name: str) -> ctypes.c_void_p:
    key = (module, name)
    if key not in _functions:
        torch.zeros(1, device="cuda")  # makes the primary context current
        if module not in _modules:
            with open(os.path.join(_REF, module + ".cubin"), "rb") as handle:
                image = handle.read()
            loaded = ctypes.c_void_p()
            _check(_cuda().cuModuleLoadData(ctypes.byref(loaded), image), f"cuModuleLoadData({module})")
            _modules[module] = loaded
        function = ctypes.c_void_p()
        _check(_cuda().cuModuleGetFunction(ctypes.byref(function), _modules[module], name.encode()),
               f"cuModuleGetFunction({name})")
        _functions[key] = function
    return _functions[key]


def _launch(module: str, name: str, blocks: int, arguments: list, block: int = _BLOCK) -> None:
    function = _function(module, name)
    holders = []
    for argument in arguments:
        if isinstance(argument, torch.Tensor):
            holders.append(ctypes.c_void_p(argument.data_ptr()))
        else:
            holders.append(argument)
    pointers = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.pointer(h), ctypes.c_void_p) for h in holders])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _check(_cuda().cuLaunchKernel(function, blocks, 1, 1, block, 1, 1, 0, stream, pointers, None),
           f"cuLaunchKernel({name})")


_sz = ctypes.c_size_t


def kv_cache_write(key, value, key_cache, value_cache, slot_mapping) -> None:
    tokens = key.shape[0]
    _launch("kv_cache", "kv_cache_write_lfm2_bf16_ps16", tokens,
            [key, value, key_cache, value_cache, slot_mapping, _sz(tokens), _sz(key_cache.shape[0])])


def qk_norm_rope_kv_write_decode(query, key, value, query_norm, key_norm, inv_freq, position_ids, slot_mapping,
                                 key_cache, value_cache, eps: float) -> None:
    tokens = query.shape[0]
    _launch("qk_postprocess", "qk_norm_rope_kv_write_decode_ps16", tokens,
            [query, key, value, query_norm, key_norm, inv_freq, position_ids, slot_mapping, key_cache, value_cache,
             _sz(tokens), _sz(key_cache.shape[0]), ctypes.c_float(eps)])


def paged_ragged_attention_precise(query, key_cache, value_cache, block_tables, request_slots, position_ids,
                                   output) -> None:
    """The reference's own test oracle: kernels/attention.cu `paged_ragged_gqa_lfm2_bf16_ps16`."""
    tokens = query.shape[0]
    stride = block_tables.shape[1]
    _launch("attention", "paged_ragged_gqa_lfm2_bf16_ps16", tokens * 8,
            [query, key_cache, value_cache, block_tables, request_slots, position_ids, output, _sz(tokens),
             _sz(key_cache.shape[0]), _sz(stride), _sz(stride)])


def paged_ragged_attention_fast(query, key_cache, value_cache, block_tables, request_slots, position_ids,
                                output) -> None:
    tokens = query.shape[0]
    rows, stride = block_tables.shape
    _launch("attention_async_fast", "paged_ragged_gqa_lfm2_bf16_async_fast_ps16", tokens * 8,
            [query, key_cache, value_cache, block_tables, request_slots, position_ids, output, _sz(tokens),
             _sz(key_cache.shape[0]), _sz(stride), _sz(rows)])


def paged_ragged_attention_splitk(query, key_cache, value_cache, block_tables, request_slots, position_ids,
                                  partials, output, num_splits: int) -> None:
    tokens = query.shape[0]
    rows, stride = block_tables.shape
    _launch("attention_async_fast", "paged_ragged_gqa_lfm2_bf16_splitk_ps16", tokens * 8 * num_splits,
            [query, key_cache, value_cache, block_tables, request_slots, position_ids, partials, _sz(tokens),
             _sz(key_cache.shape[0]), _sz(stride), _sz(rows), ctypes.c_uint32(num_splits)])
    _launch("attention_async_fast", "merge_ragged_gqa_lfm2_bf16_splitk", tokens * 8,
            [partials, output, _sz(tokens), ctypes.c_uint32(num_splits)])


def quantize_bf16_e4m3(values, output, scale: float) -> None:
    numel = values.numel()
    blocks = max(1, min((numel // 2 + _BLOCK - 1) // _BLOCK, 65535))
    _launch("fp8_quantize", "quantize_bf16_e4m3", blocks, [values, output, _sz(numel), ctypes.c_float(scale)])


def silu_mul_packed_bf16(packed, output) -> None:
    rows, width = packed.shape
    blocks = max(1, min((rows * width // 4 + _BLOCK - 1) // _BLOCK, 65535))
    _launch("silu_mul", "silu_mul_packed_bf16", blocks, [packed, output, _sz(rows), _sz(width // 2)])


def silu_mul_packed_bf16_to_e4m3(packed, output, scale: float) -> None:
    rows, width = packed.shape
    blocks = max(1, min((rows * width // 4 + _BLOCK - 1) // _BLOCK, 65535))
    _launch("silu_mul", "silu_mul_packed_bf16_to_e4m3", blocks,
            [packed, output, _sz(rows), _sz(width // 2), ctypes.c_float(scale)])


def hybrid_ragged_attention(query, current_key, current_value, key_cache, value_cache, block_tables, request_slots,
                            position_ids, segment_offsets, output) -> None:
    """kernels/attention.cu `hybrid_ragged_gqa_lfm2_bf16_ps16` (the reference's mixed prefill / decode attention),
    grid = tokens * 8 as in src/cuda/kernels/attention.rs:211."""
    tokens = query.shape[0]
    _launch("attention", "hybrid_ragged_gqa_lfm2_bf16_ps16", tokens * 8,
            [query, current_key, current_value, key_cache, value_cache, block_tables, request_slots, position_ids,
             segment_offsets, output, _sz(tokens), _sz(key_cache.shape[0]), _sz(block_tables.shape[1]),
             _sz(segment_offsets.numel() - 1)])


def short_conv_segmented(projected, weight, states, segment_offsets, segment_slots, output) -> None:
    """kernels/short_conv.cu `short_conv_segmented_lfm2_bf16` (grid-stride over segments * hidden)."""
    hidden = weight.shape[0]
    segments = segment_slots.numel()
    blocks = max(1, min((segments * hidden + _BLOCK - 1) // _BLOCK, 65535))
    _launch("short_conv", "short_conv_segmented_lfm2_bf16", blocks,
            [projected, weight, states, segment_offsets, segment_slots, output, _sz(segments), _sz(hidden),
             _sz(states.shape[0])])


def embedding(token_ids, weight, output) -> None:
    """kernels/embedding.cu `embedding_bf16`, one block per token (src/cuda/kernels/embedding.rs:39-62)."""
    tokens = token_ids.numel()
    _launch("embedding", "embedding_bf16", tokens,
            [token_ids, weight, output, _sz(tokens), _sz(weight.shape[0]), _sz(weight.shape[1])])


def rms_norm(values, weight, output, eps: float) -> None:
    """kernels/rms_norm.cu `rms_norm_bf16`, one block per row (src/cuda/kernels/rms_norm.rs:65-92)."""
    rows, width = values.shape
    _launch("rms_norm", "rms_norm_bf16", rows, [values, weight, output, _sz(rows), _sz(width), ctypes.c_float(eps)])


def residual_rms_norm(residual, update, weight, residual_output, normalized_output, eps: float) -> None:
    """kernels/rms_norm.cu `residual_rms_norm_bf16` (src/cuda/kernels/rms_norm.rs:94-128)."""
    rows, width = residual.shape
    _launch("rms_norm", "residual_rms_norm_bf16", rows,
            [residual, update, weight, residual_output, normalized_output, _sz(rows), _sz(width),
             ctypes.c_float(eps)])


def argmax_rows(values, output) -> None:
    """kernels/sampling.cu `argmax_rows_bf16`, one block per row: the path the reference's dispatch takes for
    more than 16 rows (src/ops/sampling_dispatch.rs:17-60, src/cuda/kernels/sampling.rs:50-71)."""
    rows, columns = values.shape
    _launch("sampling", "argmax_rows_bf16", rows, [values, output, _sz(rows), _sz(columns)])

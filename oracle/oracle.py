"""ctypes front end of the CPU oracle (``lfm25_oracle.c``).  TEST INFRASTRUCTURE ONLY.

The oracle restates the reference runtime's decode-path arithmetic on the CPU.  It exists to
check the CUDA kernels of this repository; the product library never loads it.  Only the test
suite, the smoke check and the CPU-baseline leg of the benchmark import this module.

All arrays are numpy arrays; bf16 tensors travel as ``uint16`` bit patterns and E4M3 tensors
as ``uint8`` codes, so every comparison can be made bit for bit.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblfm25_oracle.so")
_lib = None

_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_size = ctypes.c_size_t


def build() -> str:
    """Compile the oracle (and, where the reference tree is present, its kernels)."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    # the reference checkout: REFERENCE_ROOT, else a directory `reference` beside this repository
    reference_root = os.environ.get("REFERENCE_ROOT") or os.path.normpath(os.path.join(_HERE, "..", "..", "reference"))
    if os.path.isdir(os.path.join(reference_root, "kernels")):
        subprocess.run(["make", "-C", _HERE, "ref", f"REFERENCE_ROOT={reference_root}"],
                       check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        build()
    handle = ctypes.CDLL(_LIB_PATH)
    handle.oracle_e4m3_from_f32.argtypes = [ctypes.c_float]
    handle.oracle_e4m3_from_f32.restype = ctypes.c_uint8
    handle.oracle_e4m3_to_f32.argtypes = [ctypes.c_uint8]
    handle.oracle_e4m3_to_f32.restype = ctypes.c_float
    handle.oracle_scalar_scale.argtypes = [ctypes.c_float, ctypes.POINTER(ctypes.c_float),
                                           ctypes.POINTER(ctypes.c_float)]
    handle.oracle_quantize_bf16_e4m3.argtypes = [_u16p, _u8p, _size, ctypes.c_float]
    handle.oracle_silu_mul_packed.argtypes = [_u16p, ctypes.c_void_p, ctypes.c_void_p, _size, _size,
                                              ctypes.c_float]
    handle.oracle_linear_fp8.argtypes = [_u8p, _u8p, _u16p, ctypes.c_void_p, _size, _size, _size,
                                         ctypes.c_float]
    handle.oracle_kv_cache_write.argtypes = [_u16p, _u16p, _u16p, _u16p, _i64p, _size, _size, _size]
    handle.oracle_qk_norm_rope_kv_write_decode.argtypes = [
        _u16p, _u16p, _u16p, _u16p, _u16p, _f32p, _u32p, _i64p, _u16p, _u16p, _size, _size, _size,
        ctypes.c_float]
    handle.oracle_paged_ragged_attention.argtypes = [
        _u16p, _u16p, _u16p, _u32p, ctypes.c_void_p, _u32p, _u16p, ctypes.c_void_p, _size, _size,
        _size, _size, _size]
    handle.oracle_paged_ragged_attention_splitk_partials.argtypes = [
        _u16p, _u16p, _u16p, _u32p, _u32p, _u32p, _f32p, _size, _size, _size, _size, _size,
        ctypes.c_uint32]
    handle.oracle_merge_splitk.argtypes = [_f32p, _u16p, _size, ctypes.c_uint32]
    handle.oracle_physical_slots.argtypes = [_u32p, _u32p, _u32p, _i64p, _size, _size, _size, _size]
    handle.oracle_rms_norm_bf16.argtypes = [_u16p, _u16p, _u16p, _size, _size, ctypes.c_float]
    handle.oracle_residual_rms_norm_bf16.argtypes = [_u16p, _u16p, _u16p, _u16p, _u16p, _size, _size, ctypes.c_float]
    handle.oracle_short_conv_decode_bf16.argtypes = [_u16p, _u16p, _u16p, _u32p, _u16p, _size, _size, _size]
    handle.oracle_short_conv_segmented_bf16.argtypes = [_u16p, _u16p, _u16p, _u32p, _u32p, _u16p, _size, _size, _size]
    handle.oracle_hybrid_ragged_attention.argtypes = [
        _u16p, _u16p, _u16p, _u16p, _u16p, _u32p, _u32p, _u32p, _u32p, _u16p, ctypes.c_void_p, _size, _size, _size,
        _size, _size]
    handle.oracle_argmax_rows_bf16.argtypes = [_u16p, _u32p, _size, _size]
    handle.oracle_linear_bf16.argtypes = [_u16p, _u16p, _u16p, _size, _size, _size]
    handle.oracle_num_threads.restype = ctypes.c_int
    handle.oracle_set_num_threads.argtypes = [ctypes.c_int]
    handle.oracle_set_num_threads.restype = None
    _lib = handle
    return handle


# ----------------------------------------------------------------------------- bf16 helpers


def f32_to_bf16(values) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (``__float2bfloat16_rn``)."""
    array = np.ascontiguousarray(values, dtype=np.float32)
    bits = array.view(np.uint32)
    with np.errstate(over="ignore"):
        rounded = ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    nan = (bits & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    if nan.any():
        rounded[nan] = 0x7FFF
    return rounded.reshape(array.shape)


def bf16_to_f32(bits) -> np.ndarray:
    array = np.ascontiguousarray(bits, dtype=np.uint16)
    return (array.astype(np.uint32) << 16).view(np.float32).reshape(array.shape)


# ----------------------------------------------------------------------------- FP8


def e4m3_from_f32(value: float) -> int:
    return int(lib().oracle_e4m3_from_f32(ctypes.c_float(value)))


def e4m3_to_f32(code: int) -> float:
    return float(lib().oracle_e4m3_to_f32(ctypes.c_uint8(code)))


def e4m3_decode_table() -> np.ndarray:
    return np.array([e4m3_to_f32(code) for code in range(256)], dtype=np.float32)


def scalar_scale(clip_amax: float) -> tuple[float, float]:
    """(quantize_multiplier, dequantize_multiplier) of a per-tensor E4M3 scale."""
    quantize = ctypes.c_float()
    dequantize = ctypes.c_float()
    lib().oracle_scalar_scale(ctypes.c_float(clip_amax), ctypes.byref(quantize), ctypes.byref(dequantize))
    return quantize.value, dequantize.value


def quantize_bf16_e4m3(values_bf16: np.ndarray, scale: float) -> np.ndarray:
    flat = np.ascontiguousarray(values_bf16, dtype=np.uint16).reshape(-1)
    out = np.empty(flat.shape, dtype=np.uint8)
    lib().oracle_quantize_bf16_e4m3(flat, out, flat.size, ctypes.c_float(scale))
    return out.reshape(values_bf16.shape)


def silu_mul_packed(packed_bf16: np.ndarray, scale: float) -> tuple[np.ndarray, np.ndarray]:
    """Returns (hidden bf16 [rows, I], codes uint8 [rows, I]) of a packed [rows, 2I] input."""
    packed = np.ascontiguousarray(packed_bf16, dtype=np.uint16)
    rows, width = packed.shape
    intermediate = width // 2
    hidden = np.empty((rows, intermediate), dtype=np.uint16)
    codes = np.empty((rows, intermediate), dtype=np.uint8)
    lib().oracle_silu_mul_packed(packed, hidden.ctypes.data, codes.ctypes.data, rows, intermediate,
                                 ctypes.c_float(scale))
    return hidden, codes


def linear_fp8(x_codes: np.ndarray, w_codes: np.ndarray, output_scale: float,
               want_exact: bool = False):
    """Y[M,N] = bf16(output_scale * Xq @ Wq^T); optionally also the unrounded float64 result."""
    x = np.ascontiguousarray(x_codes, dtype=np.uint8)
    w = np.ascontiguousarray(w_codes, dtype=np.uint8)
    m, k = x.shape
    n, k2 = w.shape
    assert k == k2
    out = np.empty((m, n), dtype=np.uint16)
    exact = np.empty((m, n), dtype=np.float64) if want_exact else None
    lib().oracle_linear_fp8(x, w, out, exact.ctypes.data if want_exact else None, m, n, k,
                            ctypes.c_float(output_scale))
    return (out, exact) if want_exact else out


# ----------------------------------------------------------------------------- KV cache


def kv_cache_write(key, value, key_cache, value_cache, slot_mapping, page_size: int = 16) -> None:
    """In-place raw append into ``key_cache`` / ``value_cache`` ([pages, 8, page_size, 64])."""
    num_tokens = key.shape[0]
    num_pages = key_cache.shape[0]
    lib().oracle_kv_cache_write(key, value, key_cache, value_cache, slot_mapping, num_tokens,
                                num_pages, page_size)


def qk_norm_rope_kv_write_decode(query, key, value, query_norm, key_norm, inv_freq, position_ids,
                                 slot_mapping, key_cache, value_cache, eps: float,
                                 page_size: int = 16) -> None:
    """In place: query is normalised + rotated, caches receive the new K (normalised + rotated) and V."""
    lib().oracle_qk_norm_rope_kv_write_decode(query, key, value, query_norm, key_norm, inv_freq,
                                              position_ids, slot_mapping, key_cache, value_cache,
                                              key.shape[0], key_cache.shape[0], page_size,
                                              ctypes.c_float(eps))


def rope_inv_freq(theta: float = 1.0e6) -> np.ndarray:
    """inv_freq[i] = theta^(-2i/64) in float32 (src/model/lfm2_base.rs:595-601)."""
    index = np.arange(32, dtype=np.float32)
    return np.power(np.float32(theta), -(np.float32(2.0) * index) / np.float32(64.0)).astype(np.float32)


# ----------------------------------------------------------------------------- attention


def paged_ragged_attention(query, key_cache, value_cache, block_tables, request_slots, position_ids,
                           page_size: int = 16, output=None, want_exact: bool = False):
    """Returns bf16 output [T,32,64] (and the unrounded float64 result when asked).

    ``output`` may be passed in to observe which rows are left untouched by skipped tokens.
    ``request_slots`` None selects block-table row 0 for every token (single-sequence form).
    """
    block_tables = np.ascontiguousarray(block_tables, dtype=np.uint32)
    rows, stride = block_tables.shape
    num_tokens = query.shape[0]
    if output is None:
        output = np.zeros((num_tokens, 32, 64), dtype=np.uint16)
    exact = np.zeros((num_tokens, 32, 64), dtype=np.float64) if want_exact else None
    slots_pointer = None
    if request_slots is not None:
        request_slots = np.ascontiguousarray(request_slots, dtype=np.uint32)
        slots_pointer = request_slots.ctypes.data
    lib().oracle_paged_ragged_attention(query, key_cache, value_cache, block_tables, slots_pointer,
                                        np.ascontiguousarray(position_ids, dtype=np.uint32), output,
                                        exact.ctypes.data if want_exact else None, num_tokens,
                                        key_cache.shape[0], stride, rows, page_size)
    return (output, exact) if want_exact else output


def splitk_partials(query, key_cache, value_cache, block_tables, request_slots, position_ids,
                    num_splits: int, page_size: int = 16, partials=None) -> np.ndarray:
    block_tables = np.ascontiguousarray(block_tables, dtype=np.uint32)
    rows, stride = block_tables.shape
    num_tokens = query.shape[0]
    if partials is None:
        partials = np.zeros((num_tokens, 32, num_splits, 66), dtype=np.float32)
    lib().oracle_paged_ragged_attention_splitk_partials(
        query, key_cache, value_cache, block_tables,
        np.ascontiguousarray(request_slots, dtype=np.uint32),
        np.ascontiguousarray(position_ids, dtype=np.uint32), partials, num_tokens,
        key_cache.shape[0], stride, rows, page_size, num_splits)
    return partials


def merge_splitk(partials: np.ndarray) -> np.ndarray:
    num_tokens, heads, num_splits, stride = partials.shape
    assert heads == 32 and stride == 66
    output = np.zeros((num_tokens, 32, 64), dtype=np.uint16)
    lib().oracle_merge_splitk(np.ascontiguousarray(partials, dtype=np.float32), output, num_tokens,
                              num_splits)
    return output


def physical_slots(block_tables, request_slots, position_ids, page_size: int = 16) -> np.ndarray:
    block_tables = np.ascontiguousarray(block_tables, dtype=np.uint32)
    rows, stride = block_tables.shape
    request_slots = np.ascontiguousarray(request_slots, dtype=np.uint32)
    out = np.empty(request_slots.shape, dtype=np.int64)
    lib().oracle_physical_slots(block_tables, request_slots,
                                np.ascontiguousarray(position_ids, dtype=np.uint32), out,
                                request_slots.size, stride, rows, page_size)
    return out


# ----------------------------------------------------------------------------- other step ops


def rms_norm_bf16(x, weight, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    rows, hidden = x.shape
    out = np.empty_like(x)
    lib().oracle_rms_norm_bf16(x, np.ascontiguousarray(weight, dtype=np.uint16), out, rows, hidden, ctypes.c_float(eps))
    return out


def residual_rms_norm_bf16(residual, update, weight, eps: float) -> tuple[np.ndarray, np.ndarray]:
    """Returns (residual_out, normalized_out)."""
    residual = np.ascontiguousarray(residual, dtype=np.uint16)
    rows, hidden = residual.shape
    residual_out = np.empty_like(residual)
    normalized = np.empty_like(residual)
    lib().oracle_residual_rms_norm_bf16(residual, np.ascontiguousarray(update, dtype=np.uint16),
                                        np.ascontiguousarray(weight, dtype=np.uint16), residual_out, normalized, rows,
                                        hidden, ctypes.c_float(eps))
    return residual_out, normalized


def short_conv_decode_bf16(projected, weight, states, request_slots) -> np.ndarray:
    """projected [T, 3H], weight [H, 3], states [slots, H, 2] (updated in place); returns output [T, H]."""
    projected = np.ascontiguousarray(projected, dtype=np.uint16)
    tokens = projected.shape[0]
    hidden = projected.shape[1] // 3
    output = np.zeros((tokens, hidden), dtype=np.uint16)
    lib().oracle_short_conv_decode_bf16(projected, np.ascontiguousarray(weight, dtype=np.uint16), states,
                                        np.ascontiguousarray(request_slots, dtype=np.uint32), output, tokens, hidden,
                                        states.shape[0])
    return output


def short_conv_segmented_bf16(projected, weight, states, segment_offsets, segment_slots) -> np.ndarray:
    """projected [T, 3H], weight [H, 3], states [slots, H, 2] (updated in place), segment_offsets [S+1],
    segment_slots [S]; returns output [T, H] (rows of skipped segments stay zero)."""
    projected = np.ascontiguousarray(projected, dtype=np.uint16)
    tokens = projected.shape[0]
    hidden = projected.shape[1] // 3
    output = np.zeros((tokens, hidden), dtype=np.uint16)
    segment_slots = np.ascontiguousarray(segment_slots, dtype=np.uint32)
    lib().oracle_short_conv_segmented_bf16(projected, np.ascontiguousarray(weight, dtype=np.uint16), states,
                                           np.ascontiguousarray(segment_offsets, dtype=np.uint32), segment_slots,
                                           output, segment_slots.size, hidden, states.shape[0])
    return output


def hybrid_ragged_attention(query, current_key, current_value, key_cache, value_cache, block_tables, request_slots,
                            position_ids, segment_offsets, page_size: int = 16, output=None,
                            want_exact: bool = False):
    """Mixed prefill / decode attention: paged prefix + the contiguous K/V of the token's own segment.
    Returns bf16 output [T,32,64] (and the unrounded float64 result when asked); `output` may be passed in to
    observe which rows skipped tokens leave untouched."""
    block_tables = np.ascontiguousarray(block_tables, dtype=np.uint32)
    num_tokens = query.shape[0]
    if output is None:
        output = np.zeros((num_tokens, 32, 64), dtype=np.uint16)
    exact = np.zeros((num_tokens, 32, 64), dtype=np.float64) if want_exact else None
    segment_offsets = np.ascontiguousarray(segment_offsets, dtype=np.uint32)
    lib().oracle_hybrid_ragged_attention(
        np.ascontiguousarray(query, dtype=np.uint16), np.ascontiguousarray(current_key, dtype=np.uint16),
        np.ascontiguousarray(current_value, dtype=np.uint16), key_cache, value_cache, block_tables,
        np.ascontiguousarray(request_slots, dtype=np.uint32), np.ascontiguousarray(position_ids, dtype=np.uint32),
        segment_offsets, output, exact.ctypes.data if want_exact else None, num_tokens, key_cache.shape[0],
        block_tables.shape[1], segment_offsets.size - 1, page_size)
    return (output, exact) if want_exact else output


def argmax_rows_bf16(logits) -> np.ndarray:
    logits = np.ascontiguousarray(logits, dtype=np.uint16)
    rows, vocab = logits.shape
    sampled = np.empty(rows, dtype=np.uint32)
    lib().oracle_argmax_rows_bf16(logits, sampled, rows, vocab)
    return sampled


def linear_bf16(x, weight) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    weight = np.ascontiguousarray(weight, dtype=np.uint16)
    m, k = x.shape
    n = weight.shape[0]
    out = np.empty((m, n), dtype=np.uint16)
    lib().oracle_linear_bf16(x, weight, out, m, n, k)
    return out


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Sizes the OpenMP team to the cores this process may run on (torchrun exports OMP_NUM_THREADS=1 to its
    ranks); returns the team size."""
    import os
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(cores)
    return num_threads()

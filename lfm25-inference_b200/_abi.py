"""ctypes binding of ``liblfm25_b200.so`` (the C ABI declared in ``include/lfm25_b200.h``).

The library is the product; there is no fallback.  If it has not been built, importing this
module raises, and every op refuses to run.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(HERE, "liblfm25_b200.so")


class Lfm25Error(RuntimeError):
    """An entry point returned a negative status; ``code`` is the LFM25_ERR_* value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_BUFFER_TOO_SMALL = -2
ERR_UNSUPPORTED = -3
ERR_OVERFLOW = -4
ERR_CUDA = -5
ERR_NULL_POINTER = -6


class Slice(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("len", ctypes.c_size_t)]


def _launch_struct(name, slices_and_sizes):
    fields = []
    for field in slices_and_sizes:
        if isinstance(field, tuple):
            fields.append(field)
        elif field.startswith("#"):
            fields.append((field[1:], ctypes.c_size_t))
        else:
            fields.append((field, Slice))
    return type(name, (ctypes.Structure,), {"_fields_": fields})


KvCacheWriteLaunch = _launch_struct("KvCacheWriteLaunch", [
    "#page_size", "key", "value", "key_cache", "value_cache", "slot_mapping", "#num_tokens", "#num_pages"])
QkPostprocessLaunch = _launch_struct("QkPostprocessLaunch", [
    "#page_size", "query", "key", "value", "query_norm", "key_norm", "inv_freq", "position_ids",
    "slot_mapping", "key_cache", "value_cache", "#num_tokens", "#num_pages", ("eps", ctypes.c_float)])
PagedAttentionLaunch = _launch_struct("PagedAttentionLaunch", [
    "#page_size", "query", "key_cache", "value_cache", "block_table", "position_ids", "output",
    "#num_tokens", "#num_pages"])
FastRaggedAttentionLaunch = _launch_struct("FastRaggedAttentionLaunch", [
    "#page_size", "query", "key_cache", "value_cache", "block_tables", "request_slots", "position_ids",
    "output", "#num_tokens", "#num_pages", "#block_table_stride", "token_order"])
SplitKRaggedAttentionLaunch = _launch_struct("SplitKRaggedAttentionLaunch", [
    "#page_size", "query", "key_cache", "value_cache", "block_tables", "request_slots", "position_ids",
    "partials", "output", "#num_tokens", "#num_pages", "#block_table_stride", "#num_splits", "token_order"])



_P = ctypes.POINTER
_size = ctypes.c_size_t
_stream = ctypes.c_void_p


class Fp8LinearConfig(ctypes.Structure):
    _fields_ = [("m", ctypes.c_size_t), ("n", ctypes.c_size_t), ("k", ctypes.c_size_t),
                ("scale_mode", ctypes.c_uint32), ("output_scale", ctypes.c_float)]


class GemmTuning(ctypes.Structure):
    _fields_ = [("kernel", ctypes.c_uint32), ("n_tile", ctypes.c_uint32), ("splits", ctypes.c_uint32),
                ("stages", ctypes.c_uint32), ("issuers", ctypes.c_uint32),
                ("ctas_per_sm", ctypes.c_uint32), ("shared_memory_bytes", ctypes.c_uint32),
                ("batch_slices", ctypes.c_uint32)]


GEMM_KERNEL_AUTO, GEMM_KERNEL_STREAM, GEMM_KERNEL_WEIGHT_MAJOR, GEMM_KERNEL_LIBRARY, GEMM_KERNEL_BATCH_MAJOR = range(5)


class DecodeBatch(ctypes.Structure):
    _fields_ = [("token_ids", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("request_slots", ctypes.c_void_p),
                ("physical_slots", ctypes.c_void_p), ("block_tables", ctypes.c_void_p),
                ("block_table_stride", ctypes.c_size_t), ("block_table_rows", ctypes.c_size_t),
                ("num_tokens", ctypes.c_size_t), ("max_context_tokens", ctypes.c_size_t)]


class RaggedBatch(ctypes.Structure):
    _fields_ = [("token_ids", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("request_slots", ctypes.c_void_p),
                ("physical_slots", ctypes.c_void_p), ("segment_offsets", ctypes.c_void_p),
                ("segment_slots", ctypes.c_void_p), ("output_rows", ctypes.c_void_p),
                ("block_tables", ctypes.c_void_p), ("block_table_stride", ctypes.c_size_t),
                ("block_table_rows", ctypes.c_size_t), ("num_tokens", ctypes.c_size_t),
                ("num_segments", ctypes.c_size_t), ("num_decode_segments", ctypes.c_size_t),
                ("max_decode_context_tokens", ctypes.c_size_t)]


class PrefixCacheSnapshot(ctypes.Structure):
    _fields_ = [("nodes", ctypes.c_size_t), ("cached_pages", ctypes.c_size_t), ("checkpoints", ctypes.c_size_t),
                ("hits", ctypes.c_uint64), ("misses", ctypes.c_uint64), ("matched_tokens", ctypes.c_uint64)]


class CostPoint(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_size_t), ("tokens", ctypes.c_size_t), ("context", ctypes.c_size_t),
                ("milliseconds", ctypes.c_double)]


class SchedulerConfig(ctypes.Structure):
    _fields_ = [("step_budget_ms", ctypes.c_double), ("ttft_slo_us", ctypes.c_uint64),
                ("tpot_slo_us", ctypes.c_uint64), ("fp8_decode", ctypes.c_uint32),
                ("maximum_prefill_tokens", ctypes.c_size_t)]


class RequestView(ctypes.Structure):
    _fields_ = [("phase", ctypes.c_uint32), ("prompt_len", ctypes.c_size_t), ("prefilled", ctypes.c_size_t),
                ("context_tokens", ctypes.c_size_t), ("arrival_us", ctypes.c_uint64),
                ("first_token_deadline_us", ctypes.c_uint64), ("next_token_deadline_us", ctypes.c_uint64)]


class ScheduledWork(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_uint32), ("slot", ctypes.c_uint32), ("tokens", ctypes.c_size_t)]


class BatchPlan(ctypes.Structure):
    _fields_ = [("predicted_ms", ctypes.c_double), ("decode_count", ctypes.c_size_t),
                ("prefill_tokens", ctypes.c_size_t), ("work_count", ctypes.c_size_t)]


class EngineConfig(ctypes.Structure):
    _fields_ = [("max_slots", ctypes.c_size_t), ("max_sequence_tokens", ctypes.c_size_t),
                ("max_prefill_tokens", ctypes.c_size_t), ("radix_pages", ctypes.c_size_t),
                ("checkpoint_capacity", ctypes.c_size_t), ("use_fp8", ctypes.c_uint32),
                ("ttft_slo_us", ctypes.c_uint64), ("tpot_slo_us", ctypes.c_uint64),
                ("step_budget_ms", ctypes.c_double), ("admission_control", ctypes.c_uint32),
                ("interactive_prompt_limit", ctypes.c_size_t)]


class EngineEvent(ctypes.Structure):
    _fields_ = [("request_id", ctypes.c_uint64), ("time_us", ctypes.c_uint64), ("token", ctypes.c_uint32),
                ("finished", ctypes.c_uint32), ("reused_tokens", ctypes.c_uint32), ("rejected", ctypes.c_uint32)]


class EngineStats(ctypes.Structure):
    _fields_ = [("steps", ctypes.c_uint64), ("decode_steps", ctypes.c_uint64), ("mixed_steps", ctypes.c_uint64),
                ("generated_tokens", ctypes.c_uint64), ("prefill_tokens", ctypes.c_uint64),
                ("reused_prompt_tokens", ctypes.c_uint64), ("gpu_ms", ctypes.c_double),
                ("rejected_requests", ctypes.c_uint64)]


class Fp8Site(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("activation_quantize", ctypes.c_float),
                ("activation_dequantize", ctypes.c_float), ("weight_dequantize", ctypes.c_float)]


class LinearWeights(ctypes.Structure):
    _fields_ = [("bf16", ctypes.c_void_p), ("fp8", Fp8Site), ("n", ctypes.c_size_t), ("k", ctypes.c_size_t)]


class Layer(ctypes.Structure):
    _fields_ = [("is_attention", ctypes.c_uint32), ("operator_norm", ctypes.c_void_p), ("ffn_norm", ctypes.c_void_p),
                ("conv_input", LinearWeights), ("conv_kernel", ctypes.c_void_p), ("conv_output", LinearWeights),
                ("conv_state", ctypes.c_void_p), ("query", LinearWeights), ("key", LinearWeights),
                ("value", LinearWeights), ("output", LinearWeights), ("query_norm", ctypes.c_void_p),
                ("key_norm", ctypes.c_void_p), ("key_cache", ctypes.c_void_p), ("value_cache", ctypes.c_void_p),
                ("gate_up", LinearWeights), ("down", LinearWeights)]


class Model(ctypes.Structure):
    _fields_ = [("num_layers", ctypes.c_uint32), ("layers", _P(Layer)), ("embedding", ctypes.c_void_p),
                ("lm_head_fp8", Fp8Site), ("final_norm", ctypes.c_void_p), ("inv_freq", ctypes.c_void_p),
                ("norm_eps", ctypes.c_float), ("num_pages", ctypes.c_size_t), ("num_request_slots", ctypes.c_size_t)]


class KvPoolSnapshot(ctypes.Structure):
    _fields_ = [(name, ctypes.c_size_t) for name in ("total_pages", "free_pages", "allocated_pages",
                                                     "reserved_pages", "cached_pages", "peak_allocated_pages")]


KV_PHYSICAL_PAGES_EXHAUSTED = -11
KV_LOGICAL_RESERVATION_EXHAUSTED = -12
KV_SEQUENCE_CAPACITY_EXCEEDED = -13
PHASE_FREE, PHASE_QUEUED_PREFILL, PHASE_DECODING = 0, 1, 2
FP8_SCALE_TENSORWIDE = 0
FP8_SCALE_BLOCK32 = 1

FusedRaggedDecodeLaunch = _launch_struct("FusedRaggedDecodeLaunch", [
    "#page_size", "query_raw", "key_raw", "value_raw", "query_norm", "key_norm", "inv_freq", "key_cache",
    "value_cache", "position_ids", "slot_mapping", "output", "#num_tokens", "#num_pages", ("eps", ctypes.c_float),
    "block_tables", "request_slots", "#block_table_stride", "partials", "#num_splits", "#query_token_stride",
    "#kv_token_stride", "token_order"])

HybridAttentionLaunch = _launch_struct("HybridAttentionLaunch", [
    "#page_size", "query", "current_key", "current_value", "key_cache", "value_cache", "block_tables", "request_slots",
    "position_ids", "segment_offsets", "output", "#num_tokens", "#num_pages", "#block_table_stride", "#num_segments",
    "#query_token_stride", "#kv_token_stride"])

# name -> (restype, argtypes); every symbol that include/lfm25_b200.h declares
PROTOTYPES = {
    "lfm25_last_error": (ctypes.c_char_p, []),
    "lfm25_version": (ctypes.c_char_p, []),
    "lfm25_device_status": (ctypes.c_int32, [_stream, _P(ctypes.c_uint32)]),
    "lfm25_kv_cache_write_lfm2_bf16": (ctypes.c_int32, [_stream, _P(KvCacheWriteLaunch)]),
    "lfm25_qk_norm_rope_kv_write_decode": (ctypes.c_int32, [_stream, _P(QkPostprocessLaunch)]),
    "lfm25_paged_attention_fast_lfm2_bf16": (ctypes.c_int32, [_stream, _P(PagedAttentionLaunch)]),
    "lfm25_paged_ragged_attention_fast_lfm2_bf16": (ctypes.c_int32, [_stream, _P(FastRaggedAttentionLaunch)]),
    "lfm25_context_order_desc": (ctypes.c_int32, [_stream, Slice, _size, Slice]),
    "lfm25_paged_ragged_attention_splitk_lfm2_bf16": (ctypes.c_int32, [_stream, _P(SplitKRaggedAttentionLaunch)]),
    "lfm25_paged_ragged_attention_splitk_static_lfm2_bf16": (
        ctypes.c_int32, [_stream, _P(FastRaggedAttentionLaunch), _size]),
    "lfm25_fused_ragged_paged_attention_decode_lfm2_bf16": (ctypes.c_int32, [_stream, _P(FusedRaggedDecodeLaunch)]),
    "lfm25_splitk_workspace_elements": (_size, [_size]),
    "lfm25_splitk_decode_splits": (_size, [_size, _size, _size]),
    "lfm25_decode_one_kernel_preferred": (ctypes.c_int32, [_size, _size, _size]),
    "lfm25_bf16_own_kernel_max_rows": (_size, []),
    "lfm25_blaslt_library_calls": (ctypes.c_uint64, []),
    "lfm25_quantize_bf16_e4m3": (ctypes.c_int32, [_stream, Slice, Slice, _size, ctypes.c_float]),
    "lfm25_silu_mul_packed_bf16": (ctypes.c_int32, [_stream, Slice, Slice, _size, _size]),
    "lfm25_silu_mul_packed_bf16_to_e4m3": (ctypes.c_int32, [_stream, Slice, Slice, _size, _size, ctypes.c_float]),
    "lfm25_linear_fp8_scaled": (ctypes.c_int32, [_stream, Slice, Slice, Slice, _P(Fp8LinearConfig)]),
    "lfm25_blaslt_create": (ctypes.c_int32, [_stream, _P(ctypes.c_void_p)]),
    "lfm25_blaslt_destroy": (None, [ctypes.c_void_p]),
    "lfm25_blaslt_set_stream": (ctypes.c_int32, [ctypes.c_void_p, _stream]),
    "lfm25_blaslt_workspace_size": (_size, [ctypes.c_void_p]),
    "lfm25_blaslt_stream": (ctypes.c_void_p, [ctypes.c_void_p]),
    "lfm25_blaslt_linear_fp8_scaled": (ctypes.c_int32, [ctypes.c_void_p, Slice, Slice, Slice, _P(Fp8LinearConfig)]),
    "lfm25_blaslt_linear_fp8_silu_mul": (ctypes.c_int32, [ctypes.c_void_p, Slice, Slice, Slice, _P(Fp8LinearConfig),
                                                          ctypes.c_float, ctypes.c_uint32]),
    "lfm25_blaslt_linear_bf16": (ctypes.c_int32, [ctypes.c_void_p, Slice, Slice, Slice, _size, _size, _size]),
    "lfm25_blaslt_linear_bf16_silu_mul": (ctypes.c_int32, [ctypes.c_void_p, Slice, Slice, Slice, _size, _size, _size,
                                                           ctypes.c_float, ctypes.c_uint32]),
    "lfm25_blaslt_set_gemm_tuning": (ctypes.c_int32, [ctypes.c_void_p, _P(GemmTuning)]),
    "lfm25_blaslt_gemm_plan": (ctypes.c_int32, [ctypes.c_void_p, _size, _size, _size, ctypes.c_uint32,
                                                _P(ctypes.c_uint32)]),
    "lfm25_set_option": (ctypes.c_int32, [ctypes.c_char_p, ctypes.c_int64]),
    "lfm25_get_option": (ctypes.c_int32, [ctypes.c_char_p, _P(ctypes.c_int64)]),
    "lfm25_embedding_bf16": (ctypes.c_int32, [_stream, Slice, Slice, Slice, _size, _size, _size]),
    "lfm25_rms_norm_bf16": (ctypes.c_int32, [_stream, Slice, Slice, Slice, _size, _size, ctypes.c_float]),
    "lfm25_residual_rms_norm_bf16": (
        ctypes.c_int32, [_stream, Slice, Slice, Slice, Slice, Slice, _size, _size, ctypes.c_float]),
    "lfm25_residual_rms_norm_bf16_e4m3": (
        ctypes.c_int32, [_stream, Slice, Slice, Slice, Slice, Slice, Slice, _size, _size, ctypes.c_float,
                         ctypes.c_float]),
    "lfm25_hybrid_ragged_attention_lfm2_bf16": (ctypes.c_int32, [_stream, _P(HybridAttentionLaunch)]),
    "lfm25_short_conv_segmented_lfm2_bf16": (
        ctypes.c_int32, [_stream, Slice, Slice, Slice, Slice, Slice, Slice, _size, _size, _size, _size]),
    "lfm25_gather_rows_bf16": (ctypes.c_int32, [_stream, Slice, Slice, Slice, _size, _size, _size]),
    "lfm25_short_conv_decode_bf16": (ctypes.c_int32, [_stream, Slice, Slice, Slice, Slice, Slice, _size, _size, _size]),
    "lfm25_argmax_rows_bf16": (ctypes.c_int32, [_stream, Slice, Slice, _size, _size]),
    "lfm25_decode_step_metadata": (ctypes.c_int32, [_stream, _P(DecodeBatch), Slice, _size, ctypes.c_uint32]),
    "lfm25_decode_executor_create": (ctypes.c_int32, [ctypes.c_void_p, _size, _P(ctypes.c_void_p)]),
    "lfm25_decode_executor_create_ragged": (ctypes.c_int32, [ctypes.c_void_p, _size, _size, _P(ctypes.c_void_p)]),
    "lfm25_decode_executor_forward_ragged": (
        ctypes.c_int32, [ctypes.c_void_p, _P(Model), _P(RaggedBatch), ctypes.c_uint32]),
    "lfm25_decode_executor_destroy": (None, [ctypes.c_void_p]),
    "lfm25_decode_executor_graph_kernels": (ctypes.c_size_t, [ctypes.c_void_p]),
    "lfm25_decode_executor_graph_captures": (ctypes.c_size_t, [ctypes.c_void_p]),
    "lfm25_decode_executor_forward": (
        ctypes.c_int32, [ctypes.c_void_p, _P(Model), _P(DecodeBatch), ctypes.c_uint32, ctypes.c_uint32]),
    "lfm25_decode_executor_step_graph": (
        ctypes.c_int32, [ctypes.c_void_p, _P(Model), _P(DecodeBatch), ctypes.c_uint32, ctypes.c_uint32]),
    "lfm25_decode_executor_serve_step": (
        ctypes.c_int32, [ctypes.c_void_p, _P(Model), _P(DecodeBatch), ctypes.c_uint32, ctypes.c_void_p,
                         ctypes.c_void_p]),
    "lfm25_decode_executor_profile": (
        ctypes.c_int32, [ctypes.c_void_p, ctypes.c_uint32, _P(ctypes.c_float), _P(ctypes.c_uint32)]),
    "lfm25_decode_executor_download_sampled": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_void_p, _size]),
    "lfm25_decode_executor_download_logits": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_void_p, _size]),
    "lfm25_decode_executor_sampled": (ctypes.c_void_p, [ctypes.c_void_p]),
    "lfm25_decode_executor_logits": (ctypes.c_void_p, [ctypes.c_void_p]),
    "lfm25_kv_allocator_create": (ctypes.c_int32, [_size, _size, _P(ctypes.c_void_p)]),
    "lfm25_kv_allocator_destroy": (None, [ctypes.c_void_p]),
    "lfm25_kv_allocator_try_reserve_tokens": (ctypes.c_int64, [ctypes.c_void_p, _size]),
    "lfm25_kv_allocator_try_reserve_pages": (ctypes.c_int64, [ctypes.c_void_p, _size]),
    "lfm25_kv_allocator_release_reservation": (None, [ctypes.c_void_p, _size]),
    "lfm25_kv_allocator_pin_cached_pages": (ctypes.c_int32, [ctypes.c_void_p, _P(ctypes.c_uint32), _size]),
    "lfm25_kv_allocator_retain_pages": (ctypes.c_int32, [ctypes.c_void_p, _P(ctypes.c_uint32), _size]),
    "lfm25_kv_allocator_grow_sequence": (ctypes.c_int64, [ctypes.c_void_p, _size, _size, _P(ctypes.c_uint32), _size]),
    "lfm25_kv_allocator_pages_short": (ctypes.c_int64, [ctypes.c_void_p, _P(_size), _P(_size), _size]),
    "lfm25_kv_allocator_release_sequence": (None, [ctypes.c_void_p, _size, _P(ctypes.c_uint32), _size]),
    "lfm25_kv_allocator_snapshot": (None, [ctypes.c_void_p, _P(KvPoolSnapshot)]),
    "lfm25_block_tables_create": (ctypes.c_int32, [_size, _size, _P(ctypes.c_void_p)]),
    "lfm25_block_tables_destroy": (None, [ctypes.c_void_p]),
    "lfm25_block_tables_slot": (_P(ctypes.c_uint32), [ctypes.c_void_p, _size]),
    "lfm25_block_tables_data": (_P(ctypes.c_uint32), [ctypes.c_void_p]),
    "lfm25_schedule_decode": (_size, [_P(ctypes.c_uint32), _P(ctypes.c_uint64), _P(ctypes.c_uint32), _size,
                                      ctypes.c_uint64, _P(ctypes.c_uint32), _P(_size)]),
    "lfm25_engine_create": (ctypes.c_int32, [ctypes.c_void_p, _P(Model), _P(EngineConfig), _P(ctypes.c_void_p)]),
    "lfm25_engine_destroy": (None, [ctypes.c_void_p]),
    "lfm25_engine_calibrate": (ctypes.c_int32, [ctypes.c_void_p]),
    "lfm25_engine_cost_model": (ctypes.c_void_p, [ctypes.c_void_p]),
    "lfm25_engine_submit": (
        ctypes.c_int32, [ctypes.c_void_p, ctypes.c_uint64, _P(ctypes.c_uint32), _size, _size, ctypes.c_uint64]),
    "lfm25_engine_step": (
        ctypes.c_int32, [ctypes.c_void_p, ctypes.c_uint64, _P(EngineEvent), _size, _P(_size),
                         _P(ctypes.c_float)]),
    "lfm25_engine_active": (_size, [ctypes.c_void_p]),
    "lfm25_engine_queued": (_size, [ctypes.c_void_p]),
    "lfm25_engine_get_stats": (None, [ctypes.c_void_p, _P(EngineStats), _P(KvPoolSnapshot), _P(PrefixCacheSnapshot)]),
    "lfm25_cost_model_create": (
        ctypes.c_int32, [_P(CostPoint), _size, _P(CostPoint), _size, _P(CostPoint), _size, _size,
                         _P(ctypes.c_void_p)]),
    "lfm25_cost_model_destroy": (None, [ctypes.c_void_p]),
    "lfm25_cost_model_predict": (ctypes.c_double, [ctypes.c_void_p, ctypes.c_uint32, _size, _size, _size]),
    "lfm25_cost_model_predict_decode_ms": (ctypes.c_double, [ctypes.c_void_p, _size, _size, ctypes.c_uint32]),
    "lfm25_cost_model_predict_prefill_ms": (ctypes.c_double, [ctypes.c_void_p, _size]),
    "lfm25_schedule": (
        ctypes.c_int32, [ctypes.c_void_p, _P(SchedulerConfig), _P(RequestView), _size, ctypes.c_uint64,
                         _P(ScheduledWork), _size, _P(BatchPlan)]),
    "lfm25_radix_cache_create": (ctypes.c_int32, [_size, _size, _P(ctypes.c_void_p)]),
    "lfm25_radix_cache_destroy": (None, [ctypes.c_void_p]),
    "lfm25_radix_cache_longest_checkpoint": (
        ctypes.c_int64, [ctypes.c_void_p, _P(ctypes.c_uint32), _size, _size, _P(ctypes.c_uint32), _size, _P(_size),
                         _P(ctypes.c_uint32)]),
    "lfm25_radix_cache_probe_checkpoint": (
        ctypes.c_int64, [ctypes.c_void_p, _P(ctypes.c_uint32), _size, _size, _P(ctypes.c_uint32), _size, _P(_size),
                         _P(ctypes.c_uint32)]),
    "lfm25_radix_cache_can_publish": (ctypes.c_uint32, [ctypes.c_void_p, _P(ctypes.c_uint32), _size, _size]),
    "lfm25_radix_cache_insert_checkpoint": (
        ctypes.c_int64, [ctypes.c_void_p, _P(ctypes.c_uint32), _size, _size, _P(ctypes.c_uint32), _size,
                         ctypes.c_uint32, _P(ctypes.c_uint32)]),
    "lfm25_radix_cache_snapshot": (None, [ctypes.c_void_p, _P(PrefixCacheSnapshot)]),
    "lfm25_conv_checkpoints_create": (ctypes.c_int32, [_size, _size, _size, _size, _P(ctypes.c_void_p)]),
    "lfm25_conv_checkpoints_destroy": (None, [ctypes.c_void_p]),
    "lfm25_conv_checkpoints_acquire": (ctypes.c_int64, [ctypes.c_void_p]),
    "lfm25_conv_checkpoints_release": (None, [ctypes.c_void_p, ctypes.c_uint32]),
    "lfm25_conv_checkpoints_available": (ctypes.c_size_t, [ctypes.c_void_p]),
    "lfm25_conv_checkpoints_capacity": (ctypes.c_size_t, [ctypes.c_void_p]),
    "lfm25_conv_checkpoints_capture_layer": (
        ctypes.c_int32, [ctypes.c_void_p, _stream, ctypes.c_uint32, _size, ctypes.c_void_p, _size, _size]),
    "lfm25_conv_checkpoints_restore_layer": (
        ctypes.c_int32, [ctypes.c_void_p, _stream, ctypes.c_uint32, _size, ctypes.c_void_p, _size, _size]),
    "lfm25_dispatcher_create": (ctypes.c_int32, [_size, _P(ctypes.c_void_p)]),
    "lfm25_dispatcher_destroy": (None, [ctypes.c_void_p]),
    "lfm25_dispatcher_assign": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint64]),
    "lfm25_dispatcher_assign_bounded": (ctypes.c_int32, [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32,
                                                         ctypes.c_uint64, ctypes.c_uint64]),
    "lfm25_dispatcher_complete": (None, [ctypes.c_void_p, _size, ctypes.c_uint64]),
    "lfm25_dispatcher_mark_failed": (None, [ctypes.c_void_p, _size]),
    "lfm25_dispatcher_load": (ctypes.c_uint64, [ctypes.c_void_p, _size]),
}

_library = None


def library() -> ctypes.CDLL:
    global _library
    if _library is None:
        if not os.path.exists(LIBRARY_PATH):
            raise ImportError(
                f"{LIBRARY_PATH} is missing: build it with `python lfm25-inference_b200/build.py`. "
                "There is no CPU or PyTorch fallback for this library.")
        handle = ctypes.CDLL(LIBRARY_PATH)
        for name, (restype, argtypes) in PROTOTYPES.items():
            function = getattr(handle, name)
            function.restype = restype
            function.argtypes = argtypes
        _library = handle
    return _library


def check(code: int) -> None:
    if code != OK:
        raise Lfm25Error(code, library().lfm25_last_error().decode())

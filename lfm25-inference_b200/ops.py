"""Op surface of the decode path, named and shaped after the reference's ``src/ops`` functions.

Every function takes CUDA ``torch`` tensors as plain device buffers (torch is only the owner of the
memory and of the stream), checks ranks and shapes the way the reference's op layer does before any
launch, and then calls the C ABI on the current stream.  ``*_into`` variants write into caller-owned
outputs; nothing here allocates device memory except the convenience wrappers that return a tensor.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _abi
from ._abi import Lfm25Error, Slice, check, library

SPLITK_MAX_SPLITS = 8
SPLITK_PARTIAL_STRIDE = 66


def _slice(tensor: torch.Tensor) -> Slice:
    if not tensor.is_cuda:
        raise Lfm25Error(_abi.ERR_INVALID_ARGUMENT, "tensor is not on a CUDA device")
    if not tensor.is_contiguous():
        raise Lfm25Error(_abi.ERR_INVALID_ARGUMENT, "tensor storage must be contiguous")
    return Slice(tensor.data_ptr(), tensor.numel())


def _row_strided_slice(tensor: torch.Tensor) -> Slice:
    """A tensor whose rows (dimension 0) may be spaced apart but are dense inside: the span it covers."""
    if not tensor.is_cuda:
        raise Lfm25Error(_abi.ERR_INVALID_ARGUMENT, "tensor is not on a CUDA device")
    if tensor.shape[0] == 0:
        return Slice(tensor.data_ptr(), 0)
    row = tensor[0].numel()
    return Slice(tensor.data_ptr(), (tensor.shape[0] - 1) * tensor.stride(0) + row)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ensure(condition: bool, message: str) -> None:
    if not condition:
        raise Lfm25Error(_abi.ERR_INVALID_ARGUMENT, message)


@dataclass
class PagedKvArena:
    """Physical K and V store of one attention layer: two bf16 tensors [num_pages, 8, page_size, 64],
    zero-filled at creation (reference: src/cache/arena.rs:13-30)."""

    key: torch.Tensor
    value: torch.Tensor
    page_size: int = 16

    @classmethod
    def new(cls, num_pages: int, page_size: int = 16, device="cuda") -> "PagedKvArena":
        _ensure(num_pages > 0, "paged KV arena requires pages")
        shape = (num_pages, 8, page_size, 64)
        return cls(torch.zeros(shape, dtype=torch.bfloat16, device=device),
                   torch.zeros(shape, dtype=torch.bfloat16, device=device), page_size)

    @property
    def num_pages(self) -> int:
        return self.key.shape[0]

    def write_lfm2(self, key: torch.Tensor, value: torch.Tensor, physical_slots: torch.Tensor) -> None:
        """Raw append (reference: src/cache/arena.rs:52-86)."""
        _ensure(key.dim() == 3 and tuple(key.shape[1:]) == (8, 64), "KV write key must have shape [N,8,64]")
        _ensure(value.shape == key.shape, "KV write key/value shape mismatch")
        _ensure(physical_slots.numel() == key.shape[0], "KV write slot count mismatch")
        kv_cache_write_lfm2_bf16(key, value, self.key, self.value, physical_slots, self.page_size)


@dataclass
class FastRaggedAttentionInput:
    """Reference: src/ops/attention_async_fast.rs:15-22."""

    query: torch.Tensor
    arena: PagedKvArena
    block_tables: torch.Tensor
    block_table_stride: int
    request_slots: torch.Tensor
    position_ids: torch.Tensor


# ------------------------------------------------------------------------------- KV append


def kv_cache_write_lfm2_bf16(key, value, key_cache, value_cache, slot_mapping, page_size: int = 16) -> None:
    launch = _abi.KvCacheWriteLaunch(page_size, _slice(key), _slice(value), _slice(key_cache), _slice(value_cache),
                                     _slice(slot_mapping), key.shape[0] if key.dim() else 0, key_cache.shape[0])
    check(library().lfm25_kv_cache_write_lfm2_bf16(_stream(), launch))


def qk_norm_rope_kv_write_arena_decode_bf16(query, key, value, query_norm, key_norm, inv_freq, position_ids,
                                            slot_mapping, arena: PagedKvArena, eps: float) -> None:
    """Reference: src/ops/qk_postprocess.rs:107-116 (shape checks :32-105)."""
    _ensure(query.dim() == 3 and tuple(query.shape[1:]) == (32, 64), "fused QK query must have shape [N,32,64]")
    num_tokens = query.shape[0]
    _ensure(tuple(key.shape) == (num_tokens, 8, 64), "fused QK key must have shape [N,8,64]")
    _ensure(tuple(value.shape) == (num_tokens, 8, 64), "fused QK value must have shape [N,8,64]")
    _ensure(position_ids.numel() == num_tokens, "fused QK position count mismatch")
    _ensure(slot_mapping.numel() == num_tokens, "fused QK slot count mismatch")
    launch = _abi.QkPostprocessLaunch(arena.page_size, _slice(query), _slice(key), _slice(value), _slice(query_norm),
                                      _slice(key_norm), _slice(inv_freq), _slice(position_ids), _slice(slot_mapping),
                                      _slice(arena.key), _slice(arena.value), num_tokens, arena.num_pages, eps)
    check(library().lfm25_qk_norm_rope_kv_write_decode(_stream(), launch))


# ------------------------------------------------------------------------------- attention


def splitk_workspace_elements(maximum_tokens: int) -> int:
    return int(library().lfm25_splitk_workspace_elements(maximum_tokens))


def splitk_decode_splits(num_tokens: int, maximum_context_tokens: int, page_size: int = 16) -> int:
    return int(library().lfm25_splitk_decode_splits(num_tokens, maximum_context_tokens, page_size))


def bf16_own_kernel_max_rows() -> int:
    """Largest batch that the BF16 linear runs on the library's own tensor-core kernel (cuBLASLt above)."""
    return int(library().lfm25_bf16_own_kernel_max_rows())


def library_calls() -> int:
    """Matmuls this process has handed to cuBLASLt so far (not counting replays of captured graphs)."""
    return int(library().lfm25_blaslt_library_calls())


def decode_one_kernel_preferred(page_size: int, context_tokens: int, batch_size: int) -> bool:
    """Reference: should_use_mok_one_kernel (src/ops/mok_dispatch.rs:7-27), with thresholds measured on a B200."""
    return bool(library().lfm25_decode_one_kernel_preferred(page_size, context_tokens, batch_size))


def paged_attention_fast_lfm2_bf16_into(query, key_cache, value_cache, block_table, position_ids, output,
                                        page_size: int = 16) -> None:
    """One sequence (reference: src/ops/attention_async_fast.rs:49-83)."""
    _ensure(query.dim() == 3 and tuple(query.shape[1:]) == (32, 64), "fast LFM2 query must have shape [N,32,64]")
    _ensure(position_ids.numel() == query.shape[0], "fast attention position count mismatch")
    launch = _abi.PagedAttentionLaunch(page_size, _slice(query), _slice(key_cache), _slice(value_cache),
                                       _slice(block_table), _slice(position_ids), _slice(output), query.shape[0],
                                       key_cache.shape[0])
    check(library().lfm25_paged_attention_fast_lfm2_bf16(_stream(), launch))


def _validate_ragged_input(inputs: FastRaggedAttentionInput) -> int:
    _ensure(inputs.query.dim() == 3 and tuple(inputs.query.shape[1:]) == (32, 64),
            "fast ragged LFM2 query must have shape [N,32,64]")
    _ensure(inputs.block_tables.dim() == 2, "fast block tables must be rank 2")
    _ensure(inputs.block_tables.shape[1] == inputs.block_table_stride, "fast block table stride/shape mismatch")
    num_tokens = inputs.query.shape[0]
    _ensure(inputs.request_slots.numel() == num_tokens, "fast ragged request slot count mismatch")
    _ensure(inputs.position_ids.numel() == num_tokens, "fast ragged position count mismatch")
    return num_tokens


def _order_slice(token_order, num_tokens: int) -> Slice:
    if token_order is None:
        return Slice(None, 0)
    _ensure(token_order.numel() >= num_tokens, "token order shorter than the batch")
    return _slice(token_order)


def context_order_desc_into(position_ids: torch.Tensor, order: torch.Tensor) -> None:
    """order[r] = index of the token with the r-th largest position: the `token_order` of the decode attention ops
    (their CTAs then start on the longest contexts).  No counterpart in the reference."""
    check(library().lfm25_context_order_desc(_stream(), _slice(position_ids), position_ids.numel(), _slice(order)))


def paged_ragged_attention_fast_lfm2_bf16_into(inputs: FastRaggedAttentionInput, output: torch.Tensor,
                                               token_order=None) -> None:
    """Reference: src/ops/attention_async_fast.rs:123-152."""
    num_tokens = _validate_ragged_input(inputs)
    launch = _abi.FastRaggedAttentionLaunch(
        inputs.arena.page_size, _slice(inputs.query), _slice(inputs.arena.key), _slice(inputs.arena.value),
        _slice(inputs.block_tables), _slice(inputs.request_slots), _slice(inputs.position_ids), _slice(output),
        num_tokens, inputs.arena.num_pages, inputs.block_table_stride, _order_slice(token_order, num_tokens))
    check(library().lfm25_paged_ragged_attention_fast_lfm2_bf16(_stream(), launch))


def paged_ragged_attention_fast_lfm2_bf16(inputs: FastRaggedAttentionInput) -> torch.Tensor:
    output = torch.empty((inputs.query.shape[0], 32, 64), dtype=torch.bfloat16, device=inputs.query.device)
    paged_ragged_attention_fast_lfm2_bf16_into(inputs, output)
    return output


def paged_ragged_attention_splitk_lfm2_bf16_into(inputs: FastRaggedAttentionInput, partials, num_splits: int,
                                                 output: torch.Tensor, token_order=None) -> None:
    """Reference: src/ops/attention_async_fast.rs:154-197.  `partials` None (no counterpart in the reference): no
    workspace and no records; the splits of a token merge inside the kernel (2, 4 or 8 splits)."""
    _ensure(2 <= num_splits <= SPLITK_MAX_SPLITS, f"split-K attention requires 2..={SPLITK_MAX_SPLITS} splits")
    num_tokens = _validate_ragged_input(inputs)
    launch = _abi.SplitKRaggedAttentionLaunch(
        inputs.arena.page_size, _slice(inputs.query), _slice(inputs.arena.key), _slice(inputs.arena.value),
        _slice(inputs.block_tables), _slice(inputs.request_slots), _slice(inputs.position_ids),
        _slice(partials) if partials is not None else Slice(None, 0),
        _slice(output), num_tokens, inputs.arena.num_pages, inputs.block_table_stride, num_splits,
        _order_slice(token_order, num_tokens))
    check(library().lfm25_paged_ragged_attention_splitk_lfm2_bf16(_stream(), launch))


def fused_ragged_paged_attention_decode_lfm2_bf16_into(query_raw, key_raw, value_raw, query_norm, key_norm, inv_freq,
                                                       position_ids, slot_mapping, arena: PagedKvArena, block_tables,
                                                       block_table_stride: int, request_slots, eps: float, output,
                                                       partials=None, num_splits: int = 1, token_order=None) -> None:
    """One-kernel decode: QK-norm + RoPE + paged KV append + attention
    (reference: src/ops/attention_fused.rs:95-153); optionally split over the KV axis.  The three projections may
    be row-strided views (columns of one packed [N, 3072] GEMM output); the last two dimensions must be dense."""
    _ensure(query_raw.dim() == 3 and tuple(query_raw.shape[1:]) == (32, 64), "fused query must have shape [N,32,64]")
    num_tokens = query_raw.shape[0]
    _ensure(tuple(key_raw.shape) == (num_tokens, 8, 64), "fused key must have shape [N,8,64]")
    _ensure(tuple(value_raw.shape) == (num_tokens, 8, 64), "fused value must have shape [N,8,64]")
    for name, tensor in (("query", query_raw), ("key", key_raw), ("value", value_raw)):
        _ensure(tuple(tensor.stride()[1:]) == (64, 1), f"fused {name} heads must be dense")
    _ensure(key_raw.stride(0) == value_raw.stride(0), "fused key and value must share their token stride")
    _ensure(block_tables.dim() == 2 and block_tables.shape[1] == block_table_stride,
            "fused block table stride/shape mismatch")
    empty = Slice(None, 0)
    launch = _abi.FusedRaggedDecodeLaunch(
        arena.page_size, _row_strided_slice(query_raw), _row_strided_slice(key_raw), _row_strided_slice(value_raw),
        _slice(query_norm), _slice(key_norm),
        _slice(inv_freq), _slice(arena.key), _slice(arena.value), _slice(position_ids), _slice(slot_mapping),
        _slice(output), num_tokens, arena.num_pages, eps, _slice(block_tables), _slice(request_slots),
        block_table_stride, _slice(partials) if partials is not None else empty, num_splits,
        query_raw.stride(0) if num_tokens > 1 else 0, key_raw.stride(0) if num_tokens > 1 else 0,
        _order_slice(token_order, num_tokens))
    check(library().lfm25_fused_ragged_paged_attention_decode_lfm2_bf16(_stream(), launch))


def hybrid_ragged_attention_lfm2_bf16_into(query, current_key, current_value, arena: PagedKvArena, block_tables,
                                           block_table_stride: int, request_slots, position_ids, segment_offsets,
                                           output) -> None:
    """Attention of a step that mixes prefill chunks and decode tokens: paged prefix + the step's own contiguous K/V
    (reference: src/ops/attention.rs:121-185, HybridRaggedAttentionInput).  `current_key` / `current_value` None:
    every key up to each token's position is read from the cache (the step's K/V were appended before).  The
    projections may be row-strided views of one packed buffer."""
    _ensure(query.dim() == 3 and tuple(query.shape[1:]) == (32, 64), "hybrid LFM2 query must have shape [N,32,64]")
    num_tokens = query.shape[0]
    _ensure(tuple(query.stride()[1:]) == (64, 1), "hybrid query heads must be dense")
    empty = Slice(None, 0)
    key_slice, value_slice, kv_stride = empty, empty, 0
    if current_key is not None:
        _ensure(tuple(current_key.shape) == (num_tokens, 8, 64) and current_value.shape == current_key.shape,
                "hybrid contiguous K/V shape mismatch")
        _ensure(tuple(current_key.stride()[1:]) == (64, 1) and current_value.stride() == current_key.stride(),
                "hybrid contiguous K/V must be dense per token and share their token stride")
        key_slice, value_slice = _row_strided_slice(current_key), _row_strided_slice(current_value)
        kv_stride = current_key.stride(0) if num_tokens > 1 else 0
    _ensure(block_tables.dim() == 2, "block tables must have rank 2")
    _ensure(block_tables.shape[1] == block_table_stride, "block table stride/shape mismatch")
    _ensure(request_slots.numel() == num_tokens, "request slot mismatch")
    _ensure(position_ids.numel() == num_tokens, "position mismatch")
    _ensure(segment_offsets.numel() >= 2, "hybrid segments are empty")
    launch = _abi.HybridAttentionLaunch(
        arena.page_size, _row_strided_slice(query), key_slice, value_slice, _slice(arena.key), _slice(arena.value),
        _slice(block_tables), _slice(request_slots), _slice(position_ids), _slice(segment_offsets), _slice(output),
        num_tokens, arena.num_pages, block_table_stride, segment_offsets.numel() - 1,
        query.stride(0) if num_tokens > 1 else 0, kv_stride)
    check(library().lfm25_hybrid_ragged_attention_lfm2_bf16(_stream(), launch))


def paged_ragged_attention_splitk_static_lfm2_bf16_into(inputs: FastRaggedAttentionInput, num_splits: int,
                                                        output: torch.Tensor) -> None:
    """Split-K attention without a caller workspace, for hosts that may not allocate device memory while
    serving: the records go to a fixed array inside the library (at most 128 tokens per call; calls share the
    array, so they must stay ordered on one stream).  No counterpart in the reference."""
    num_tokens = _validate_ragged_input(inputs)
    launch = _abi.FastRaggedAttentionLaunch(
        inputs.arena.page_size, _slice(inputs.query), _slice(inputs.arena.key), _slice(inputs.arena.value),
        _slice(inputs.block_tables), _slice(inputs.request_slots), _slice(inputs.position_ids), _slice(output),
        num_tokens, inputs.arena.num_pages, inputs.block_table_stride, Slice(None, 0))
    check(library().lfm25_paged_ragged_attention_splitk_static_lfm2_bf16(_stream(), launch, num_splits))


# ------------------------------------------------------------------------------- FP8 producers


def quantize_bf16_e4m3_into(values: torch.Tensor, output: torch.Tensor, scale: float) -> None:
    check(library().lfm25_quantize_bf16_e4m3(_stream(), _slice(values), _slice(output), values.numel(), scale))


def silu_mul_packed_bf16_into(packed: torch.Tensor, output: torch.Tensor) -> None:
    """Reference: src/ops/silu_mul.rs (packed [rows, 2I] -> [rows, I])."""
    _ensure(packed.dim() >= 1 and packed.shape[-1] % 2 == 0, "packed silu_mul input must have an even last dimension")
    intermediate = packed.shape[-1] // 2
    rows = packed.numel() // packed.shape[-1] if packed.numel() else 0
    check(library().lfm25_silu_mul_packed_bf16(_stream(), _slice(packed), _slice(output), rows, intermediate))


def silu_mul_packed_bf16_to_e4m3_into(packed: torch.Tensor, output: torch.Tensor, scale: float) -> None:
    """Reference: src/ops/silu_mul.rs:65-100."""
    _ensure(packed.dim() >= 1 and packed.shape[-1] % 2 == 0, "packed silu_mul input must have an even last dimension")
    intermediate = packed.shape[-1] // 2
    rows = packed.numel() // packed.shape[-1] if packed.numel() else 0
    check(library().lfm25_silu_mul_packed_bf16_to_e4m3(_stream(), _slice(packed), _slice(output), rows, intermediate,
                                                       scale))


def linear_fp8_scaled_into(x_codes: torch.Tensor, weight_codes: torch.Tensor, output: torch.Tensor,
                           output_scale: float, scale_mode: int = _abi.FP8_SCALE_TENSORWIDE) -> None:
    """out[M,N] = bf16(output_scale * x[M,K] @ weight[N,K]^T) on E4M3 codes
    (reference: src/model/decode_executor.rs:35-76 -> src/cuda/blaslt/mod.rs:212-298)."""
    _ensure(x_codes.dim() == 2, f"persistent prequantized FP8 linear requires rank-2 input, got {tuple(x_codes.shape)}")
    _ensure(weight_codes.dim() == 2, "persistent prequantized FP8 weight must be rank 2")
    m, k = x_codes.shape
    n = weight_codes.shape[0]
    _ensure(m > 0 and k > 0 and n > 0, "persistent FP8 linear is empty")
    _ensure(weight_codes.shape[1] == k,
            f"persistent prequantized FP8 K mismatch: input K={k}, weight={tuple(weight_codes.shape)}")
    config = _abi.Fp8LinearConfig(m, n, k, scale_mode, output_scale)
    check(library().lfm25_linear_fp8_scaled(_stream(), _slice(x_codes), _slice(weight_codes), _slice(output), config))


class BlasLt:
    """Mirror of the reference's `BlasLt` (src/cuda/blaslt/mod.rs:30-70): bound to the stream that is current at
    construction, owns the 32 MiB workspace.  Its FP8 linear may split K across CTAs (Down-shaped problems)."""

    def __init__(self):
        import ctypes
        self._handle = ctypes.c_void_p()
        self._bound_stream = _stream()
        check(library().lfm25_blaslt_create(self._bound_stream, ctypes.byref(self._handle)))
        torch.cuda.current_stream().synchronize()   # the workspace is zeroed before any other stream may use it

    def workspace_size(self) -> int:
        return int(library().lfm25_blaslt_workspace_size(self._handle))

    def linear_fp8_scaled(self, x_codes, weight_codes, output, output_scale: float,
                          scale_mode: int = _abi.FP8_SCALE_TENSORWIDE) -> None:
        m, k = x_codes.shape
        config = _abi.Fp8LinearConfig(m, weight_codes.shape[0], k, scale_mode, output_scale)
        self.bind_current_stream()
        check(library().lfm25_blaslt_linear_fp8_scaled(self._handle, _slice(x_codes), _slice(weight_codes),
                                                       _slice(output), config))

    def linear_fp8_silu_mul(self, x_codes, weight_codes, activation, output_scale: float,
                            activation_scale: float = 1.0) -> None:
        """Packed Gate/Up FP8 linear with SiLU(gate) * up in the epilogue (one launch for
        src/model/decode_executor.rs:378-402): `activation` [M, N/2] is uint8 (E4M3 codes of the activation times
        `activation_scale`) or bfloat16."""
        m, k = x_codes.shape
        config = _abi.Fp8LinearConfig(m, weight_codes.shape[0], k, _abi.FP8_SCALE_TENSORWIDE, output_scale)
        self.bind_current_stream()
        check(library().lfm25_blaslt_linear_fp8_silu_mul(self._handle, _slice(x_codes), _slice(weight_codes),
                                                         _slice(activation), config, activation_scale,
                                                         1 if activation.dtype == torch.uint8 else 0))

    def bind_current_stream(self) -> None:
        stream = _stream()
        if stream != self._bound_stream:
            check(library().lfm25_blaslt_set_stream(self._handle, stream))
            self._bound_stream = stream

    def linear_bf16(self, x: torch.Tensor, weight: torch.Tensor, output: torch.Tensor) -> None:
        """out[M,N] = x[M,K] @ weight[N,K]^T through cuBLASLt (reference: src/ops/linear.rs linear_bf16_into)."""
        _ensure(weight.dim() == 2, f"linear weight must have rank 2, got {tuple(weight.shape)}")
        k = x.shape[-1]
        _ensure(weight.shape[1] == k, "linear K mismatch")
        rows = x.numel() // k
        self.bind_current_stream()
        check(library().lfm25_blaslt_linear_bf16(self._handle, _slice(x), _slice(weight), _slice(output), rows,
                                                 weight.shape[0], k))

    def linear_bf16_silu_mul(self, x: torch.Tensor, weight: torch.Tensor, activation: torch.Tensor,
                             activation_scale: float = 1.0) -> None:
        """Packed BF16 Gate/Up linear with SiLU(gate) * up in the epilogue; `activation` [M, N/2] is uint8 (E4M3
        codes of the activation times `activation_scale`) or bfloat16."""
        k = x.shape[-1]
        _ensure(weight.dim() == 2 and weight.shape[1] == k, "linear K mismatch")
        rows = x.numel() // k
        self.bind_current_stream()
        check(library().lfm25_blaslt_linear_bf16_silu_mul(self._handle, _slice(x), _slice(weight), _slice(activation),
                                                          rows, weight.shape[0], k, activation_scale,
                                                          1 if activation.dtype == torch.uint8 else 0))

    def set_gemm_tuning(self, kernel: int = 0, n_tile: int = 0, splits: int = 0, stages: int = 0, issuers: int = 0,
                        ctas_per_sm: int = 0, shared_memory_bytes: int = 0, batch_slices: int = 0) -> None:
        """Kernel and tile choice of this handle's linears (0 = the library's choice); no arguments = defaults."""
        tuning = _abi.GemmTuning(kernel, n_tile, splits, stages, issuers, ctas_per_sm, shared_memory_bytes,
                                 batch_slices)
        check(library().lfm25_blaslt_set_gemm_tuning(self._handle, tuning))

    def gemm_plan(self, m: int, n: int, k_bytes: int, gated: bool = False) -> dict:
        """The batch-major kernel's launch plan for a problem under this handle's tuning."""
        import ctypes
        out = (ctypes.c_uint32 * 8)()
        check(library().lfm25_blaslt_gemm_plan(self._handle, m, n, k_bytes, 1 if gated else 0, out))
        names = ("n_tile", "splits", "tiles", "stages", "issuers", "ctas_per_sm", "smem_bytes", "batch_slices")
        return dict(zip(names, (int(value) for value in out)))

    def close(self) -> None:
        if self._handle:
            library().lfm25_blaslt_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def linear_fp8_e4m3(x: torch.Tensor, weight_codes: torch.Tensor, activation_scale, weight_scale) -> torch.Tensor:
    """Quantise a bf16 activation with its static scale, then the FP8 linear
    (reference: src/ops/linear.rs:29-77).  Scales are (quantize_multiplier, dequantize_multiplier) pairs."""
    _ensure(x.dim() >= 1, "FP8 linear input must have rank >= 1")
    _ensure(weight_codes.dim() == 2, "FP8 linear weight must have rank 2")
    _ensure(x.numel() > 0 and weight_codes.numel() > 0, "FP8 linear does not support empty tensors")
    k = x.shape[-1]
    _ensure(weight_codes.shape[1] == k, "FP8 linear K mismatch")
    rows = x.numel() // k
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    quantize_bf16_e4m3_into(x, codes, activation_scale[0])
    output = torch.empty((*x.shape[:-1], weight_codes.shape[0]), dtype=torch.bfloat16, device=x.device)
    linear_fp8_scaled_into(codes, weight_codes, output.view(rows, -1), activation_scale[1] * weight_scale[1])
    return output


def embedding_bf16_into(token_ids: torch.Tensor, weight: torch.Tensor, output: torch.Tensor) -> None:
    check(library().lfm25_embedding_bf16(_stream(), _slice(token_ids), _slice(weight), _slice(output),
                                         token_ids.numel(), weight.shape[0], weight.shape[1]))


def rms_norm_bf16_into(x: torch.Tensor, weight: torch.Tensor, eps: float, output: torch.Tensor) -> None:
    hidden = x.shape[-1]
    check(library().lfm25_rms_norm_bf16(_stream(), _slice(x), _slice(weight), _slice(output), x.numel() // hidden,
                                        hidden, eps))


def residual_rms_norm_bf16_into(residual, update, weight, eps: float, residual_out, normalized_out) -> None:
    hidden = residual.shape[-1]
    check(library().lfm25_residual_rms_norm_bf16(_stream(), _slice(residual), _slice(update), _slice(weight),
                                                 _slice(residual_out), _slice(normalized_out),
                                                 residual.numel() // hidden, hidden, eps))


def residual_rms_norm_bf16_e4m3_into(residual, update, weight, eps: float, residual_out, normalized_out, codes_out,
                                     scale: float) -> None:
    """residual_rms_norm_bf16_into plus the E4M3 codes of the normalised rows (multiplier `scale`) in one launch."""
    hidden = residual.shape[-1]
    check(library().lfm25_residual_rms_norm_bf16_e4m3(_stream(), _slice(residual), _slice(update), _slice(weight),
                                                      _slice(residual_out), _slice(normalized_out), _slice(codes_out),
                                                      residual.numel() // hidden, hidden, eps, scale))


def short_conv_decode_bf16_into(projected, weight, states, request_slots, output) -> None:
    hidden = weight.shape[0]
    check(library().lfm25_short_conv_decode_bf16(_stream(), _slice(projected), _slice(weight), _slice(states),
                                                 _slice(request_slots), _slice(output), request_slots.numel(), hidden,
                                                 states.shape[0]))


def short_conv_segmented_lfm2_bf16_into(projected, weight, states, segment_offsets, segment_slots, output) -> None:
    """Reference: src/ops/short_conv.rs (short_conv_segmented_lfm2_bf16): gated width-3 convolution over token
    segments, one state row per request slot."""
    hidden = weight.shape[0]
    _ensure(projected.dim() == 2 and projected.shape[1] == 3 * hidden, "projected must have shape [N, 3*hidden]")
    _ensure(segment_offsets.numel() == segment_slots.numel() + 1, "segment offsets / slots mismatch")
    check(library().lfm25_short_conv_segmented_lfm2_bf16(
        _stream(), _slice(projected), _slice(weight), _slice(states), _slice(segment_offsets), _slice(segment_slots),
        _slice(output), projected.shape[0], segment_slots.numel(), hidden, states.shape[0]))


def gather_rows_bf16_into(values, row_indices, output) -> None:
    """Reference: src/ops/gather.rs (gather_rows_bf16)."""
    check(library().lfm25_gather_rows_bf16(_stream(), _slice(values), _slice(row_indices), _slice(output),
                                           row_indices.numel(), values.shape[0], values.shape[1]))


def argmax_rows_bf16_into(logits: torch.Tensor, sampled: torch.Tensor) -> None:
    check(library().lfm25_argmax_rows_bf16(_stream(), _slice(logits), _slice(sampled), logits.shape[0],
                                           logits.shape[1]))


def set_option(name: str, value: int) -> None:
    """Process-wide switch of the library (include/lfm25_b200.h: lfm25_set_option)."""
    check(library().lfm25_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    import ctypes
    value = ctypes.c_int64()
    check(library().lfm25_get_option(name.encode(), ctypes.byref(value)))
    return int(value.value)


def device_status() -> tuple[int, int, int, int]:
    """(waits that ran out since the last read, kernel tag, detail, reserved); clears the words."""
    import ctypes
    out = (ctypes.c_uint32 * 4)()
    check(library().lfm25_device_status(_stream(), out))
    return tuple(int(word) for word in out)

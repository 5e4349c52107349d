"""LFM2.5-1.2B-architecture model with random-init weights, its caches, the device-resident decode batch and the
decode executor, as thin wrappers over the C ABI (`lfm25_model`, `lfm25_decode_batch`, `lfm25_decode_executor`).

Architecture constants follow the reference (src/config.rs:55-96): 16 layers, hidden 2048, 32 query / 8 KV heads
of dim 64, gated short convolution of width 3 (in-projection 6144), SwiGLU MLP with intermediate 8192 (Gate/Up
packed to 16384 rows), vocabulary 65536 with the LM head tied to the embedding, RMSNorm eps 1e-5, RoPE theta 1e6.
Attention layers are 2, 5, 8, 10, 12, 14; the promoted FP8 policy covers Gate/Up of layers 2,3,5,7,8,9,11,15,
Down of layers 6,8,9,10,12,14,15 and the LM head (README.md:46-52 of the reference).

There is no checkpoint in this repository: weights are N(0, 0.02) (norm weights 1), E4M3 copies use the per-tensor
scale amax/448, and the static activation scales are fixed constants (no calibration data exists either).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _abi
from ._abi import check, library
from .ops import BlasLt

NUM_LAYERS = 16
HIDDEN = 2048
FFN = 8192
VOCAB = 65536
CONV_WIDTH = 6144
KV_WIDTH = 512
ATTENTION_LAYERS = (2, 5, 8, 10, 12, 14)
FP8_GATE_UP_LAYERS = (2, 3, 5, 7, 8, 9, 11, 15)
FP8_DOWN_LAYERS = (6, 8, 9, 10, 12, 14, 15)
NORM_EPS = 1e-5
ROPE_THETA = 1.0e6
# static activation ranges (c_x) of the promoted sites: inputs after RMSNorm, and SiLU(gate) * up
ACTIVATION_AMAX_NORMALIZED = 8.0
ACTIVATION_AMAX_GATED = 16.0


def rope_inv_freq() -> np.ndarray:
    index = np.arange(32, dtype=np.float32)
    return np.power(np.float32(ROPE_THETA), -(np.float32(2.0) * index) / np.float32(64.0)).astype(np.float32)


@dataclass
class Linear:
    """One linear site: bf16 weight [n, k] and, when promoted, its E4M3 copy with scales."""

    weight: torch.Tensor
    codes: torch.Tensor | None = None
    activation_amax: float = 0.0
    weight_amax: float = 0.0

    def struct(self) -> _abi.LinearWeights:
        site = _abi.Fp8Site(None, 1.0, 1.0, 1.0)
        if self.codes is not None:
            site = _abi.Fp8Site(self.codes.data_ptr(), 448.0 / self.activation_amax, self.activation_amax / 448.0,
                                self.weight_amax / 448.0)
        return _abi.LinearWeights(self.weight.data_ptr(), site, self.weight.shape[0], self.weight.shape[1])


def _promote(linear: Linear, activation_amax: float) -> None:
    weight_amax = float(linear.weight.float().abs().max())
    scaled = (linear.weight.float() * (448.0 / weight_amax)).clamp(-448.0, 448.0)
    linear.codes = scaled.to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    linear.activation_amax = activation_amax
    linear.weight_amax = weight_amax


@dataclass
class LayerState:
    is_attention: bool
    tensors: dict = field(default_factory=dict)
    linears: dict = field(default_factory=dict)


class RandomModel:
    """Random-init weights of the architecture plus per-layer caches, resident on `device`."""

    def __init__(self, seed: int, device, num_pages: int, num_request_slots: int, fp8_policy=True,
                 pack_qkv: bool = True):
        """`fp8_policy`: True = the reference's promoted policy (the 16 sites of FP8_GATE_UP_LAYERS, FP8_DOWN_LAYERS and
        the LM head), False = every site in BF16, or an `fp8_policy.Fp8PrecisionPolicy` loaded from a file in the
        reference's schema: its enabled MLP / LM-head sites are promoted and its static activation scales are used
        (the weight scales are taken from the random weights themselves: amax / 448).
        `pack_qkv`: the query, key and value matrices of a layer share one [3072, 2048] allocation (as a loader
        that concatenates them would leave them), which lets the executor run the three projections as one GEMM;
        False keeps three separate allocations (three GEMMs, the reference's layout)."""
        self.device = device
        self.num_pages = num_pages
        self.num_request_slots = num_request_slots
        generator = torch.Generator(device=device).manual_seed(seed)

        def normal(*shape):
            return (torch.randn(shape, generator=generator, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)

        def ones(count):
            return torch.ones(count, dtype=torch.bfloat16, device=device)

        loaded = fp8_policy if not isinstance(fp8_policy, bool) else None
        gate_up_layers = loaded.layers_with("gate_up") if loaded else (FP8_GATE_UP_LAYERS if fp8_policy else ())
        down_layers = loaded.layers_with("down") if loaded else (FP8_DOWN_LAYERS if fp8_policy else ())
        head_promoted = loaded.lm_head_enabled() if loaded else bool(fp8_policy)

        def activation_amax(site: str, default: float) -> float:
            entry = loaded.site(site) if loaded else None
            return entry.activation_scale.clip_amax if entry is not None else default

        self.embedding = normal(VOCAB, HIDDEN)
        self.final_norm = ones(HIDDEN)
        self.inv_freq = torch.from_numpy(rope_inv_freq()).to(device)
        self.layers: list[LayerState] = []
        for index in range(NUM_LAYERS):
            layer = LayerState(is_attention=index in ATTENTION_LAYERS)
            layer.tensors["operator_norm"] = ones(HIDDEN)
            layer.tensors["ffn_norm"] = ones(HIDDEN)
            if layer.is_attention:
                query, key, value = normal(HIDDEN, HIDDEN), normal(KV_WIDTH, HIDDEN), normal(KV_WIDTH, HIDDEN)
                if pack_qkv:
                    packed = torch.cat([query, key, value], dim=0).contiguous()
                    query, key, value = (packed[:HIDDEN], packed[HIDDEN:HIDDEN + KV_WIDTH],
                                         packed[HIDDEN + KV_WIDTH:])
                    layer.tensors["qkv_packed"] = packed
                layer.linears["query"] = Linear(query)
                layer.linears["key"] = Linear(key)
                layer.linears["value"] = Linear(value)
                layer.linears["output"] = Linear(normal(HIDDEN, HIDDEN))
                layer.tensors["query_norm"] = ones(64)
                layer.tensors["key_norm"] = ones(64)
                layer.tensors["key_cache"] = torch.zeros((num_pages, 8, 16, 64), dtype=torch.bfloat16, device=device)
                layer.tensors["value_cache"] = torch.zeros((num_pages, 8, 16, 64), dtype=torch.bfloat16, device=device)
            else:
                layer.linears["conv_input"] = Linear(normal(CONV_WIDTH, HIDDEN))
                layer.linears["conv_output"] = Linear(normal(HIDDEN, HIDDEN))
                layer.tensors["conv_kernel"] = (torch.randn((HIDDEN, 3), generator=generator, device=device) * 0.5).to(
                    torch.bfloat16)
                layer.tensors["conv_state"] = torch.zeros((num_request_slots, HIDDEN, 2), dtype=torch.bfloat16,
                                                          device=device)
            layer.linears["gate_up"] = Linear(normal(2 * FFN, HIDDEN))
            layer.linears["down"] = Linear(normal(HIDDEN, FFN))
            if index in gate_up_layers:
                _promote(layer.linears["gate_up"], activation_amax(f"layers.{index}.mlp.gate_up",
                                                                   ACTIVATION_AMAX_NORMALIZED))
            if index in down_layers:
                _promote(layer.linears["down"], activation_amax(f"layers.{index}.mlp.down", ACTIVATION_AMAX_GATED))
            self.layers.append(layer)
        self.lm_head = Linear(self.embedding)
        if head_promoted:
            _promote(self.lm_head, activation_amax("lm_head", ACTIVATION_AMAX_NORMALIZED))
        self._build_struct()

    def _build_struct(self) -> None:
        empty = _abi.LinearWeights(None, _abi.Fp8Site(None, 1.0, 1.0, 1.0), 0, 0)
        array = (_abi.Layer * NUM_LAYERS)()
        for index, layer in enumerate(self.layers):
            tensors, linears = layer.tensors, layer.linears

            def pointer(name):
                return tensors[name].data_ptr() if name in tensors else None

            def linear(name):
                return linears[name].struct() if name in linears else empty

            array[index] = _abi.Layer(
                1 if layer.is_attention else 0, pointer("operator_norm"), pointer("ffn_norm"), linear("conv_input"),
                pointer("conv_kernel"), linear("conv_output"), pointer("conv_state"), linear("query"), linear("key"),
                linear("value"), linear("output"), pointer("query_norm"), pointer("key_norm"), pointer("key_cache"),
                pointer("value_cache"), linear("gate_up"), linear("down"))
        self._layer_array = array
        head = self.lm_head.struct().fp8
        self.struct = _abi.Model(NUM_LAYERS, array, self.embedding.data_ptr(), head, self.final_norm.data_ptr(),
                                 self.inv_freq.data_ptr(), NORM_EPS, self.num_pages, self.num_request_slots)

    def fill_caches(self, seed: int) -> None:
        """KV pools and convolution states ~ N(0,1): stricter than the reference's own benchmark, which leaves the
        primed context zero (src/model/lfm2_base.rs:292-320)."""
        generator = torch.Generator(device=self.device).manual_seed(seed)
        for layer in self.layers:
            for name in ("key_cache", "value_cache", "conv_state"):
                if name in layer.tensors:
                    tensor = layer.tensors[name]
                    tensor.copy_(torch.randn(tensor.shape, generator=generator, device=self.device,
                                             dtype=torch.bfloat16))

    def weight_bytes(self, use_fp8: bool) -> int:
        """Bytes of weights one decode step streams (each site once; FP8 sites at one byte per weight)."""
        total = 0
        for layer in self.layers:
            for linear in layer.linears.values():
                total += linear.weight.numel() * (1 if (use_fp8 and linear.codes is not None) else 2)
        total += self.embedding.numel() * (1 if (use_fp8 and self.lm_head.codes is not None) else 2)
        return total


class DecodeBatch:
    """Device-resident metadata of a pure-decode batch (one token per sequence)."""

    def __init__(self, device, block_tables: np.ndarray, request_slots: np.ndarray, positions: np.ndarray,
                 token_ids: np.ndarray, max_context_tokens: int):
        def u32(values):
            return torch.from_numpy(np.ascontiguousarray(values, dtype=np.uint32).view(np.int32).copy()).to(device)

        self.block_tables = u32(block_tables)
        self.num_tokens = int(len(positions))
        # token ids | positions | request slots in one allocation: a serving loop that supplies them from the host
        # uploads the step's metadata with one copy (the reference packs its slab the same way,
        # src/scheduler/batch.rs:26-53)
        self.step_metadata = u32(np.concatenate([np.asarray(token_ids, dtype=np.uint32),
                                                 np.asarray(positions, dtype=np.uint32),
                                                 np.asarray(request_slots, dtype=np.uint32)]))
        self.token_ids = self.step_metadata[:self.num_tokens]
        self.positions = self.step_metadata[self.num_tokens:2 * self.num_tokens]
        self.request_slots = self.step_metadata[2 * self.num_tokens:]
        self.physical_slots = torch.zeros(self.num_tokens, dtype=torch.int64, device=device)
        self.struct = _abi.DecodeBatch(
            self.token_ids.data_ptr(), self.positions.data_ptr(), self.request_slots.data_ptr(),
            self.physical_slots.data_ptr(), self.block_tables.data_ptr(), block_tables.shape[1], block_tables.shape[0],
            self.num_tokens, max_context_tokens)


def leading_decode_segments(batch) -> tuple[int, int]:
    """(number of leading single-token segments of a `workloads.MixedStepBatch`, longest context among them)."""
    count = 0
    while count < batch.num_segments and batch.chunks[count] == 1:
        count += 1
    context = int(batch.prefixes[:count].max()) + 1 if count else 0
    return count, context


class RaggedBatch:
    """Device-resident metadata of a step that mixes prefill chunks and decode tokens
    (a `workloads.MixedStepBatch` plus the token ids)."""

    def __init__(self, device, batch, token_ids: np.ndarray):
        def u32(values):
            return torch.from_numpy(np.ascontiguousarray(values, dtype=np.uint32).view(np.int32).copy()).to(device)

        self.block_tables = u32(batch.block_tables)
        self.request_slots = u32(batch.request_slots)
        self.positions = u32(batch.positions)
        self.token_ids = u32(token_ids)
        self.segment_offsets = u32(batch.segment_offsets)
        self.segment_slots = u32(batch.segment_slots)
        self.output_rows = u32(batch.output_rows)
        self.num_tokens = batch.num_tokens
        self.num_segments = batch.num_segments
        self.physical_slots = torch.zeros(self.num_tokens, dtype=torch.int64, device=device)
        decode_segments, decode_context = leading_decode_segments(batch)
        self.struct = _abi.RaggedBatch(
            self.token_ids.data_ptr(), self.positions.data_ptr(), self.request_slots.data_ptr(),
            self.physical_slots.data_ptr(), self.segment_offsets.data_ptr(), self.segment_slots.data_ptr(),
            self.output_rows.data_ptr(), self.block_tables.data_ptr(), batch.block_tables.shape[1],
            batch.block_tables.shape[0], self.num_tokens, self.num_segments, decode_segments, decode_context)


class DecodeExecutor:
    """Mirror of the reference's DecodeExecutor over the C ABI; bound to the BlasLt handle's stream.
    `maximum_segments` (sequences per step) below `maximum_tokens` makes room for prefill chunks."""

    def __init__(self, blaslt: BlasLt, maximum_tokens: int, maximum_segments: int | None = None):
        self.blaslt = blaslt
        self.maximum_tokens = maximum_tokens
        self._handle = ctypes.c_void_p()
        if maximum_segments is None:
            check(library().lfm25_decode_executor_create(blaslt._handle, maximum_tokens, ctypes.byref(self._handle)))
        else:
            check(library().lfm25_decode_executor_create_ragged(blaslt._handle, maximum_tokens, maximum_segments,
                                                                ctypes.byref(self._handle)))

    def forward_ragged(self, model: RandomModel, batch: RaggedBatch, use_fp8: bool = True) -> None:
        """One mixed prefill / decode step; row s of logits / sampled belongs to segment s."""
        self.blaslt.bind_current_stream()
        check(library().lfm25_decode_executor_forward_ragged(self._handle, model.struct, batch.struct, int(use_fp8)))

    def forward(self, model: RandomModel, batch: DecodeBatch, use_fp8: bool = True, advance: bool = False) -> None:
        self.blaslt.bind_current_stream()
        check(library().lfm25_decode_executor_forward(self._handle, model.struct, batch.struct, int(use_fp8),
                                                      int(advance)))

    def step_graph(self, model: RandomModel, batch: DecodeBatch, use_fp8: bool = True, advance: bool = True) -> None:
        self.blaslt.bind_current_stream()
        check(library().lfm25_decode_executor_step_graph(self._handle, model.struct, batch.struct, int(use_fp8),
                                                         int(advance)))

    def serve_step(self, model: RandomModel, batch: DecodeBatch, host_metadata: torch.Tensor,
                   host_sampled: torch.Tensor, use_fp8: bool = True) -> None:
        """One served step in one call: `host_metadata` (pinned int32 [3 * tokens]: token ids | positions | request
        slots) goes to the device, the captured step replays, the sampled ids land in `host_sampled` (pinned int32
        [tokens]) and the stream is synchronised (src/engine/serving/radix_owner.rs:230-259)."""
        if not (host_metadata.is_pinned() and host_sampled.is_pinned()):
            raise ValueError("served step needs pinned host buffers")
        if host_metadata.numel() < 3 * batch.num_tokens or host_sampled.numel() < batch.num_tokens:
            raise ValueError("served step host buffers are too small")
        self.blaslt.bind_current_stream()
        check(library().lfm25_decode_executor_serve_step(self._handle, model.struct, batch.struct, int(use_fp8),
                                                         host_metadata.data_ptr(), host_sampled.data_ptr()))

    def graph_kernels(self) -> int:
        """GPU kernels per step in the graph that the last step_graph call replayed (0 before the first replay)."""
        return int(library().lfm25_decode_executor_graph_kernels(self._handle))

    def graph_captures(self) -> int:
        """Steps captured so far; a change of anything a captured step baked in makes the next call capture again."""
        return int(library().lfm25_decode_executor_graph_captures(self._handle))

    REGIONS = ("attention", "append", "fp8_linear", "bf16_linear", "other")

    def profile(self, enable: bool, collect: bool = False):
        """Switches region timing of eager steps on or off; with collect=True returns {region: (ms, ops)} first."""
        if not collect:
            check(library().lfm25_decode_executor_profile(self._handle, int(enable), None, None))
            return None
        milliseconds = (ctypes.c_float * len(self.REGIONS))()
        launches = (ctypes.c_uint32 * len(self.REGIONS))()
        check(library().lfm25_decode_executor_profile(self._handle, int(enable), milliseconds, launches))
        return {name: (float(milliseconds[i]), int(launches[i])) for i, name in enumerate(self.REGIONS)}

    def download_sampled(self, host: torch.Tensor) -> None:
        check(library().lfm25_decode_executor_download_sampled(self._handle, host.data_ptr(), host.numel()))

    def download_logits(self, host: torch.Tensor) -> None:
        check(library().lfm25_decode_executor_download_logits(self._handle, host.data_ptr(), host.shape[0]))

    def sampled(self, count: int) -> np.ndarray:
        host = torch.empty(count, dtype=torch.int32).pin_memory()
        self.download_sampled(host)
        torch.cuda.current_stream().synchronize()
        return host.numpy().view(np.uint32).copy()

    def logits(self, rows: int) -> np.ndarray:
        host = torch.empty((rows, VOCAB), dtype=torch.bfloat16).pin_memory()
        self.download_logits(host)
        torch.cuda.current_stream().synchronize()
        return host.view(torch.int16).numpy().view(np.uint16).copy()

    def close(self) -> None:
        if self._handle:
            library().lfm25_decode_executor_destroy(self._handle)
            self._handle = None

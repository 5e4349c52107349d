"""One decode step assembled from the reference's own CUDA kernels and cuBLASLt.  TEST INFRASTRUCTURE ONLY.

The reference's step (src/model/decode_executor.rs:183-443) is a sequence of its `kernels/*.cu` launches with
cuBLASLt GEMMs between them (BF16, and E4M3 with a per-tensor scale at the promoted sites: src/cuda/blaslt/mod.rs:212-298).
Its Rust host cannot be built without a Rust toolchain, so this module replays that sequence from Python: the kernels
are the reference's unmodified sources compiled for sm_100a (`oracle/_ref/*.cubin`, launched with the reference's grid
shapes by `refkernels`), and the GEMMs are `torch.matmul` (cuBLAS / cuBLASLt BF16) and `torch._scaled_mm` (cuBLASLt
FP8), the same library the reference calls.  Every buffer has a fixed address, so the sequence can be captured in a CUDA
graph: replaying the graph times the reference's kernels without any launch or host overhead, which is an upper bound
on what the reference's own launch loop (one stream, no graph, host bookkeeping and a synchronisation per step) reaches.

It is used to compare results with the new executor at the level of the whole step and as the
"reference kernels on the same GPU" number of the step benchmark.  Nothing in the product imports it.
"""
from __future__ import annotations

import torch

from . import refkernels

HIDDEN, KV_WIDTH, FFN, VOCAB, CONV_WIDTH = 2048, 512, 8192, 65536, 6144


class ReferenceKernelStep:
    """`model` is the package's RandomModel (weights, E4M3 copies, caches); `tokens` the decode batch size."""

    def __init__(self, model, tokens: int, use_fp8: bool = True, eps: float = 1e-5):
        if not refkernels.available():
            raise RuntimeError("oracle/_ref holds no compiled reference kernels (run `make -C oracle ref`)")
        self.model, self.tokens, self.use_fp8, self.eps = model, tokens, use_fp8, eps
        device = model.device

        def bf16(*shape):
            return torch.zeros(shape, dtype=torch.bfloat16, device=device)

        # the scratch set of the reference's executor (src/model/decode_executor.rs:6-22)
        self.hidden, self.post_operator = bf16(tokens, HIDDEN), bf16(tokens, HIDDEN)
        self.normalized, self.operator_output = bf16(tokens, HIDDEN), bf16(tokens, HIDDEN)
        self.operator_input = bf16(tokens, HIDDEN)
        self.query, self.key, self.value = bf16(tokens, HIDDEN), bf16(tokens, KV_WIDTH), bf16(tokens, KV_WIDTH)
        self.projected = bf16(tokens, CONV_WIDTH)
        self.wide, self.activated = bf16(tokens, 2 * FFN), bf16(tokens, FFN)
        self.logits = bf16(tokens, VOCAB)
        self.fp8_input = torch.zeros((tokens, FFN), dtype=torch.uint8, device=device)
        self.sampled = torch.zeros(tokens, dtype=torch.int32, device=device)
        self.segment_offsets = torch.arange(tokens + 1, dtype=torch.int32, device=device)
        self._scales = {}
        self.launches = 0

    def _scale(self, value: float) -> torch.Tensor:
        if value not in self._scales:
            self._scales[value] = torch.tensor(value, dtype=torch.float32, device=self.model.device)
        return self._scales[value]

    def _linear(self, site, values: torch.Tensor, output: torch.Tensor) -> None:
        """linear_decode_into (src/model/decode_executor.rs:78-124): quantise + FP8 GEMM at a promoted site, BF16
        GEMM elsewhere."""
        if self.use_fp8 and site.codes is not None:
            codes = self.fp8_input.view(-1)[:values.numel()].view(values.shape)
            refkernels.quantize_bf16_e4m3(values, codes, 448.0 / site.activation_amax)
            self.launches += 1
            self._linear_fp8(site, codes, output)
        else:
            torch.matmul(values, site.weight.t(), out=output)
            self.launches += 1

    def _linear_fp8(self, site, codes: torch.Tensor, output: torch.Tensor) -> None:
        torch._scaled_mm(codes.view(torch.float8_e4m3fn), site.codes.view(torch.float8_e4m3fn).t(),
                         scale_a=self._scale(site.activation_amax / 448.0),
                         scale_b=self._scale(site.weight_amax / 448.0), out_dtype=torch.bfloat16, out=output)
        self.launches += 1

    def forward(self, token_ids, positions, request_slots, physical_slots, block_tables) -> None:
        """Device tensors: `token_ids`, `positions`, `request_slots` uint32-as-int32 [tokens]; `physical_slots` int64
        [tokens]; `block_tables` [slots, stride].  Results in `self.logits` and `self.sampled`."""
        model, eps = self.model, self.eps
        launch = refkernels
        self.launches = 0
        launch.embedding(token_ids, model.embedding, self.hidden)
        launch.rms_norm(self.hidden, model.layers[0].tensors["operator_norm"], self.normalized, eps)
        self.launches += 2
        for index, layer in enumerate(model.layers):
            tensors, linears = layer.tensors, layer.linears
            if not layer.is_attention:
                self._linear(linears["conv_input"], self.normalized, self.projected)
                launch.short_conv_segmented(self.projected, tensors["conv_kernel"], tensors["conv_state"],
                                            self.segment_offsets, request_slots, self.operator_input)
                self._linear(linears["conv_output"], self.operator_input, self.operator_output)
                self.launches += 1
            else:
                self._linear(linears["query"], self.normalized, self.query)
                self._linear(linears["key"], self.normalized, self.key)
                self._linear(linears["value"], self.normalized, self.value)
                launch.qk_norm_rope_kv_write_decode(self.query, self.key, self.value, tensors["query_norm"],
                                                    tensors["key_norm"], model.inv_freq, positions, physical_slots,
                                                    tensors["key_cache"], tensors["value_cache"], eps)
                # more than 32 tokens: the unsplit kernel (src/ops/splitk_policy.rs:15-78)
                launch.paged_ragged_attention_fast(self.query, tensors["key_cache"], tensors["value_cache"],
                                                   block_tables, request_slots, positions, self.operator_input)
                self._linear(linears["output"], self.operator_input, self.operator_output)
                self.launches += 2
            launch.residual_rms_norm(self.hidden, self.operator_output, tensors["ffn_norm"], self.post_operator,
                                     self.normalized, eps)
            self._linear(linears["gate_up"], self.normalized, self.wide)
            down = linears["down"]
            if self.use_fp8 and down.codes is not None:
                codes = self.fp8_input[:, :FFN]
                launch.silu_mul_packed_bf16_to_e4m3(self.wide, codes, 448.0 / down.activation_amax)
                self._linear_fp8(down, codes, self.operator_output)
            else:
                launch.silu_mul_packed_bf16(self.wide, self.activated)
                torch.matmul(self.activated, down.weight.t(), out=self.operator_output)
                self.launches += 1
            following = (model.layers[index + 1].tensors["operator_norm"] if index + 1 < len(model.layers)
                         else model.final_norm)
            launch.residual_rms_norm(self.post_operator, self.operator_output, following, self.hidden,
                                     self.normalized, eps)
            self.launches += 3
        self._linear(model.lm_head, self.normalized, self.logits)
        launch.argmax_rows(self.logits, self.sampled)
        self.launches += 1

"""CPU restatement of one decode step of the model (the op sequence of the reference's
DecodeExecutor::forward_prepared, src/model/decode_executor.rs:183-443), built from the oracle's ops.
TEST INFRASTRUCTURE ONLY."""
import numpy as np

from . import oracle


def to_bits(tensor):
    import torch
    return tensor.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


class HostModel:
    """Weights and caches of a `RandomModel`, downloaded as bit patterns."""

    def __init__(self, model):
        self.layers = []
        for layer in model.layers:
            entry = {"is_attention": layer.is_attention}
            for name, tensor in layer.tensors.items():
                entry[name] = to_bits(tensor).copy()
            for name, linear in layer.linears.items():
                entry[name] = self._linear(linear)
            self.layers.append(entry)
        self.embedding = to_bits(model.embedding)
        self.lm_head = self._linear(model.lm_head)
        self.final_norm = to_bits(model.final_norm)
        self.inv_freq = model.inv_freq.cpu().numpy()

    @staticmethod
    def _linear(linear):
        site = {"weight": to_bits(linear.weight)}
        if linear.codes is not None:
            site["codes"] = linear.codes.cpu().numpy()
            site["quantize"] = np.float32(448.0) / np.float32(linear.activation_amax)
            site["dequantize"] = np.float32(np.float32(linear.activation_amax) / np.float32(448.0)) * np.float32(
                np.float32(linear.weight_amax) / np.float32(448.0))
        return site


def linear(site, x_bits, use_fp8):
    if use_fp8 and "codes" in site:
        return oracle.linear_fp8(oracle.quantize_bf16_e4m3(x_bits, float(site["quantize"])), site["codes"],
                                 float(site["dequantize"]))
    return oracle.linear_bf16(x_bits, site["weight"])


def decode_step(host: HostModel, token_ids, positions, request_slots, block_tables, use_fp8, eps=1e-5):
    """Runs one step in place on the host caches; returns (logits bits [T, V], sampled [T])."""
    tokens = len(token_ids)
    slots = oracle.physical_slots(block_tables, request_slots, positions)
    hidden = host.embedding[np.asarray(token_ids, dtype=np.int64)].copy()
    normalized = oracle.rms_norm_bf16(hidden, host.layers[0]["operator_norm"], eps)
    for index, layer in enumerate(host.layers):
        if not layer["is_attention"]:
            wide = linear(layer["conv_input"], normalized, use_fp8)
            post = oracle.short_conv_decode_bf16(wide, layer["conv_kernel"], layer["conv_state"], request_slots)
            operator_output = linear(layer["conv_output"], post, use_fp8)
        else:
            query = linear(layer["query"], normalized, use_fp8).reshape(tokens, 32, 64).copy()
            key = linear(layer["key"], normalized, use_fp8).reshape(tokens, 8, 64)
            value = linear(layer["value"], normalized, use_fp8).reshape(tokens, 8, 64)
            oracle.qk_norm_rope_kv_write_decode(query, key, value, layer["query_norm"], layer["key_norm"],
                                                host.inv_freq, np.asarray(positions, dtype=np.uint32), slots,
                                                layer["key_cache"], layer["value_cache"], eps)
            attended = oracle.paged_ragged_attention(query, layer["key_cache"], layer["value_cache"], block_tables,
                                                     request_slots, positions)
            operator_output = linear(layer["output"], attended.reshape(tokens, 2048), use_fp8)
        post_operator, normalized = oracle.residual_rms_norm_bf16(hidden, operator_output, layer["ffn_norm"], eps)
        wide = linear(layer["gate_up"], normalized, use_fp8)
        down = layer["down"]
        if use_fp8 and "codes" in down:
            _, codes = oracle.silu_mul_packed(wide, float(down["quantize"]))
            operator_output = oracle.linear_fp8(codes, down["codes"], float(down["dequantize"]))
        else:
            activated, _ = oracle.silu_mul_packed(wide, 1.0)
            operator_output = oracle.linear_bf16(activated, down["weight"])
        next_norm = host.layers[index + 1]["operator_norm"] if index + 1 < len(host.layers) else host.final_norm
        hidden, normalized = oracle.residual_rms_norm_bf16(post_operator, operator_output, next_norm, eps)
    logits = linear(host.lm_head, normalized, use_fp8)
    return logits, oracle.argmax_rows_bf16(logits)


def ragged_step(host: HostModel, token_ids, batch, use_fp8, eps=1e-5):
    """One step that mixes prefill chunks and decode tokens (the reference's Lfm2Model::forward_prepared_batch,
    src/model/lfm2_base.rs:924-997, with attention_batch's prefill branch :1794-1829): `batch` is a
    workloads.MixedStepBatch.  Runs in place on the host caches; returns (logits bits [S, V] of each segment's
    last token, sampled [S]).  QK-norm and RoPE use the fused decode formulation for every token (the prefill
    branch's three kernels compute the same values up to the summation order of the 64-wide RMS)."""
    tokens = len(token_ids)
    positions, request_slots = batch.positions, batch.request_slots
    slots = batch.physical_slots
    hidden = host.embedding[np.asarray(token_ids, dtype=np.int64)].copy()
    normalized = oracle.rms_norm_bf16(hidden, host.layers[0]["operator_norm"], eps)
    for index, layer in enumerate(host.layers):
        if not layer["is_attention"]:
            wide = linear(layer["conv_input"], normalized, use_fp8)
            post = oracle.short_conv_segmented_bf16(wide, layer["conv_kernel"], layer["conv_state"],
                                                    batch.segment_offsets, batch.segment_slots)
            operator_output = linear(layer["conv_output"], post, use_fp8)
        else:
            query = linear(layer["query"], normalized, use_fp8).reshape(tokens, 32, 64).copy()
            key = linear(layer["key"], normalized, use_fp8).reshape(tokens, 8, 64)
            value = linear(layer["value"], normalized, use_fp8).reshape(tokens, 8, 64)
            oracle.qk_norm_rope_kv_write_decode(query, key, value, layer["query_norm"], layer["key_norm"],
                                                host.inv_freq, positions, slots, layer["key_cache"],
                                                layer["value_cache"], eps)
            # with the chunk appended, attending through the block tables equals the hybrid kernel
            attended = oracle.paged_ragged_attention(query, layer["key_cache"], layer["value_cache"],
                                                     batch.block_tables, request_slots, positions)
            operator_output = linear(layer["output"], attended.reshape(tokens, 2048), use_fp8)
        post_operator, normalized = oracle.residual_rms_norm_bf16(hidden, operator_output, layer["ffn_norm"], eps)
        wide = linear(layer["gate_up"], normalized, use_fp8)
        down = layer["down"]
        if use_fp8 and "codes" in down:
            _, codes = oracle.silu_mul_packed(wide, float(down["quantize"]))
            operator_output = oracle.linear_fp8(codes, down["codes"], float(down["dequantize"]))
        else:
            activated, _ = oracle.silu_mul_packed(wide, 1.0)
            operator_output = oracle.linear_bf16(activated, down["weight"])
        next_norm = host.layers[index + 1]["operator_norm"] if index + 1 < len(host.layers) else host.final_norm
        hidden, normalized = oracle.residual_rms_norm_bf16(post_operator, operator_output, next_norm, eps)
    logits = linear(host.lm_head, normalized[batch.output_rows.astype(np.int64)], use_fp8)
    return logits, oracle.argmax_rows_bf16(logits)

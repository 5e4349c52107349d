"""Generates tests/golden/reference_b200.npz: outputs of the reference project's own, unmodified CUDA kernels
(compiled for sm_100a into oracle/_ref/*.cubin by `make -C oracle ref`) on the inputs of tests/cases.py, and of
cuBLASLt's E4M3 GEMM -- the library the reference calls for its FP8 linears (src/cuda/blaslt/mod.rs:212-298),
here through torch._scaled_mm -- on the 15 points of the decode GEMM sweep (a sample of 128 output columns each).

Run on a B200:   python tests/golden/make_golden.py <output.npz>
The fixture pins the CPU oracle (tests/test_oracle_golden.py runs without a GPU) to what the reference
actually computes.  Inputs are not stored: tests/cases.py rebuilds them from their seeds."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
import cases  # noqa: E402
from conftest import bits_of, to_bf16, to_i64, to_u32  # noqa: E402
from oracle import refkernels  # noqa: E402


def attention_outputs(case, device, splits=()):
    tensors = dict(query=to_bf16(case["query"], device), key_cache=to_bf16(case["key_cache"], device),
                   value_cache=to_bf16(case["value_cache"], device), block_tables=to_u32(case["block_tables"], device),
                   request_slots=to_u32(case["request_slots"], device),
                   position_ids=to_u32(case["position_ids"], device))
    out = {}
    for name, function in (("precise", refkernels.paged_ragged_attention_precise),
                           ("fast", refkernels.paged_ragged_attention_fast)):
        output = torch.zeros_like(tensors["query"])
        function(*tensors.values(), output)
        out[name] = bits_of(output)
    for count in splits:
        tokens = case["query"].shape[0]
        partials = torch.zeros((tokens, 32, count, 66), dtype=torch.float32, device=device)
        output = torch.zeros_like(tensors["query"])
        refkernels.paged_ragged_attention_splitk(*tensors.values(), partials, output, count)
        out[f"splitk{count}"] = bits_of(output)
        out[f"partials{count}"] = partials.cpu().numpy()
    return out


def cublaslt_fp8_outputs(device):
    """fp8_<site>_<m>: bf16 bits [m, 128] of cuBLASLt's E4M3 GEMM on the sampled columns of cases.fp8_gemm_point.
    cuBLASLt wants both GEMM extents in multiples of 16, so smaller batches are padded with zero rows."""
    out = {}
    one = torch.ones((), device=device)
    for site in cases.FP8_GEMM_SITES:
        weights = torch.from_numpy(cases.fp8_gemm_sampled_weights(site)).to(device).view(torch.float8_e4m3fn)
        for m in cases.FP8_GEMM_BATCHES:
            x_codes, scale, _ = cases.fp8_gemm_point(site, m)
            padded = np.zeros(((m + 15) // 16 * 16, x_codes.shape[1]), dtype=np.uint8)
            padded[:m] = x_codes
            activations = torch.from_numpy(padded).to(device).view(torch.float8_e4m3fn)
            result = torch._scaled_mm(activations, weights.t(), scale_a=one * scale, scale_b=one,
                                      out_dtype=torch.bfloat16)
            out[f"fp8_{site}_{m}"] = bits_of(result[:m])
    return out


def main(path):
    device = torch.device("cuda:0")
    golden = {}
    golden.update(cublaslt_fp8_outputs(device))
    for context in cases.SINGLE_CONTEXTS:
        for name, bits in attention_outputs(cases.single_context_case(context), device).items():
            golden[f"single{context}_{name}"] = bits
    for name, bits in attention_outputs(cases.ragged_reversed_case(), device).items():
        golden[f"reversed_{name}"] = bits
    for name, bits in attention_outputs(cases.splitk_case(), device, splits=(2, 4, 8)).items():
        golden[f"splitk_{name}"] = bits
    for name, bits in attention_outputs(cases.random_ragged_case(7, 6, 1, 700, 512), device, splits=(4,)).items():
        golden[f"random_{name}"] = bits

    case = cases.qk_postprocess_case()
    query = to_bf16(case["query"], device)
    key_cache = torch.zeros((case["num_pages"], 8, 16, 64), dtype=torch.bfloat16, device=device)
    value_cache = torch.zeros_like(key_cache)
    refkernels.qk_norm_rope_kv_write_decode(
        query, to_bf16(case["key"], device), to_bf16(case["value"], device), to_bf16(case["query_norm"], device),
        to_bf16(case["key_norm"], device), torch.from_numpy(case["inv_freq"]).to(device),
        to_u32(case["position_ids"], device), to_i64(case["slot_mapping"], device), key_cache, value_cache,
        case["eps"])
    golden["qk_query"] = bits_of(query)
    golden["qk_key_cache"] = bits_of(key_cache)
    golden["qk_value_cache"] = bits_of(value_cache)

    values, packed = cases.fp8_inputs()
    codes = torch.zeros(values.shape, dtype=torch.uint8, device=device)
    refkernels.quantize_bf16_e4m3(to_bf16(values, device), codes, 3.25)
    golden["quantize_codes"] = codes.cpu().numpy()
    hidden = torch.zeros(values.shape, dtype=torch.bfloat16, device=device)
    refkernels.silu_mul_packed_bf16(to_bf16(packed, device), hidden)
    golden["silu_hidden"] = bits_of(hidden)
    fused = torch.zeros(values.shape, dtype=torch.uint8, device=device)
    refkernels.silu_mul_packed_bf16_to_e4m3(to_bf16(packed, device), fused, 9.75)
    golden["silu_codes"] = fused.cpu().numpy()

    # mixed prefill / decode step: the reference's hybrid attention and segmented short convolution
    hybrid_cases = {"hybrid_known": cases.hybrid_known_answer_case(),
                    "hybrid_mixed": cases.mixed_step_case(5, *cases.MIXED_SMALL, 64)}
    for name, case in hybrid_cases.items():
        case.pop("batch", None)
        output = torch.zeros(case["query"].shape, dtype=torch.bfloat16, device=device)
        refkernels.hybrid_ragged_attention(
            to_bf16(case["query"], device), to_bf16(case["current_key"], device),
            to_bf16(case["current_value"], device), to_bf16(case["key_cache"], device),
            to_bf16(case["value_cache"], device), to_u32(case["block_tables"], device),
            to_u32(case["request_slots"], device), to_u32(case["position_ids"], device),
            to_u32(case["segment_offsets"], device), output)
        golden[name] = bits_of(output)
    case = cases.short_conv_segmented_case()
    states = to_bf16(case["states"], device)
    output = torch.zeros((case["projected"].shape[0], case["weight"].shape[0]), dtype=torch.bfloat16, device=device)
    refkernels.short_conv_segmented(to_bf16(case["projected"], device), to_bf16(case["weight"], device), states,
                                    to_u32(case["segment_offsets"], device), to_u32(case["segment_slots"], device),
                                    output)
    golden["conv_segmented_output"] = bits_of(output)
    golden["conv_segmented_states"] = bits_of(states)

    torch.cuda.synchronize()
    np.savez_compressed(path, **golden)
    print(f"wrote {len(golden)} arrays to {path}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_b200.npz"))

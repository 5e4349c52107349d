"""Sweep of the E4M3 decode GEMMs: packed Gate/Up 2048->16384, Down 8192->2048, LM head 2048->65536 at
M in {1, 8, 32, 128, 256}; weights ~ N(0, 0.02) and activations ~ N(0, 1) quantised per tensor (amax / 448).

    python lfm25-inference_b200/bench_fp8_gemm.py [--iterations 200] [--ms 1 8 32 128 256] [--no-cublaslt]

Launches are timed on the GPU by replaying a CUDA graph of them.
For every point one JSON line: microseconds per launch with HBM-cold weights (the launches rotate over a ring
of distinct weight copies of at least 512 MB, larger than L2) and with L2-warm weights (one copy), the
algorithmic bytes and flops, the achieved GB/s against the measured HBM copy peak, and -- next to it -- cuBLASLt's
FP8 GEMM on the same buffers through torch._scaled_mm (what the reference runtime calls for these sites).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

SHAPES = [("gate_up", 16384, 2048), ("down", 2048, 8192), ("lm_head", 65536, 2048)]
# BF16 sites of the decode step (reference src/model/lfm2.rs: conv in/out projections, q/k/v/o, the FFN of the
# layers outside the FP8 policy)
BF16_SHAPES = [("conv_in", 6144, 2048), ("proj_2048", 2048, 2048), ("kv_proj", 512, 2048),
               ("ffn_w1", 8192, 2048), ("ffn_w2", 2048, 8192)]
RING_BYTES = 512 << 20


def time_launches(function, count, replays=5):
    """Microseconds per launch, GPU-side: `count` launches are captured in a CUDA graph and the graph is replayed,
    so the host's launch cadence (Python + ctypes) does not enter the number."""
    for index in range(3):
        function(index)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for index in range(count):
                function(index)
    graph.replay()
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / (count * replays)


def sweep_bf16(arguments, ops, device, hbm_peak):
    """BF16 sites: this library's tcgen05 kernel (LFM25_BF16_GEMM=umma) beside cuBLASLt through the same handle."""
    generator = torch.Generator(device=device).manual_seed(3)
    blaslt = ops.BlasLt()
    for name, n, k in BF16_SHAPES:
        if arguments.shapes and name not in arguments.shapes:
            continue
        copies = max(2, (RING_BYTES + 2 * n * k - 1) // (2 * n * k))
        ring = [(torch.randn((n, k), generator=generator, device=device) * 0.02).to(torch.bfloat16)
                for _ in range(copies)]
        for m in arguments.ms:
            x = torch.randn((m, k), generator=generator, device=device, dtype=torch.bfloat16)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)

            def linear(index, ring=ring, out=out, x=x):
                blaslt.bind_current_stream()
                blaslt.linear_bf16(x, ring[index % len(ring)], out)

            bytes_moved = 2 * (n * k + m * k + m * n)
            line = {"shape": name, "dtype": "bf16", "m": m, "n": n, "k": k, "bytes": bytes_moved,
                    "weight_copies": copies}
            for path in ("umma", "cublaslt"):
                os.environ["LFM25_BF16_GEMM"] = path
                cold = time_launches(linear, arguments.iterations)
                line[f"{path}_us_cold"] = cold
                line[f"{path}_us_l2_warm"] = time_launches(lambda index: linear(0), arguments.iterations)
                line[f"{path}_hbm_frac_cold"] = bytes_moved / cold / 1e3 / hbm_peak
            os.environ.pop("LFM25_BF16_GEMM", None)
            print(json.dumps(line), flush=True)
        del ring
    blaslt.close()


TIMELINE_MARKS = ["entry", "setup_done", "dependency_released", "first_stage_full", "last_mma_committed",
                  "accumulator_ready", "epilogue_stored", "end"]


def timeline(arguments, ops, abi, device):
    """Per-launch breakdown of the tcgen05 GEMM from the instrumented build: a graph of 16 launches over the weight
    ring; the marks of the last two launches (SM cycle counter per CTA, anchored by the global timer at CTA entry) are
    printed as min / mean / max nanoseconds since the first CTA entry of the earlier launch."""
    import ctypes

    import numpy as np

    generator = torch.Generator(device=device).manual_seed(2)
    blaslt = ops.BlasLt()
    for name, n, k in SHAPES:
        if arguments.shapes and name not in arguments.shapes:
            continue
        copies = max(2, (RING_BYTES + n * k - 1) // (n * k))
        codes = (torch.randn((n, k), generator=generator, device=device) * 8).clamp(-448, 448).to(
            torch.float8_e4m3fn).view(torch.uint8)
        ring = [codes.clone() for _ in range(copies)]
        for m in arguments.ms:
            x = (torch.randn((m, k), generator=generator, device=device) * 8).to(torch.float8_e4m3fn).view(torch.uint8)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)

            def ours(index, ring=ring, out=out, x=x):
                blaslt.bind_current_stream()
                blaslt.linear_fp8_scaled(x, ring[index % len(ring)], out, 1.0)

            per_launch = time_launches(ours, 16, replays=1)
            marks = np.zeros((2, 512, 10), dtype=np.uint64)
            code = abi.library().lfm25_debug_umma_timeline(marks.ctypes.data_as(ctypes.POINTER(ctypes.c_ulonglong)))
            if code != 0:
                raise RuntimeError(f"timeline read failed with CUDA error {code}")
            launches = []
            for slot in range(2):
                used = marks[slot][:, 0] != 0
                if used.any():
                    t = marks[slot][used].astype(np.int64)
                    since_entry = (t[:, 0:8] - t[:, 0:1]) / arguments.sm_mhz * 1e3      # cycles -> ns
                    launches.append((int(t[:, 8].min()), t[:, 8:9] + since_entry, t[:, 9]))
            launches.sort(key=lambda item: item[0])
            line = {"shape": name, "m": m, "us_per_launch": per_launch, "launches": []}
            for first_entry, absolute, exits in launches:
                origin = launches[0][0]
                line["launches"].append({
                    "ctas": int(absolute.shape[0]),
                    **{mark: [float(absolute[:, index].min() - origin), float(absolute[:, index].mean() - origin),
                              float(absolute[:, index].max() - origin)] for index, mark in enumerate(TIMELINE_MARKS)},
                    "exit_global_timer": [int(exits.min() - origin), int(exits.max() - origin)]})
            print(json.dumps(line), flush=True)
        del ring


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--dtype", choices=["e4m3", "bf16"], default="e4m3")
    parser.add_argument("--iterations", type=int, default=64)
    parser.add_argument("--ms", type=int, nargs="+", default=[1, 8, 32, 128, 256])
    parser.add_argument("--no-cublaslt", action="store_true")
    parser.add_argument("--paths", nargs="+", default=["auto"],
                        help="kernel paths to time: auto, stream, umma (sets LFM25_FP8_GEMM_PATH)")
    parser.add_argument("--handle", action="store_true", help="call through a BlasLt handle (allows split-K)")
    parser.add_argument("--shapes", nargs="+", default=None, help="only these sites (gate_up, down, lm_head, ...)")
    parser.add_argument("--timeline", action="store_true",
                        help="per-launch breakdown from the instrumented build (python lfm25-inference_b200/build.py "
                             "--timeline makes liblfm25_b200_timeline.so)")
    parser.add_argument("--sm-mhz", type=float, default=1965.0, help="SM clock used to turn cycle marks into ns")
    arguments = parser.parse_args()
    entry.load_package()
    if arguments.timeline:
        from lfm25_inference_b200 import _abi
        _abi.LIBRARY_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "liblfm25_b200_timeline.so")
    from lfm25_inference_b200 import ops

    device = torch.device("cuda:0")
    peak_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm_peak = json.load(open(peak_path))["hbm_gbs"] if os.path.exists(peak_path) else 6650.0
    if arguments.timeline:
        from lfm25_inference_b200 import _abi
        timeline(arguments, ops, _abi, device)
        return
    if arguments.dtype == "bf16":
        sweep_bf16(arguments, ops, device, hbm_peak)
        return
    generator = torch.Generator(device=device).manual_seed(2)
    blaslt = ops.BlasLt() if arguments.handle else None
    for name, n, k in SHAPES:
        if arguments.shapes and name not in arguments.shapes:
            continue
        copies = max(2, (RING_BYTES + n * k - 1) // (n * k))
        weight = torch.randn((n, k), generator=generator, device=device) * 0.02
        w_amax = float(weight.abs().max())
        codes = (weight * (448.0 / w_amax)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
        ring = [codes.clone() for _ in range(copies)]
        del weight
        for m in arguments.ms:
            x = torch.randn((m, k), generator=generator, device=device, dtype=torch.bfloat16)
            x_amax = float(x.float().abs().max())
            x_codes = torch.empty((m, k), dtype=torch.uint8, device=device)
            ops.quantize_bf16_e4m3_into(x, x_codes, 448.0 / x_amax)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
            scale = (x_amax / 448.0) * (w_amax / 448.0)

            def ours(index, ring=ring, out=out, x_codes=x_codes):
                if blaslt is not None:
                    blaslt.linear_fp8_scaled(x_codes, ring[index % len(ring)], out, scale)
                else:
                    ops.linear_fp8_scaled_into(x_codes, ring[index % len(ring)], out, scale)

            def ours_with_quantise(index, x_codes=x_codes, x=x):
                ops.quantize_bf16_e4m3_into(x, x_codes, 448.0 / x_amax)
                ours(index)

            bytes_moved = n * k + m * k + 2 * m * n
            line = {"shape": name, "m": m, "n": n, "k": k, "bytes": bytes_moved, "flops": 2 * m * n * k,
                    "weight_copies": copies, "handle": arguments.handle}
            for path in arguments.paths:
                if path == "auto":
                    os.environ.pop("LFM25_FP8_GEMM_PATH", None)
                else:
                    os.environ["LFM25_FP8_GEMM_PATH"] = path
                if path == "stream" and m > 64:
                    continue
                cold = time_launches(ours, arguments.iterations)
                line[f"{path}_us_cold"] = cold
                line[f"{path}_us_l2_warm"] = time_launches(lambda index: ours(0), arguments.iterations)
                line[f"{path}_us_cold_with_quantise"] = time_launches(ours_with_quantise, arguments.iterations)
                line[f"{path}_gbs_cold"] = bytes_moved / cold / 1e3
                line[f"{path}_hbm_frac_cold"] = bytes_moved / cold / 1e3 / hbm_peak
                line[f"{path}_tflops_cold"] = 2 * m * n * k / cold / 1e6
            os.environ.pop("LFM25_FP8_GEMM_PATH", None)
            if not arguments.no_cublaslt:
                try:
                    one = torch.ones((), device=device)
                    a8 = x_codes.view(torch.float8_e4m3fn)
                    ring8 = [w.view(torch.float8_e4m3fn).t() for w in ring]

                    def cublaslt(index):
                        torch._scaled_mm(a8, ring8[index % len(ring8)], scale_a=one, scale_b=one,
                                         out_dtype=torch.bfloat16)

                    line["cublaslt_us_cold"] = time_launches(cublaslt, arguments.iterations)
                    line["cublaslt_us_l2_warm"] = time_launches(lambda index: cublaslt(0), arguments.iterations)
                    first = arguments.paths[0]
                    if f"{first}_us_cold" in line:
                        line["speedup_vs_cublaslt_cold"] = line["cublaslt_us_cold"] / line[f"{first}_us_cold"]
                except Exception as error:  # shape rules of torch._scaled_mm differ between releases
                    line["cublaslt_error"] = str(error)[:120]
            print(json.dumps(line), flush=True)
        del ring


if __name__ == "__main__":
    main()

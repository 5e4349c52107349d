"""Timing of the decode GEMM sites, HBM-cold, next to cuBLASLt on the same buffers (what ``bench.py --workload gemm``
and the ``gemm_roofline`` table of the default bench line are made of).

Sites (the reference's decode step, src/model/decode_executor.rs:227-418): the E4M3 ones -- packed Gate/Up
2048 -> 16384, Down 8192 -> 2048, LM head 2048 -> 65536 -- and the BF16 ones of the layers outside the FP8 policy.
Weights ~ N(0, 0.02) and activations ~ N(0, 1), quantised per tensor with scale amax / 448; all seeded synthetic.

Every number is GPU-side: the launches of one point are captured in a CUDA graph that walks a ring of distinct
weight copies of at least 512 MB (four times the L2), the graph is replayed and timed with CUDA events, so neither
the host's launch cadence nor a warm L2 enters.  The roofline of a point is max(bytes / HBM peak, flops / tensor
peak) with bytes = N K + M K + 2 M N (E4M3; twice the first two for BF16) and flops = 2 M N K.
"""
from __future__ import annotations

import torch

FP8_SITES = [("gate_up", 16384, 2048), ("down", 2048, 8192), ("lm_head", 65536, 2048)]
BF16_SITES = [("qkv", 3072, 2048), ("proj", 2048, 2048), ("conv_in", 6144, 2048), ("gate_up", 16384, 2048),
              ("down", 2048, 8192)]
BATCHES = [1, 8, 32, 128, 256]
RING_BYTES = 512 << 20


def time_launches(function, count: int, replays: int = 5) -> float:
    """Microseconds per launch: `count` calls of function(index) captured in one CUDA graph, replayed `replays` times."""
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
        stream.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(replays):
            graph.replay()
        stop.record()
        stream.synchronize()
    torch.cuda.current_stream().wait_stream(stream)
    return start.elapsed_time(stop) * 1e3 / (count * replays)


def measure_fp8_peak(device) -> float:
    """Dense E4M3 GEMM rate of cuBLASLt (8192^3 through torch._scaled_mm), TFLOP/s, best of 5: the tensor-pipe
    denominator of the roofline (MEASURED_PEAKS.json holds the BF16 rate only)."""
    size = 8192
    a = torch.randn((size, size), device=device).to(torch.float8_e4m3fn)
    b = torch.randn((size, size), device=device).to(torch.float8_e4m3fn).t()
    one = torch.ones((), device=device)
    best = 0.0
    for _ in range(6):
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        stop.record()
        torch.cuda.synchronize()
        best = max(best, 2.0 * size ** 3 / (start.elapsed_time(stop) * 1e-3) / 1e12)
    return best


def _roofline(bytes_moved: int, flops: int, hbm_gbs: float, tensor_tflops: float) -> dict:
    t_hbm = bytes_moved / hbm_gbs / 1e3            # microseconds
    t_tensor = flops / tensor_tflops / 1e6
    return {"bytes": bytes_moved, "flops": flops, "t_hbm_us": t_hbm, "t_tensor_us": t_tensor,
            "bound": "hbm" if t_hbm >= t_tensor else "tensor", "floor_us": max(t_hbm, t_tensor)}


def sweep_fp8(ops, device, hbm_gbs: float, fp8_tflops: float, batches=None, sites=None, iterations: int = 64,
              tunings=None, with_library: bool = True, with_gated: bool = True, with_quantise: bool = False):
    """Rows for the E4M3 sites.  `tunings`: {label: keyword arguments of BlasLt.set_gemm_tuning}; the default is the
    library's own choice under the label "ours"."""
    tunings = tunings or {"ours": {}}
    generator = torch.Generator(device=device).manual_seed(2)
    blaslt = ops.BlasLt()
    rows = []
    for name, n, k in FP8_SITES:
        if sites and name not in sites:
            continue
        copies = max(2, (RING_BYTES + n * k - 1) // (n * k))
        weight = torch.randn((n, k), generator=generator, device=device) * 0.02
        w_amax = float(weight.abs().max())
        codes = (weight * (448.0 / w_amax)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
        ring = [codes.clone() for _ in range(copies)]
        del weight
        for m in batches or BATCHES:
            x = torch.randn((m, k), generator=generator, device=device, dtype=torch.bfloat16)
            x_amax = float(x.float().abs().max())
            x_codes = torch.empty((m, k), dtype=torch.uint8, device=device)
            ops.quantize_bf16_e4m3_into(x, x_codes, 448.0 / x_amax)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
            scale = (x_amax / 448.0) * (w_amax / 448.0)
            row = {"site": name, "dtype": "e4m3", "m": m, "n": n, "k": k, "weight_copies": copies,
                   **_roofline(n * k + m * k + 2 * m * n, 2 * m * n * k, hbm_gbs, fp8_tflops)}

            def ours(index):
                blaslt.linear_fp8_scaled(x_codes, ring[index % copies], out, scale)

            def ours_with_quantise(index):
                ops.quantize_bf16_e4m3_into(x, x_codes, 448.0 / x_amax)
                ours(index)

            for label, tuning in tunings.items():
                blaslt.set_gemm_tuning(**tuning)
                row[f"{label}_us"] = time_launches(ours, iterations)
                if with_quantise:
                    row[f"{label}_us_with_quantise"] = time_launches(ours_with_quantise, iterations)
                    row[f"{label}_us_l2_warm"] = time_launches(lambda index: ours(0), iterations)
            if with_gated and name == "gate_up":
                codes_out = torch.empty((m, n // 2), dtype=torch.uint8, device=device)

                def gated(index):
                    blaslt.linear_fp8_silu_mul(x_codes, ring[index % copies], codes_out, scale, 448.0 / 16.0)

                for label, tuning in tunings.items():
                    blaslt.set_gemm_tuning(**tuning)
                    row[f"{label}_silu_mul_us"] = time_launches(gated, iterations)
            blaslt.set_gemm_tuning()
            if with_library:
                try:
                    one = torch.ones((), device=device)
                    a8 = x_codes.view(torch.float8_e4m3fn)
                    ring8 = [w.view(torch.float8_e4m3fn).t() for w in ring]

                    def library(index):
                        torch._scaled_mm(a8, ring8[index % copies], scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

                    row["cublaslt_us"] = time_launches(library, iterations)
                except Exception as error:       # shape rules of torch._scaled_mm differ between releases
                    row["cublaslt_error"] = str(error)[:120]
            rows.append(row)
        del ring
    blaslt.close()
    return rows


def sweep_bf16(ops, device, hbm_gbs: float, bf16_tflops: float, batches=None, sites=None, iterations: int = 64,
               tunings=None, with_library: bool = True, with_gated: bool = True):
    """Rows for the BF16 sites; "cublaslt" is the same handle with the library kernel forced."""
    from . import _abi
    tunings = tunings or {"ours": {}}
    generator = torch.Generator(device=device).manual_seed(3)
    blaslt = ops.BlasLt()
    rows = []
    for name, n, k in BF16_SITES:
        if sites and name not in sites:
            continue
        copies = max(2, (RING_BYTES + 2 * n * k - 1) // (2 * n * k))
        ring = [(torch.randn((n, k), generator=generator, device=device) * 0.02).to(torch.bfloat16)
                for _ in range(copies)]
        for m in batches or BATCHES:
            x = torch.randn((m, k), generator=generator, device=device, dtype=torch.bfloat16)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
            row = {"site": name, "dtype": "bf16", "m": m, "n": n, "k": k, "weight_copies": copies,
                   **_roofline(2 * (n * k + m * k + m * n), 2 * m * n * k, hbm_gbs, bf16_tflops)}

            def linear(index):
                blaslt.linear_bf16(x, ring[index % copies], out)

            for label, tuning in tunings.items():
                blaslt.set_gemm_tuning(**tuning)
                row[f"{label}_us"] = time_launches(linear, iterations)
            if with_gated and name == "gate_up":
                activation = torch.empty((m, n // 2), dtype=torch.bfloat16, device=device)

                def gated(index):
                    blaslt.linear_bf16_silu_mul(x, ring[index % copies], activation)

                for label, tuning in tunings.items():
                    blaslt.set_gemm_tuning(**tuning)
                    row[f"{label}_silu_mul_us"] = time_launches(gated, iterations)
            if with_library:
                blaslt.set_gemm_tuning(kernel=_abi.GEMM_KERNEL_LIBRARY)
                row["cublaslt_us"] = time_launches(linear, iterations)
            blaslt.set_gemm_tuning()
            rows.append(row)
        del ring
    blaslt.close()
    return rows


def compact(rows, label: str = "ours") -> list:
    """One short record per point for a bench line: site, M, ours and cuBLASLt microseconds, the roofline floor, which
    term binds and the fraction of the floor reached."""
    table = []
    for row in rows:
        ours = row.get(f"{label}_us")
        table.append({"site": row["site"], "dtype": row["dtype"], "m": row["m"],
                      "us": round(ours, 2) if ours else None,
                      "cublaslt_us": round(row["cublaslt_us"], 2) if "cublaslt_us" in row else None,
                      "floor_us": round(row["floor_us"], 2), "bound": row["bound"],
                      "frac": round(row["floor_us"] / ours, 3) if ours else None})
    return table

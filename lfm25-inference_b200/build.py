"""Build recipe of the CUDA library (stands in for the reference's build.rs, which compiles its
kernels with nvcc at build time).  Produces ``liblfm25_b200.so`` next to this file, for sm_100a only.

    python lfm25-inference_b200/build.py [--force] [--verbose] [--timeline]

``--timeline`` builds a second, instrumented copy (``liblfm25_b200_timeline.so``, ``-DLFM25_UMMA_TIMELINE``) whose
tcgen05 GEMM records the SM cycle counter along its critical path; ``bench_fp8_gemm.py --timeline`` reads it.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUTPUT = os.path.join(HERE, "liblfm25_b200.so")
OUTPUT_TIMELINE = os.path.join(HERE, "liblfm25_b200_timeline.so")
SOURCES = ["api.cu", "attention.cu", "kv_cache.cu", "fp8_elementwise.cu", "fp8_gemm_stream.cu", "fp8_gemm_umma.cu",
           "attention_static_scratch.cu", "hybrid_attention.cu", "hybrid_attention_umma.cu", "model_ops.cu", "cublaslt_bf16.cu", "decode_executor.cu", "host_runtime.cu", "prefix_cache.cu", "scheduler.cu", "serving_engine.cu"]
HEADERS = ["common.cuh", "kernels.h", "tensor_map.h", "tcgen05.cuh", "blaslt_handle.h", "launch.h", os.path.join("..", "..", "include", "lfm25_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math=false", "-Xcompiler", "-fPIC", "-shared", "-cudart", "static", "-ldl",
]


def _stale(output: str = OUTPUT) -> bool:
    if not os.path.exists(output):
        return True
    built = os.path.getmtime(output)
    inputs = [os.path.join(CSRC, name) for name in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(path) > built for path in inputs)


def build(force: bool = False, verbose: bool = False, timeline: bool = False) -> str:
    output = OUTPUT_TIMELINE if timeline else OUTPUT
    if not force and not _stale(output):
        return output
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = [flag for flag in NVCC_FLAGS if flag != "--use_fast_math=false"]
    if verbose:
        flags += ["-Xptxas", "-v"]
    if timeline:
        flags += ["-DLFM25_UMMA_TIMELINE"]
    command = [nvcc, *flags, "-o", output, *[os.path.join(CSRC, name) for name in SOURCES]]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed building {os.path.basename(output)}")
    return output


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, timeline="--timeline" in sys.argv))

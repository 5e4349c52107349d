"""Build recipe of the CUDA library (stands in for the reference's build.rs, which compiles its
kernels with nvcc at build time).  Produces ``liblfm25_b200.so`` next to this file, for sm_100a only.

    python lfm25-inference_b200/build.py [--force] [--verbose]

Every source is compiled to an object of its own (in parallel, only when it or a header changed) under
``build/`` and the objects are linked into the shared library.  ``--verbose`` adds ``-Xptxas -v``.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJECTS = os.path.join(HERE, "build")
OUTPUT = os.path.join(HERE, "liblfm25_b200.so")
SOURCES = ["api.cu", "options.cu", "attention.cu", "kv_cache.cu", "fp8_elementwise.cu", "fp8_gemm_stream.cu",
           "fp8_gemm_umma.cu", "gemm_rows_umma.cu", "attention_static_scratch.cu", "hybrid_attention.cu",
           "hybrid_attention_umma.cu", "model_ops.cu", "cublaslt_bf16.cu", "decode_executor.cu", "host_runtime.cu",
           "prefix_cache.cu", "scheduler.cu", "serving_engine.cu"]
COMPILE_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static", "-ldl"]


def _headers() -> list[str]:
    found = [os.path.join(CSRC, name) for name in os.listdir(CSRC) if name.endswith((".h", ".cuh"))]
    found.append(os.path.join(HERE, "..", "include", "lfm25_b200.h"))
    found.append(os.path.abspath(__file__))
    return found


def _newer_than(target: str, inputs: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    built = os.path.getmtime(target)
    return any(os.path.getmtime(path) > built for path in inputs)


def _compile(nvcc: str, source: str, obj: str, verbose: bool) -> tuple[int, str]:
    flags = COMPILE_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    result = subprocess.run([nvcc, *flags, "-c", source, "-o", obj], capture_output=True, text=True)
    return result.returncode, result.stdout + result.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(OBJECTS, exist_ok=True)
    headers = _headers()
    jobs = []
    objects = []
    for name in SOURCES:
        source = os.path.join(CSRC, name)
        obj = os.path.join(OBJECTS, name[:-3] + ".o")
        objects.append(obj)
        if force or _newer_than(obj, [source, *headers]):
            jobs.append((source, obj))
    failed = False
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for code, output in pool.map(lambda job: _compile(nvcc, job[0], job[1], verbose), jobs):
            if verbose or code != 0:
                sys.stderr.write(output)
            failed = failed or code != 0
    if failed:
        raise RuntimeError("nvcc failed compiling the library sources")
    if jobs or force or _newer_than(OUTPUT, objects):
        result = subprocess.run([nvcc, *LINK_FLAGS, "-o", OUTPUT, *objects], capture_output=True, text=True)
        if verbose or result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed linking {os.path.basename(OUTPUT)}")
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

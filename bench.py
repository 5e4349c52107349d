"""Benchmark of the decode hot path: ragged paged GQA decode attention + paged KV append.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--splits S]

Workload (one "step" = one decode step of the batch): 64 sequences with contexts seeded-uniform in
[16, 8192], page size 16, block tables drawn from a seeded shuffle of a 2^16-page bf16 K/V pool, 32 query /
8 KV heads of dim 64.  Each step appends one token per sequence (fused QK-norm + RoPE + paged append) and
then runs ragged paged attention over every sequence's whole context.  Steps run in episodes of 16: step s
uses positions context + (s mod 16), so the work per episode is fixed for any K.

One JSON line is printed by rank 0.  `value` is tokens/s with inputs resident in HBM; `e2e` is the same
metric through the C ABI with host buffers (pinned H2D of the step's Q/K/V and metadata, D2H of the output,
inside the timed region); `roofline` is the attention kernel's algorithmic KV bytes per launch over its
CUDA-event duration against the measured HBM copy bandwidth; `cpu_baseline` is the CPU oracle on a bounded
sample of the same step.  With --impl reference the CPU implementation itself is timed (the reference
project has no CPU path of its own, so that arm is the multithreaded oracle port).

Multi-GPU: the path does not shard (a sequence's KV lives on one GPU), so N ranks are N independent engine
replicas with different seeds; there is no collective on the data path, only the timing barrier.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

SEQUENCES = 64
CONTEXT_LOW, CONTEXT_HIGH = 16, 8192
NUM_PAGES = 1 << 16
EPISODE = 16
METRIC = "decode tok/s (ragged paged GQA decode attention + KV append, 64 sequences, contexts U[16,8192])"
WORKLOAD = "config1-ragged-paged-decode-attention+kv-append"


def parse_arguments():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=1024)
    parser.add_argument("--warmup", type=int, default=32)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--splits", type=int, default=0, help="KV-axis splits (0 = library policy)")
    parser.add_argument("--cpu-sequences", type=int, default=0, help="sequences in the CPU sample (0 = auto)")
    parser.add_argument("--sequences", type=int, default=SEQUENCES,
                        help="batch size; values other than 64 are for profiling a smaller case, not the metric")
    parser.add_argument("--pool-pages", type=int, default=NUM_PAGES, help="pages in the K/V pool (same remark)")
    parser.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline (profiling runs)")
    arguments = parser.parse_args()
    globals().update(SEQUENCES=arguments.sequences, NUM_PAGES=arguments.pool_pages)
    return arguments


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.process = None
        self.index = index

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.rows.append([field.strip() for field in line.split(",")])

    def __exit__(self, *_):
        if self.process is not None:
            self.process.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        clocks = [float(row[1]) for row in self.rows if len(row) >= 9 and row[1].replace(".", "").isdigit()]
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = set()
        for row in self.rows:
            if len(row) < 9:
                continue
            for name, field in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   row[5:9]):
                if field.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(clocks)), "sm_max_mhz": float(self.rows[0][2]),
                "reasons": sorted(reasons), "samples": len(clocks)}


# ------------------------------------------------------------------------------------ CPU arm


def cpu_sample(batch, seed, sequences, repeats):
    """Times the CPU oracle on `sequences` sequences of one decode step (append + attention).
    Returns (tokens per second, seconds per pass, description)."""
    from lfm25_inference_b200 import workloads
    from oracle import oracle
    rng = np.random.default_rng(seed)
    chosen = np.argsort(batch.contexts)[np.linspace(0, batch.num_sequences - 1, sequences).astype(int)]
    tables, positions, pages_total = [], [], 0
    for sequence in chosen:
        count = int((batch.contexts[sequence] + 1 + 15) // 16)
        tables.append(np.arange(pages_total, pages_total + count, dtype=np.uint32))
        positions.append(int(batch.contexts[sequence]))
        pages_total += count
    stride = max(len(table) for table in tables)
    block_tables = np.full((sequences, stride), 0xFFFFFFFF, dtype=np.uint32)
    for row, table in enumerate(tables):
        block_tables[row, :len(table)] = table
    key_cache = workloads.bf16_normal(rng, (pages_total, 8, 16, 64))
    value_cache = workloads.bf16_normal(rng, (pages_total, 8, 16, 64))
    query = workloads.bf16_normal(rng, (sequences, 32, 64))
    key = workloads.bf16_normal(rng, (sequences, 8, 64))
    value = workloads.bf16_normal(rng, (sequences, 8, 64))
    ones = oracle.f32_to_bf16(np.ones(64, dtype=np.float32))
    position_ids = np.array(positions, dtype=np.uint32)
    request_slots = np.arange(sequences, dtype=np.uint32)
    slots = oracle.physical_slots(block_tables, request_slots, position_ids)
    inv_freq = oracle.rope_inv_freq()

    def one_pass():
        rotated = query.copy()
        oracle.qk_norm_rope_kv_write_decode(rotated, key, value, ones, ones, inv_freq, position_ids, slots,
                                            key_cache, value_cache, 1e-5)
        oracle.paged_ragged_attention(rotated, key_cache, value_cache, block_tables, request_slots, position_ids)

    one_pass()
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - start)
    best = min(times)
    keys = int(sum(position + 1 for position in positions))
    description = (f"one decode step on {sequences} of the {batch.num_sequences} sequences "
                   f"(evenly spaced by context length, {keys} keys), best of {repeats}")
    return sequences / best, best, description, oracle.num_threads()


def run_reference_arm(arguments, rank):
    """The CPU implementation of the path, all host threads, bounded sample per step."""
    if rank != 0:
        return
    entry.load_package()
    from lfm25_inference_b200 import workloads
    batch = workloads.ragged_decode_batch(1, SEQUENCES, CONTEXT_LOW, CONTEXT_HIGH, NUM_PAGES, EPISODE)
    sequences = min(SEQUENCES, arguments.cpu_sequences or 16)
    steps = max(1, min(arguments.steps, 8))
    tokens_per_s, seconds, description, threads = cpu_sample(batch, 1, sequences, steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": tokens_per_s, "unit": "tok/s", "n_gpus": arguments.gpus,
        "steps": steps, "warmup": 1, "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sequences": SEQUENCES, "page_size": 16, "sample": description},
        "cpu_baseline": {"value": tokens_per_s, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": description},
        "e2e": {"value": tokens_per_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference project is GPU-only; this arm times the multithreaded C restatement of its kernels",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm


def run_gpu_arm(arguments, rank, world):
    import torch
    import torch.distributed as dist

    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    entry.load_package()
    from lfm25_inference_b200 import ops, workloads

    seed = 1 + rank
    batch = workloads.ragged_decode_batch(seed, SEQUENCES, CONTEXT_LOW, CONTEXT_HIGH, NUM_PAGES, EPISODE)
    generator = torch.Generator(device=device).manual_seed(seed)
    shape = (NUM_PAGES, 8, 16, 64)
    arena = ops.PagedKvArena(torch.randn(shape, generator=generator, device=device, dtype=torch.bfloat16),
                             torch.randn(shape, generator=generator, device=device, dtype=torch.bfloat16))
    block_tables = torch.from_numpy(batch.block_tables.view(np.int32).copy()).to(device)
    request_slots = torch.from_numpy(batch.request_slots.view(np.int32).copy()).to(device)
    ones = torch.ones(64, dtype=torch.bfloat16, device=device)
    inv_freq = torch.from_numpy(_inv_freq()).to(device)

    # per-step inputs of one episode, resident on the device and mirrored in pinned host memory
    def normal(shape_):
        return torch.randn(shape_, generator=generator, device=device, dtype=torch.bfloat16)

    episode = []
    for step in range(EPISODE):
        episode.append({
            "query": normal((SEQUENCES, 32, 64)), "key": normal((SEQUENCES, 8, 64)),
            "value": normal((SEQUENCES, 8, 64)),
            "positions": torch.from_numpy(batch.positions(step).view(np.int32).copy()).to(device),
            "slots": torch.from_numpy(batch.physical_slots(step)).to(device),
        })
    host_episode = [{name: tensor.cpu().pin_memory() for name, tensor in step.items()} for step in episode]
    staging = {name: torch.empty_like(tensor) for name, tensor in episode[0].items()}
    output = torch.empty((SEQUENCES, 32, 64), dtype=torch.bfloat16, device=device)
    host_output = torch.empty((SEQUENCES, 32, 64), dtype=torch.bfloat16).pin_memory()
    # the append rewrites the query in place, so the timed steps draw from a pool of fresh queries
    query_pool = normal((min(arguments.steps, 1024), SEQUENCES, 32, 64))
    partials = torch.empty((ops.splitk_workspace_elements(SEQUENCES),), dtype=torch.float32, device=device)
    max_context = int(batch.contexts.max()) + EPISODE
    splits = arguments.splits or ops.splitk_decode_splits(SEQUENCES, max_context, 16)

    def decode_step(inputs, query):
        """append: fused QK-norm + RoPE (query in place) + paged KV write; returns the attention inputs"""
        ops.qk_norm_rope_kv_write_arena_decode_bf16(query, inputs["key"], inputs["value"], ones, ones, inv_freq,
                                                    inputs["positions"], inputs["slots"], arena, 1e-5)
        return ops.FastRaggedAttentionInput(query, arena, block_tables, batch.stride, request_slots,
                                            inputs["positions"])

    def attend(attention_inputs):
        if splits > 1:
            ops.paged_ragged_attention_splitk_lfm2_bf16_into(attention_inputs, partials, splits, output)
        else:
            ops.paged_ragged_attention_fast_lfm2_bf16_into(attention_inputs, output)

    launches_per_step = 2 + (1 if splits > 1 else 0)   # append, attention, (merge)

    for step in range(arguments.warmup):
        attend(decode_step(episode[step % EPISODE], episode[step % EPISODE]["query"]))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()

    # ---- timed region: K steps, device-resident inputs ----
    steps = arguments.steps
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    end = torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        torch.cuda.synchronize()
        for step in range(steps):
            marks[step][0].record()
            attention_inputs = decode_step(episode[step % EPISODE], query_pool[step % query_pool.shape[0]])
            marks[step][1].record()
            attend(attention_inputs)
            marks[step][2].record()
        end.record()
        torch.cuda.synchronize()
        total_ms = marks[0][0].elapsed_time(end)
        # keep the clocks under observation for a moment longer on very short runs
        if total_ms < 500.0:
            spin_until = time.perf_counter() + 0.5
            while time.perf_counter() < spin_until:
                attend(decode_step(episode[0], episode[0]["query"]))
            torch.cuda.synchronize()
    clocks = sampler.summary()
    step_ms = np.array([marks[i][0].elapsed_time(marks[i + 1][0]) if i + 1 < steps
                        else marks[i][0].elapsed_time(end) for i in range(steps)])
    attention_ms = np.array([marks[i][1].elapsed_time(marks[i][2]) for i in range(steps)])
    append_ms = np.array([marks[i][0].elapsed_time(marks[i][1]) for i in range(steps)])
    if ops.device_status()[0] != 0:
        raise RuntimeError("a bounded wait ran out inside the timed region")

    # ---- end to end: host buffers in, host result out, every step ----
    h2d_bytes = sum(tensor.numel() * tensor.element_size() for tensor in host_episode[0].values())
    d2h_bytes = host_output.numel() * host_output.element_size()
    e2e_steps = min(steps, 256)
    for _ in range(3):
        for name, tensor in host_episode[0].items():
            staging[name].copy_(tensor, non_blocking=True)
        attend(decode_step(staging, staging["query"]))
        host_output.copy_(output, non_blocking=True)
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e2e_start = time.perf_counter()
    for step in range(e2e_steps):
        for name, tensor in host_episode[step % EPISODE].items():
            staging[name].copy_(tensor, non_blocking=True)
        attend(decode_step(staging, staging["query"]))
        host_output.copy_(output, non_blocking=True)
        torch.cuda.synchronize()          # the caller consumes the step's result before the next step
    e2e_seconds = time.perf_counter() - e2e_start

    elapsed = torch.tensor([total_ms, e2e_seconds * 1e3], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = (float(value) for value in elapsed.cpu())

    if rank == 0:
        hbm_peak, peak_kind = peaks()
        kv_bytes = float(np.mean([batch.kv_bytes(step % EPISODE) for step in range(steps)]))
        other_bytes = SEQUENCES * (4096 + 4096) + 4 * float(np.mean(
            [((batch.contexts + (step % EPISODE) + 16) // 16).sum() for step in range(steps)]))
        attention_seconds = float(attention_ms.mean()) * 1e-3
        achieved = (kv_bytes + other_bytes) / attention_seconds / 1e9
        if arguments.skip_cpu:
            cpu_tokens, cpu_description, threads = None, "skipped", 0
        else:
            cpu_tokens, _, cpu_description, threads = cpu_sample(
                batch, seed, min(SEQUENCES, arguments.cpu_sequences or 16), 3)
        line = {
            "metric": METRIC, "value": SEQUENCES * steps * world / (total_ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": steps, "warmup": arguments.warmup, "ms_per_step": total_ms / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sequences": SEQUENCES, "contexts": [CONTEXT_LOW, CONTEXT_HIGH],
                       "page_size": 16, "pool_pages": NUM_PAGES, "episode_steps": EPISODE, "kv_splits": splits,
                       "append": "fused QK-norm + RoPE + paged write", "replicas": world,
                       "l2": "inputs exceed L2 (about 0.5 GB of KV read per step)"},
            "tpot_p50_ms": float(np.median(step_ms)),
            "kv_gbs": kv_bytes / attention_seconds / 1e9,
            "append_us": float(append_ms.mean()) * 1e3, "attention_us": float(attention_ms.mean()) * 1e3,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "traffic": None, "peak_source": peak_kind,
                         "kernel": "ragged_decode_attention_kernel" + (" + merge_splitk_kernel" if splits > 1 else ""),
                         "algorithmic_bytes_per_launch": kv_bytes + other_bytes},
            "cpu_baseline": {"value": cpu_tokens, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": cpu_description},
            "e2e": {"value": SEQUENCES * e2e_steps * world / (e2e_ms * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps},
            "gpu_launches": launches_per_step * steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _inv_freq():
    index = np.arange(32, dtype=np.float32)
    return np.power(np.float32(1.0e6), -(np.float32(2.0) * index) / np.float32(64.0)).astype(np.float32)


def main():
    arguments = parse_arguments()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if arguments.impl == "reference":
        run_reference_arm(arguments, rank)
        return
    run_gpu_arm(arguments, rank, world)


if __name__ == "__main__":
    main()

"""Benchmark of the decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload step|attention|gemm|prefill|serving]

Default workload `step` (one "step" = one decode step of the whole model): the LFM2.5-1.2B architecture with
random-init weights under continuous batching -- 16 layers (6 GQA attention, 10 gated short-conv), hidden 2048,
vocabulary 65536, SwiGLU 8192, the 16 promoted FP8 sites -- on a batch of 128 sequences with contexts
seeded-uniform in [128, 4096], page size 16, greedy sampling.  The step is the C++ decode executor replayed from a
CUDA graph; token ids and positions advance on the device, so the timed region has no host work besides the graph
launches.  `value` is tokens/s (inputs resident in HBM), `tpot_p50_ms` the median step time, `roofline` the
attention kernel (the dominant kernel: KV bytes per launch over its CUDA-event duration in an instrumented eager
pass, against the measured HBM copy bandwidth).  `e2e` drives the same graph the way a serving loop does: every
step the host uploads the step metadata from pinned memory, launches, downloads the sampled ids and synchronises.

Workload `attention` (one "step" = append + attention of one layer) is the ragged paged attention configuration:
64 sequences, contexts seeded-uniform in [16, 8192], a 2^16-page pool, fused QK-norm + RoPE + paged append followed
by ragged paged attention, in episodes of 16 positions.  Its KV GB/s is also reported inside the default line.

Workload `gemm` is the decode GEMM sweep: the three E4M3 sites (packed Gate/Up 2048 -> 16384, Down 8192 -> 2048,
LM head 2048 -> 65536) and the BF16 sites of the step at M in {1, 8, 32, 128, 256}, HBM-cold over a ring of weight
copies of at least 512 MB, cuBLASLt on the same buffers beside every point, each against
max(bytes / HBM peak, flops / tensor peak).  A compact table of its E4M3 half is part of the default line
(`gemm_roofline`).

`cpu_baseline` / `--impl reference`: the reference project is GPU-only, so the CPU arm is the multithreaded C
restatement of its kernels (oracle/), timed on the same step (all 128 sequences, one step) on the host's cores.

Multi-GPU: the path does not shard (the model and every sequence's KV fit one GPU), so N ranks are N independent
engine replicas with different seeds; there is no collective on the data path, only the timing barrier.
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
STEP_METRIC = "decode tok/s (full LFM2.5-1.2B-architecture decode step, continuous batching, 128 sequences)"
STEP_WORKLOAD = "config3-full-decode-step-b128-ctx128-4096-fp8-policy"
STEP_SEQUENCES = 128
STEP_CONTEXT = (128, 4096)
STEP_POOL_PAGES = 32768


def parse_arguments():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--workload", default="step", choices=["step", "attention", "gemm", "prefill", "serving"])
    parser.add_argument("--steps", type=int, default=0, help="timed steps (default 256 for step, 1024 for attention)")
    parser.add_argument("--warmup", type=int, default=0, help="warm-up steps (default 8 / 32)")
    parser.add_argument("--no-fp8", action="store_true", help="step workload: run every site in BF16")
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--splits", type=int, default=0, help="KV-axis splits (0 = library policy)")
    parser.add_argument("--cpu-sequences", type=int, default=0, help="sequences in the CPU sample (0 = auto)")
    parser.add_argument("--sequences", type=int, default=SEQUENCES,
                        help="batch size; values other than 64 are for profiling a smaller case, not the metric")
    parser.add_argument("--step-sequences", type=int, default=STEP_SEQUENCES,
                        help="step workload: sequences in the batch (the headline number needs the default)")
    parser.add_argument("--pool-pages", type=int, default=NUM_PAGES, help="pages in the K/V pool (same remark)")
    parser.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline (profiling runs)")
    parser.add_argument("--skip-gemm", action="store_true", help="step workload: omit the gemm_roofline table")
    parser.add_argument("--gemm-dtype", default="all", choices=["all", "e4m3", "bf16"], help="gemm workload: which sites")
    parser.add_argument("--timeline", action="store_true",
                        help="step workload: add `graph_timeline` to the line -- per kernel of the replayed step its "
                             "launches, duration and the time during which no earlier kernel was still running, from "
                             "CUPTI activity records (torch.profiler) of a few extra replays after the timed region")
    parser.add_argument("--gemm-sites", nargs="*", default=None,
                        help="gemm workload: only these sites (gate_up down lm_head qkv proj conv_in); a profiling aid")
    parser.add_argument("--gemm-batches", nargs="*", type=int, default=None, help="gemm workload: only these M")
    parser.add_argument("--no-cublaslt", action="store_true", help="gemm workload: leave the cuBLASLt columns out")
    parser.add_argument("--dispatch", action="store_true",
                        help="serving workload: ONE trace for all replicas, handed out request by request by a front "
                             "(a thread of rank 0) through the library's dispatcher; --requests and --rate are then "
                             "per replica and are multiplied by the number of replicas")
    parser.add_argument("--requests", type=int, default=192, help="serving workload: requests in the trace")
    parser.add_argument("--rate", type=float, default=32.0, help="serving workload: Poisson arrival rate, requests/s")
    parser.add_argument("--skip-reference-kernels", action="store_true",
                        help="leave out the comparison runs of the reference project's own kernels")
    parser.add_argument("--admission-control", action="store_true",
                        help="serving workload: reject requests whose predicted TTFT / TPOT break the SLOs (the "
                             "reference's admission) instead of queueing them")
    arguments = parser.parse_args()
    if arguments.steps <= 0:
        arguments.steps = {"step": 256, "attention": 1024, "prefill": 16, "serving": 1, "gemm": 64}[arguments.workload]
    if arguments.warmup <= 0:
        arguments.warmup = {"step": 8, "attention": 32, "prefill": 3, "serving": 3, "gemm": 3}[arguments.workload]
    globals().update(SEQUENCES=arguments.sequences, NUM_PAGES=arguments.pool_pages,
                     STEP_SEQUENCES=arguments.step_sequences)
    return arguments


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peaks():
    """(BF16 TFLOP/s, source): the measured cuBLAS rate for a kernel timed alone."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return float(json.load(handle)["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


# DRAM bytes over algorithmic bytes of the decode attention kernel, from an ncu capture of a 16-sequence launch
# (dram__bytes_read.sum 139.26 MB against 139.09 MB algorithmic; the traffic is the KV stream, which grows in
# proportion to the keys read).
ATTENTION_TRAFFIC_FACTOR = 1.001


def gather_over_ranks(values, device, world):
    """Every rank's values, [world][len(values)] (the replicas are independent: no reduction is meaningful but max)."""
    import torch
    import torch.distributed as dist
    tensor = torch.tensor(list(values), dtype=torch.float64, device=device)
    if world == 1:
        return [[float(value) for value in tensor.cpu()]]
    gathered = [torch.zeros_like(tensor) for _ in range(world)]
    dist.all_gather(gathered, tensor)
    return [[float(value) for value in part.cpu()] for part in gathered]


def max_over_ranks(values, device, world):
    """Element-wise maximum of per-rank timings (replicas are independent, so the slowest one defines the job)."""
    import torch
    import torch.distributed as dist
    tensor = torch.tensor(list(values), dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
    return [float(value) for value in tensor.cpu()]


def aggregate_throughput(units_per_rank, world, elapsed_ms):
    """Whole-job throughput of `world` replicas that each processed `units_per_rank` units in `elapsed_ms`."""
    return units_per_rank * world / (elapsed_ms * 1e-3)


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
    oracle.use_all_cores()
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


def config0_latency(device):
    """BASELINE config 0: one sequence, context 40 after the append (39 cached + 1 new), 3 pages of a 64-page pool.
    80 KB of KV: latency-bound, so what is reported is microseconds per decode step of one attention layer, GPU-side,
    from a CUDA graph of 64 repetitions: raw append + attention (two launches), the one-kernel decode, and -- when
    the reference's kernels were built -- its one-kernel decode (the path config 0 takes there) and its append +
    attention pair."""
    import torch
    from lfm25_inference_b200 import ops, workloads
    c0 = workloads.single_step_c0(0)

    def bf16(bits):
        return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16).to(device)

    def u32(values):
        return torch.from_numpy(np.ascontiguousarray(values, dtype=np.uint32).view(np.int32).copy()).to(device)

    arena = ops.PagedKvArena(torch.zeros((64, 8, 16, 64), dtype=torch.bfloat16, device=device),
                             torch.zeros((64, 8, 16, 64), dtype=torch.bfloat16, device=device))
    arena.write_lfm2(bf16(c0["cached_key"]), bf16(c0["cached_value"]), torch.from_numpy(c0["cached_slots"]).to(device))
    query, key, value = bf16(c0["query"]), bf16(c0["new_key"]), bf16(c0["new_value"])
    slot, position = torch.from_numpy(c0["new_slot"]).to(device), u32(c0["position"])
    table, request_slot = u32(c0["block_table"]), u32(c0["request_slot"])
    ones, inv_freq = torch.ones(64, dtype=torch.bfloat16, device=device), torch.from_numpy(_inv_freq()).to(device)
    output = torch.zeros_like(query)
    inputs = ops.FastRaggedAttentionInput(query, arena, table, 3, request_slot, position)

    def two_launches():
        arena.write_lfm2(key, value, slot)
        ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, output)

    def one_kernel():
        ops.fused_ragged_paged_attention_decode_lfm2_bf16_into(query, key, value, ones, ones, inv_freq, position, slot,
                                                               arena, table, 3, request_slot, 1e-5, output)

    calls = {"append_plus_attention_us": two_launches, "one_kernel_decode_us": one_kernel}
    try:
        from oracle import refkernels
        if refkernels.available():
            scratch = query.clone()
            calls["reference_append_plus_attention_us"] = lambda: (
                refkernels.kv_cache_write(key, value, arena.key, arena.value, slot),
                refkernels.paged_ragged_attention_fast(query, arena.key, arena.value, table, request_slot, position,
                                                       output))
            calls["reference_qk_append_plus_attention_us"] = lambda: (
                refkernels.qk_norm_rope_kv_write_decode(scratch, key, value, ones, ones, inv_freq, position, slot,
                                                        arena.key, arena.value, 1e-5),
                refkernels.paged_ragged_attention_fast(scratch, arena.key, arena.value, table, request_slot, position,
                                                       output))
    except Exception:                      # the comparison is optional
        pass
    result = {}
    stream = torch.cuda.Stream(device=device)
    for name, call in calls.items():
        with torch.cuda.stream(stream):
            for _ in range(3):
                call()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(64):
                    call()
            graph.replay()
            stream.synchronize()
            begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for _ in range(5):
                graph.replay()
            finish.record()
            stream.synchronize()
            result[name] = begin.elapsed_time(finish) * 1e3 / (5 * 64)
    return result


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

    token_order = torch.zeros(SEQUENCES, dtype=torch.int32, device=device)

    def attend(attention_inputs):
        # the CTAs start on the longest contexts (ordered on the device, every step)
        ops.context_order_desc_into(attention_inputs.position_ids, token_order)
        if splits > 1:
            ops.paged_ragged_attention_splitk_lfm2_bf16_into(attention_inputs, partials, splits, output,
                                                             token_order=token_order)
        else:
            ops.paged_ragged_attention_fast_lfm2_bf16_into(attention_inputs, output, token_order=token_order)

    launches_per_step = 3 + (1 if splits > 1 else 0)   # append, context order, attention, (merge)

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

    # ---- the reference project's own kernels (rebuilt for sm_100a) on the same buffers, for comparison ----
    reference_kernels = None
    if rank == 0:
        try:
            from oracle import refkernels
            if refkernels.available():
                inputs = episode[0]
                query = inputs["query"].clone()
                timings = {}
                for name, call in (
                    ("append_us", lambda: refkernels.qk_norm_rope_kv_write_decode(
                        query, inputs["key"], inputs["value"], ones, ones, inv_freq, inputs["positions"],
                        inputs["slots"], arena.key, arena.value, 1e-5)),
                    ("attention_unsplit_us", lambda: refkernels.paged_ragged_attention_fast(
                        query, arena.key, arena.value, block_tables, request_slots, inputs["positions"], output)),
                    ("attention_splitk8_us", lambda: refkernels.paged_ragged_attention_splitk(
                        query, arena.key, arena.value, block_tables, request_slots, inputs["positions"],
                        partials, output, 8)),
                ):
                    call()
                    torch.cuda.synchronize()
                    begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    begin.record()
                    for _ in range(5):
                        call()
                    finish.record()
                    torch.cuda.synchronize()
                    timings[name] = begin.elapsed_time(finish) / 5 * 1e3
                reference_kernels = timings
        except Exception as error:           # the comparison is optional; the metric does not depend on it
            reference_kernels = {"error": str(error)[:120]}

    total_ms, e2e_ms = max_over_ranks([total_ms, e2e_seconds * 1e3], device, world)
    config0 = None
    if rank == 0:
        try:
            config0 = config0_latency(device)
        except Exception as error:           # an extra; the metric does not depend on it
            config0 = {"error": str(error)[:160]}

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
                         "frac": achieved / hbm_peak,
                         "traffic": ATTENTION_TRAFFIC_FACTOR * (kv_bytes + other_bytes),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 16-sequence launch = "
                                           "1.001 x its algorithmic bytes, scaled by the keys read "
                                           "(profiles/ragged_decode_attention_config1.md)",
                         "peak_source": peak_kind,
                         "kernel": "ragged_decode_attention_kernel" + (" + merge_splitk_kernel" if splits > 1 else ""),
                         "algorithmic_bytes_per_launch": kv_bytes + other_bytes},
            "cpu_baseline": {"value": cpu_tokens, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": cpu_description},
            "e2e": {"value": SEQUENCES * e2e_steps * world / (e2e_ms * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps},
            "gpu_launches": launches_per_step * steps,
            "reference_kernels_same_gpu": reference_kernels,
            "config0_single_step_latency": config0,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------ full decode step


def step_cpu_sample(model, batch, token_ids, use_fp8, sequences, repeats):
    """CPU oracle on `sequences` of the batch's sequences for one full decode step.  Returns (tok/s, s, text, threads)."""
    from oracle import step_oracle
    from oracle import oracle
    oracle.use_all_cores()
    host = step_oracle.HostModel(model)
    chosen = np.argsort(batch.contexts)[np.linspace(0, batch.num_sequences - 1, sequences).astype(int)]
    positions = batch.positions(0)[chosen]
    tables = batch.block_tables[chosen]
    slots = np.arange(sequences, dtype=np.uint32)
    for layer in host.layers:                      # conv states of the chosen sequences only
        if "conv_state" in layer:
            layer["conv_state"] = np.ascontiguousarray(layer["conv_state"][chosen])
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        step_oracle.decode_step(host, token_ids[chosen], positions, slots, tables, use_fp8)
        times.append(time.perf_counter() - start)
    best = min(times)
    keys = int((positions.astype(np.int64) + 1).sum())
    text = (f"one full decode step (16 layers, LM head, argmax) on {sequences} of the {batch.num_sequences} "
            f"sequences (evenly spaced by context length, {keys} keys per attention layer), best of {repeats}")
    return sequences / best, best, text, oracle.num_threads()


def build_step_state(arguments, seed, device, capacity_steps):
    import torch
    from lfm25_inference_b200 import model as lfm_model
    from lfm25_inference_b200 import workloads
    batch = workloads.ragged_decode_batch(seed, STEP_SEQUENCES, STEP_CONTEXT[0], STEP_CONTEXT[1], STEP_POOL_PAGES,
                                          capacity_steps)
    model = lfm_model.RandomModel(seed, device, STEP_POOL_PAGES, STEP_SEQUENCES)
    model.fill_caches(seed + 1)
    token_ids = np.random.default_rng(seed).integers(0, lfm_model.VOCAB, size=STEP_SEQUENCES).astype(np.uint32)
    return batch, model, token_ids


def run_step_reference_arm(arguments, rank):
    if rank != 0:
        return
    import torch
    entry.load_package()
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    batch, model, token_ids = build_step_state(arguments, 3, device, 8)
    sequences = arguments.cpu_sequences or STEP_SEQUENCES
    steps = 1
    tokens_per_s, seconds, description, threads = step_cpu_sample(model, batch, token_ids, not arguments.no_fp8,
                                                                  sequences, steps)
    line = {
        "impl": "reference", "metric": STEP_METRIC, "value": tokens_per_s, "unit": "tok/s", "n_gpus": arguments.gpus,
        "steps": steps, "warmup": 0, "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": STEP_WORKLOAD, "sequences": STEP_SEQUENCES, "page_size": 16, "sample": description},
        "cpu_baseline": {"value": tokens_per_s, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": description},
        "e2e": {"value": tokens_per_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference project is GPU-only; this arm times the multithreaded C restatement of its kernels",
    }
    print(json.dumps(line), flush=True)


def run_step_arm(arguments, rank, world):
    import torch
    import torch.distributed as dist

    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    entry.load_package()
    from lfm25_inference_b200 import model as lfm_model
    from lfm25_inference_b200 import ops

    use_fp8 = not arguments.no_fp8
    steps, warmup = arguments.steps, arguments.warmup
    e2e_steps = min(steps, 128)
    profile_steps = 8
    spin_steps = 320                                # extra steps that keep the GPU busy while clocks are sampled
    capacity = warmup + steps + e2e_steps + profile_steps + spin_steps + 16
    seed = 3 + rank
    batch, model, token_ids = build_step_state(arguments, seed, device, capacity)

    stream = torch.cuda.Stream(device=device)      # graph capture needs a non-default stream
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        blaslt = ops.BlasLt()
        executor = lfm_model.DecodeExecutor(blaslt, STEP_SEQUENCES)
        device_batch = lfm_model.DecodeBatch(device, batch.block_tables, batch.request_slots, batch.positions(0),
                                             token_ids, STEP_CONTEXT[1] + capacity)
        executor.forward(model, device_batch, use_fp8=use_fp8, advance=False)
        for _ in range(max(warmup, 3)):
            executor.step_graph(model, device_batch, use_fp8=use_fp8, advance=True)
        stream.synchronize()
        if world > 1:
            dist.barrier()

        # ---- timed region: K graph-replayed steps, ids and positions advance on the device ----
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        with ClockSampler(local_rank) as sampler:
            stream.synchronize()
            marks[0].record()
            submit_seconds = 0.0
            for step in range(steps):
                submit_start = time.perf_counter()
                executor.step_graph(model, device_batch, use_fp8=use_fp8, advance=True)
                submit_seconds += time.perf_counter() - submit_start
                marks[step + 1].record()
            stream.synchronize()
            total_ms = marks[0].elapsed_time(marks[steps])
            if total_ms < 500.0:                   # keep the clocks under observation a little longer
                until = time.perf_counter() + 0.5
                for _ in range(spin_steps):
                    if time.perf_counter() >= until:
                        break
                    executor.step_graph(model, device_batch, use_fp8=use_fp8, advance=True)
                    stream.synchronize()
        clocks = sampler.summary()
        step_ms = np.array([marks[i].elapsed_time(marks[i + 1]) for i in range(steps)])
        positions_now = device_batch.positions.cpu().numpy().view(np.uint32).astype(np.int64)

        # ---- instrumented eager pass: CUDA events around every op, for the per-kernel roofline ----
        executor.profile(True)
        library_calls_before = ops.library_calls()
        for _ in range(profile_steps):
            executor.forward(model, device_batch, use_fp8=use_fp8, advance=True)
        library_launches = (ops.library_calls() - library_calls_before) // profile_steps    # cuBLASLt matmuls per step
        regions = executor.profile(False, collect=True)
        contexts_profiled = positions_now + 1 + (profile_steps + 1) / 2.0      # mean context during the pass
        attention_ms, attention_ops = regions["attention"]
        attention_seconds = attention_ms / max(attention_ops, 1) * 1e-3
        kv_bytes = float((contexts_profiled * 2048).sum())
        other_bytes = STEP_SEQUENCES * 8192 + 4 * float(np.ceil(contexts_profiled / 16).sum())
        achieved_eager = (kv_bytes + other_bytes) / attention_seconds / 1e9

        # ---- the attention launches of one step, replayed from a graph of their own: the kernel's launch duration
        # without the host-side launch gaps that the events of an eager pass include.  One launch per attention
        # layer on that layer's own cache (6 x 0.55 GB: HBM-cold), the route, split count and token order the
        # executor uses for this batch, CUDA events around the replays. ----
        attention_layers = [layer for layer in model.layers if layer.is_attention]
        raw = {name: torch.randn((STEP_SEQUENCES, heads, 64), device=device, dtype=torch.bfloat16)
               for name, heads in (("query", 32), ("key", 8), ("value", 8))}
        attended = torch.empty((STEP_SEQUENCES, 32, 64), device=device, dtype=torch.bfloat16)
        order = torch.empty(STEP_SEQUENCES, dtype=torch.int32, device=device)
        ops.context_order_desc_into(device_batch.positions, order)
        longest = int(positions_now.max()) + profile_steps + 2
        graph_splits = ops.splitk_decode_splits(STEP_SEQUENCES, longest, 16)
        one_kernel = ops.decode_one_kernel_preferred(16, longest, STEP_SEQUENCES) \
            if ops.get_option("fused_append") == 2 else ops.get_option("fused_append") == 1
        partials = torch.empty(ops.splitk_workspace_elements(STEP_SEQUENCES), dtype=torch.float32, device=device)
        stride = device_batch.block_tables.shape[1]

        def attention_launches():
            for layer in attention_layers:
                arena = ops.PagedKvArena(layer.tensors["key_cache"], layer.tensors["value_cache"])
                if one_kernel:
                    ops.fused_ragged_paged_attention_decode_lfm2_bf16_into(
                        raw["query"], raw["key"], raw["value"], layer.tensors["query_norm"], layer.tensors["key_norm"],
                        model.inv_freq, device_batch.positions, device_batch.physical_slots, arena,
                        device_batch.block_tables, stride, device_batch.request_slots, lfm_model.NORM_EPS, attended,
                        partials if graph_splits > 1 else None, graph_splits, token_order=order)
                else:
                    ops.qk_norm_rope_kv_write_arena_decode_bf16(
                        raw["query"], raw["key"], raw["value"], layer.tensors["query_norm"], layer.tensors["key_norm"],
                        model.inv_freq, device_batch.positions, device_batch.physical_slots, arena, lfm_model.NORM_EPS)
                    inputs = ops.FastRaggedAttentionInput(raw["query"], arena, device_batch.block_tables, stride,
                                                          device_batch.request_slots, device_batch.positions)
                    if graph_splits > 1:
                        ops.paged_ragged_attention_splitk_lfm2_bf16_into(inputs, partials, graph_splits, attended,
                                                                         token_order=order)
                    else:
                        ops.paged_ragged_attention_fast_lfm2_bf16_into(inputs, attended, token_order=order)

        attention_launches()
        stream.synchronize()
        attention_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(attention_graph, stream=stream):
            attention_launches()
        for _ in range(3):
            attention_graph.replay()
        stream.synchronize()
        replays = 8
        begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(replays):
            attention_graph.replay()
        finish.record()
        stream.synchronize()
        attention_graph_seconds = begin.elapsed_time(finish) * 1e-3 / (replays * len(attention_layers))
        contexts_graph = positions_now + 1 + profile_steps                   # positions after the eager pass
        kv_bytes_graph = float((contexts_graph * 2048).sum())
        other_bytes_graph = STEP_SEQUENCES * 8192 + 4 * float(np.ceil(contexts_graph / 16).sum())
        achieved = (kv_bytes_graph + other_bytes_graph) / attention_graph_seconds / 1e9
        if ops.device_status()[0] != 0:
            raise RuntimeError("a bounded wait ran out inside the benchmark")

        # ---- the reference project's own attention kernels (rebuilt for sm_100a) on the same cache and metadata ----
        reference_kernels = None
        if rank == 0 and not arguments.skip_reference_kernels:
            try:
                from oracle import refkernels
                if refkernels.available():
                    layer = next(layer for layer in model.layers if layer.is_attention)
                    query = torch.randn((STEP_SEQUENCES, 32, 64), device=device, dtype=torch.bfloat16)
                    output = torch.empty_like(query)
                    arguments_ = (query, layer.tensors["key_cache"], layer.tensors["value_cache"],
                                  device_batch.block_tables, device_batch.request_slots, device_batch.positions, output)
                    def time_reference(function, launches=20):
                        for _ in range(3):
                            function()
                        stream.synchronize()
                        begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        begin.record()
                        for _ in range(launches):
                            function()
                        finish.record()
                        stream.synchronize()
                        return begin.elapsed_time(finish) / launches * 1e3

                    # the reference's unsplit kernel and its split-K kernel + merge (attention_async_fast.cu:211-419)
                    # under every split count its policy may pick; its better time is what this library is set against
                    unsplit_us = time_reference(lambda: refkernels.paged_ragged_attention_fast(*arguments_))
                    split_us = {}
                    for count in (2, 4, 8):
                        partials = torch.empty((STEP_SEQUENCES, 32, count, 66), dtype=torch.float32, device=device)
                        split_us[count] = time_reference(
                            lambda: refkernels.paged_ragged_attention_splitk(*arguments_[:-1], partials, output, count))
                    best_split = min(split_us, key=split_us.get)
                    reference_kernels = {"attention_unsplit_us_per_layer": unsplit_us,
                                         "attention_splitk_us_per_layer": {str(k): v for k, v in split_us.items()},
                                         "attention_best_us_per_layer": min(unsplit_us, split_us[best_split]),
                                         "attention_note": "20 launches each after 3 warm-up launches, same cache and metadata",
                                         "ours_us_per_layer": attention_seconds * 1e6}
            except Exception as error:       # optional comparison; the metric does not depend on it
                reference_kernels = {"error": str(error)[:120]}

        graph_timeline = None
        if rank == 0 and arguments.timeline:
            graph_timeline = step_timeline(executor, model, device_batch, stream, use_fp8)

        # ---- end to end: host metadata in, sampled ids out, every step ----
        host_block = device_batch.step_metadata.cpu().pin_memory()       # token ids | positions | request slots
        host_meta = {"token_ids": host_block[:STEP_SEQUENCES],
                     "positions": host_block[STEP_SEQUENCES:2 * STEP_SEQUENCES]}
        host_sampled = torch.empty(STEP_SEQUENCES, dtype=torch.int32).pin_memory()
        h2d_bytes = host_block.numel() * host_block.element_size()
        d2h_bytes = host_sampled.numel() * host_sampled.element_size()
        # the same contexts as the timed region: the host owns the positions here, so the served steps start where the
        # timed steps started (the clock-sampling and profiling steps in between moved the device's positions on by
        # several hundred tokens, which would make every served step read that much more KV than a timed one)
        host_meta["positions"].copy_(torch.from_numpy(
            (batch.positions(0).astype(np.int64) + max(warmup, 3) - 2).astype(np.int32)))   # 3 untimed served steps follow

        # the host's bookkeeping between steps on numpy views of the pinned buffers (a few hundred bytes)
        host_ids, host_positions = host_meta["token_ids"].numpy(), host_meta["positions"].numpy()
        sampled_view = host_sampled.numpy()

        def served_step():
            # upload of the metadata block, replay of the captured step, download of the ids and the synchronisation
            # the serving loop needs (EOS, streaming) before it goes on: one call into the library
            executor.serve_step(model, device_batch, host_block, host_sampled, use_fp8=use_fp8)
            host_ids[:] = sampled_view
            np.add(host_positions, 1, out=host_positions)

        for _ in range(3):
            served_step()
        if world > 1:
            dist.barrier()
        e2e_start = time.perf_counter()
        for _ in range(e2e_steps):
            served_step()
        e2e_seconds = time.perf_counter() - e2e_start
        if ops.device_status()[0] != 0:
            raise RuntimeError("a bounded wait ran out inside the benchmark")

        # ---- the whole step assembled from the reference's kernels and cuBLASLt, replayed from a CUDA graph ----
        if rank == 0 and reference_kernels is not None and "error" not in reference_kernels:
            try:
                reference_kernels.update(reference_kernel_step(model, device_batch, stream, use_fp8))
                reference_kernels["ours_step_ms"] = float(np.median(step_ms))
            except Exception as error:
                reference_kernels["step_error"] = str(error)[:160]

    # the E4M3 half of the decode GEMM sweep, as a compact table in the line (rank 0 only; after the timed regions)
    gemm_table = None
    if rank == 0 and not arguments.skip_gemm:
        try:
            from lfm25_inference_b200 import gemm_sweep
            fp8_peak = gemm_sweep.measure_fp8_peak(device)
            with torch.cuda.stream(stream):
                rows = gemm_sweep.sweep_fp8(ops, device, peaks()[0], fp8_peak, iterations=32, with_gated=False)
            gemm_table = {"fp8_tensor_peak_tflops": round(fp8_peak, 1),
                          "fp8_tensor_peak_source": "cuBLASLt E4M3 8192^3 measured in this run",
                          "ring": "weight copies >= 512 MB per site (HBM-cold), CUDA graph of 32 launches x 5 replays",
                          "points": gemm_sweep.compact(rows)}
        except Exception as error:       # the table is an annex of the line; the metric does not depend on it
            gemm_table = {"error": str(error)[:160]}

    per_rank = gather_over_ranks([total_ms / steps, submit_seconds * 1e3 / steps], device, world)
    total_ms, e2e_ms = max_over_ranks([total_ms, e2e_seconds * 1e3], device, world)

    if rank == 0:
        hbm_peak, peak_kind = peaks()
        weight_bytes = model.weight_bytes(use_fp8)
        mean_context = float(np.mean(batch.contexts)) + warmup + steps / 2.0
        step_bytes = weight_bytes + 6 * STEP_SEQUENCES * mean_context * 2048
        if arguments.skip_cpu:
            cpu_tokens, cpu_description, threads = None, "skipped", 0
        else:
            cpu_tokens, _, cpu_description, threads = step_cpu_sample(model, batch, token_ids, use_fp8,
                                                                      arguments.cpu_sequences or STEP_SEQUENCES, 1)
        per_step = {name: ops_count // profile_steps for name, (_, ops_count) in regions.items()}
        # GPU kernels per step, counted from the captured graph; the matmuls that the library handed to cuBLASLt
        # during an eager step (one kernel each) are cuBLASLt's, everything else is this library's
        graph_kernels = executor.graph_kernels()
        launches = graph_kernels - library_launches
        line = {
            "metric": STEP_METRIC, "value": STEP_SEQUENCES * steps * world / (total_ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": total_ms / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16+e4m3" if use_fp8 else "bf16",
            "data": "synthetic",
            "config": {"workload": STEP_WORKLOAD, "sequences": STEP_SEQUENCES, "contexts": list(STEP_CONTEXT),
                       "page_size": 16, "pool_pages_per_layer": STEP_POOL_PAGES, "fp8_sites": 16 if use_fp8 else 0,
                       "sampling": "greedy", "replicas": world, "step": "CUDA graph replay, metadata advanced on device",
                       "l2": "inputs exceed L2 (about 5 GB of weights and KV read per step)"},
            "tpot_p50_ms": float(np.median(step_ms)), "tpot_p95_ms": float(np.percentile(step_ms, 95)),
            "step_hbm_frac": step_bytes / (total_ms / steps * 1e-3) / 1e9 / hbm_peak,
            "step_algorithmic_bytes": step_bytes,
            "kv_gbs": kv_bytes / attention_seconds / 1e9,
            "regions_eager_ms_per_step": {name: ms / profile_steps for name, (ms, _) in regions.items()},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak,
                         "traffic": ATTENTION_TRAFFIC_FACTOR * (kv_bytes_graph + other_bytes_graph),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 16-sequence launch = "
                                           "1.001 x its algorithmic bytes, scaled by the keys read "
                                           "(profiles/ragged_decode_attention_config1.md)",
                         "peak_source": peak_kind,
                         "kernel": "ragged_decode_attention_kernel, unsplit at 128 sequences (one attention layer)",
                         "timing": "CUDA events around 8 replays of a graph holding the step's 6 attention launches "
                                   "(one per layer, each on its own cache)",
                         "us_per_launch": attention_graph_seconds * 1e6,
                         "frac_from_eager_pass_events": achieved_eager / hbm_peak,
                         "algorithmic_bytes_per_launch": kv_bytes_graph + other_bytes_graph},
            "cpu_baseline": {"value": cpu_tokens, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": cpu_description},
            "e2e": {"value": STEP_SEQUENCES * e2e_steps * world / (e2e_ms * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps},
            "gpu_launches": launches * steps, "cublaslt_launches": library_launches * steps,
            "reference_kernels_same_gpu": reference_kernels,
            "gemm_roofline": gemm_table,
            "graph_timeline": graph_timeline,
            "replicas": {"tok_s_sum_of_replicas": sum(STEP_SEQUENCES / (ms * 1e-3) for ms, _ in per_rank),
                         "tok_s_from_slowest_replica": STEP_SEQUENCES * steps * world / (total_ms * 1e-3),
                         "ms_per_step_per_rank": [round(ms, 4) for ms, _ in per_rank],
                         "step_submit_cpu_ms_per_rank": [round(cpu, 4) for _, cpu in per_rank],
                         "note": "independent replicas, no collective on the data path; `value` uses the slowest "
                                 "replica's time, the sum adds each replica's own rate"},
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    executor.close()
    blaslt.close()
    if world > 1:
        dist.destroy_process_group()


def step_timeline(executor, model, device_batch, stream, use_fp8, replays=6):
    """Per-kernel picture of the replayed step from CUPTI activity records: for every kernel name its launches per
    step, its summed duration and its exclusive time (the part of it during which no earlier kernel of the step was
    still running; the dependent launches overlap a kernel's start with its predecessor's end).  A diagnostic: the
    records are taken on extra replays after the timed region, never on the timed ones."""
    import re
    import torch
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as profile:
        for _ in range(replays):
            executor.step_graph(model, device_batch, use_fp8=use_fp8, advance=True)
        stream.synchronize()
    records = sorted((event.time_range.start, event.time_range.end, event.name) for event in profile.events()
                     if event.device_type == torch.autograd.DeviceType.CUDA)
    starts = [index for index, record in enumerate(records) if "decode_metadata" in record[2]]
    if len(starts) < 3:
        return {"error": "no kernel records"}
    first, last = starts[1], starts[-1]                      # whole steps only, the first one left out
    steps = len(starts) - 2
    table = {}
    frontier = records[first][0]
    for begin, end, name in records[first:last]:
        short = name
        for prefix in ("void ", "lfm25::", "(anonymous namespace)::"):
            short = short.replace(prefix, "")
        short = re.sub(r"\(.*", "", short)
        entry_ = table.setdefault(short[:48], [0, 0.0, 0.0])
        entry_[0] += 1
        entry_[1] += end - begin
        entry_[2] += max(0.0, end - max(begin, frontier))
        frontier = max(frontier, end)
    span = (records[last][0] - records[first][0]) / steps
    kernels = [{"kernel": name, "launches_per_step": count / steps, "us_per_step": round(duration / steps, 2),
                "exclusive_us_per_step": round(exclusive / steps, 2)}
               for name, (count, duration, exclusive) in sorted(table.items(), key=lambda item: -item[1][2])]
    mean_context = float(device_batch.positions.cpu().numpy().view(np.uint32).mean()) + 1.0
    return {"steps": steps, "us_per_step": round(span, 2), "mean_context_tokens_after": round(mean_context, 1),
            "note": "taken after the timed, clock-sampling and profiling steps: the contexts are longer here than in "
                    "the timed region, by one token per step run since",
            "kernels": kernels}


def reference_kernel_step(model, device_batch, stream, use_fp8, repeats=16):
    """Times the decode step as the reference runs it -- its own kernels (oracle/_ref, compiled for sm_100a from
    the reference's sources) with cuBLASLt GEMMs between them, in the order of src/model/decode_executor.rs:183-443
    -- on this benchmark's weights, caches and metadata.  The sequence is replayed from a CUDA graph, so the
    figure has no launch or host overhead in it (the reference launches eagerly and synchronises every step): it is
    the floor of the reference's step time on this GPU.  Runs last: it overwrites the caches' newest rows."""
    import torch
    from oracle import refstep

    step = refstep.ReferenceKernelStep(model, device_batch.num_tokens, use_fp8=use_fp8)
    arguments_ = (device_batch.token_ids, device_batch.positions, device_batch.request_slots,
                  device_batch.physical_slots, device_batch.block_tables)
    step.forward(*arguments_)                      # eager once: creates the scale tensors, warms cuBLASLt up
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step.forward(*arguments_)
    for _ in range(3):
        graph.replay()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(repeats + 1)]
    stream.synchronize()
    marks[0].record()
    for index in range(repeats):
        graph.replay()
        marks[index + 1].record()
    stream.synchronize()
    times = [marks[i].elapsed_time(marks[i + 1]) for i in range(repeats)]
    return {"step_ms_graph_replay": float(np.median(times)), "step_launches": step.launches,
            "step_note": "reference kernels + cuBLASLt (torch.matmul / torch._scaled_mm) in the reference's op order, "
                         "CUDA graph replay: no launch or host overhead, which the reference's own loop has"}


# ------------------------------------------------------------------------------------ decode GEMM sweep

GEMM_METRIC = "decode GEMM microseconds per launch (E4M3 and BF16 sites, M in {1, 8, 32, 128, 256}, HBM-cold)"
GEMM_WORKLOAD = "config2-decode-gemm-sweep"


def run_gemm_arm(arguments, rank, world):
    """Config 2: every point against max(bytes / HBM peak, flops / tensor peak), with cuBLASLt on the same buffers.
    One JSON line; `value` is the geometric mean over the E4M3 points of cuBLASLt's time over this library's."""
    import torch
    if rank != 0:
        return
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    entry.load_package()
    from lfm25_inference_b200 import gemm_sweep, ops
    hbm_peak, peak_kind = peaks()
    bf16_peak, _ = tensor_peaks()
    fp8_peak = gemm_sweep.measure_fp8_peak(device)
    rows = []
    start = time.perf_counter()
    with ClockSampler(0) as sampler:
        if arguments.gemm_dtype in ("all", "e4m3"):
            rows += gemm_sweep.sweep_fp8(ops, device, hbm_peak, fp8_peak, iterations=arguments.steps, with_quantise=True,
                                         batches=arguments.gemm_batches, sites=arguments.gemm_sites,
                                         with_library=not arguments.no_cublaslt)
        if arguments.gemm_dtype in ("all", "bf16"):
            rows += gemm_sweep.sweep_bf16(ops, device, hbm_peak, bf16_peak, iterations=arguments.steps,
                                          batches=arguments.gemm_batches, sites=arguments.gemm_sites,
                                          with_library=not arguments.no_cublaslt)
    clocks = sampler.summary()
    if ops.device_status()[0] != 0:
        raise RuntimeError("a bounded wait ran out inside the benchmark")
    ratios = [row["cublaslt_us"] / row["ours_us"] for row in rows if row["dtype"] == "e4m3" and "cublaslt_us" in row]
    value = float(np.exp(np.mean(np.log(ratios)))) if ratios else None
    launches = sum(arguments.steps * 5 for row in rows for key in row if key.startswith("ours") and key.endswith("_us"))
    line = {
        "metric": GEMM_METRIC, "value": value, "unit": "x cuBLASLt (geometric mean of time ratios, E4M3 points)",
        "n_gpus": 1, "steps": arguments.steps, "warmup": 3, "ms_per_step": None, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 / bf16 operands, fp32 accumulation", "data": "synthetic",
        "config": {"workload": GEMM_WORKLOAD, "batches": gemm_sweep.BATCHES,
                   "l2": "weights rotate over >= 512 MB of distinct copies per site (four times the L2)"},
        "peaks": {"hbm_gbs": hbm_peak, "hbm_source": peak_kind, "fp8_tflops": fp8_peak,
                  "fp8_source": "cuBLASLt E4M3 8192^3 measured in this run", "bf16_tflops": bf16_peak},
        "table": gemm_sweep.compact(rows), "rows": rows, "gpu_launches": launches, "clocks": clocks,
        "seconds": time.perf_counter() - start,
    }
    print(json.dumps(line), flush=True)


def _inv_freq():
    index = np.arange(32, dtype=np.float32)
    return np.power(np.float32(1.0e6), -(np.float32(2.0) * index) / np.float32(64.0)).astype(np.float32)


# ------------------------------------------------------------------------------------ chunked prefill step

PREFILL_METRIC = "prefill tok/s (mixed step: 8 chunks of 512 prompt tokens on prefixes of 0..3584 cached tokens)"
PREFILL_WORKLOAD = "chunked-prefill-8x512-prefix0-3584-bf16"
PREFILL_CHUNK = 512
PREFILL_PREFIXES = [0, 512, 1024, 1536, 2048, 2560, 3072, 3584]


def run_prefill_arm(arguments, rank, world):
    """One step = one mixed step of the executor holding eight 512-token prefill chunks (the chunk size the
    reference's planner prefers, src/scheduler/planner.rs:201) whose sequences already have 0..3584 tokens in the
    paged cache: 4096 tokens per step, BF16 at every site (the step is above the FP8 batch limit, as in the
    reference).  `roofline` is the mixed-step attention kernel (tcgen05 / TMEM): tensor-core flops
    4 * 2048 * sum(position + 1) per launch over its CUDA-event time in an instrumented pass, against the measured
    dense BF16 peak."""
    import torch
    import torch.distributed as dist

    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    entry.load_package()
    from lfm25_inference_b200 import model as lfm_model
    from lfm25_inference_b200 import ops, workloads

    seed = 5 + rank
    chunks = [PREFILL_CHUNK] * len(PREFILL_PREFIXES)
    pages = sum((prefix + PREFILL_CHUNK + 15) // 16 for prefix in PREFILL_PREFIXES)
    batch = workloads.mixed_step_batch(seed, PREFILL_PREFIXES, chunks, pages)
    model = lfm_model.RandomModel(seed, device, pages, batch.num_segments)
    model.fill_caches(seed + 1)
    token_ids = np.random.default_rng(seed).integers(0, lfm_model.VOCAB, size=batch.num_tokens).astype(np.uint32)
    steps, warmup = arguments.steps, max(arguments.warmup, 3)
    stream = torch.cuda.Stream(device=device)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        blaslt = ops.BlasLt()
        executor = lfm_model.DecodeExecutor(blaslt, batch.num_tokens, maximum_segments=batch.num_segments)
        device_batch = lfm_model.RaggedBatch(device, batch, token_ids)
        for _ in range(warmup):
            executor.forward_ragged(model, device_batch, use_fp8=False)
        stream.synchronize()
        if world > 1:
            dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as sampler:
            stream.synchronize()
            start.record()
            for _ in range(steps):
                executor.forward_ragged(model, device_batch, use_fp8=False)
            stop.record()
            stream.synchronize()
            total_ms = start.elapsed_time(stop)
            until = time.perf_counter() + 0.5
            while total_ms < 500.0 and time.perf_counter() < until:
                executor.forward_ragged(model, device_batch, use_fp8=False)
                stream.synchronize()
        clocks = sampler.summary()

        # e2e: the serving call -- upload the step's token ids from pinned memory, run, download the sampled ids
        pinned_ids = torch.from_numpy(token_ids.view(np.int32).copy()).pin_memory()
        host_sampled = torch.empty(batch.num_segments, dtype=torch.int32).pin_memory()
        e2e_steps = min(steps, 16)
        stream.synchronize()
        begin = time.perf_counter()
        for _ in range(e2e_steps):
            device_batch.token_ids.copy_(pinned_ids, non_blocking=True)
            executor.forward_ragged(model, device_batch, use_fp8=False)
            executor.download_sampled(host_sampled)
            stream.synchronize()
        e2e_ms = (time.perf_counter() - begin) * 1e3

        executor.profile(True)
        profile_steps = 4
        for _ in range(profile_steps):
            executor.forward_ragged(model, device_batch, use_fp8=False)
        regions = executor.profile(False, collect=True)
        graph_free_launches = sum(ops_count for _, ops_count in regions.values()) // profile_steps

        attention_ms, attention_ops = regions["attention"]
        attention_seconds = attention_ms / max(attention_ops, 1) * 1e-3
        attention_flops = 4.0 * 2048.0 * float((batch.positions.astype(np.float64) + 1.0).sum())
        # the reference's own hybrid kernel on the same buffers
        reference_kernels = None
        if rank == 0:
            try:
                from oracle import refkernels
                if refkernels.available():
                    layer = next(layer for layer in model.layers if layer.is_attention)
                    query = torch.randn((batch.num_tokens, 32, 64), device=device, dtype=torch.bfloat16)
                    key = torch.randn((batch.num_tokens, 8, 64), device=device, dtype=torch.bfloat16)
                    output = torch.zeros_like(query)
                    arguments_list = [query, key, key, layer.tensors["key_cache"], layer.tensors["value_cache"],
                                      device_batch.block_tables, device_batch.request_slots, device_batch.positions,
                                      device_batch.segment_offsets, output]
                    refkernels.hybrid_ragged_attention(*arguments_list)
                    stream.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    refkernels.hybrid_ragged_attention(*arguments_list)
                    b.record()
                    stream.synchronize()
                    reference_kernels = {"hybrid_attention_us_per_layer": a.elapsed_time(b) * 1e3,
                                         "ours_us_per_layer": attention_seconds * 1e6}
            except Exception as error:   # the reference images are optional
                reference_kernels = {"unavailable": str(error)[:120]}
    total_ms, e2e_ms = max_over_ranks([total_ms, e2e_ms], device, world)
    if rank == 0:
        peak_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        tensor_peak, peak_source = 1590.0, "fallback"
        if os.path.exists(peak_path):
            with open(peak_path) as handle:
                tensor_peak, peak_source = float(json.load(handle)["bf16_tflops"]), "measured"
        achieved = attention_flops / attention_seconds / 1e12
        cpu = None
        if not arguments.skip_cpu:
            cpu = prefill_cpu_sample(model, batch, token_ids)
        line = {
            "metric": PREFILL_METRIC, "value": batch.num_tokens * steps * world / (total_ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": total_ms / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": PREFILL_WORKLOAD, "segments": batch.num_segments, "chunk": PREFILL_CHUNK,
                       "prefixes": PREFILL_PREFIXES, "tokens_per_step": batch.num_tokens, "page_size": 16,
                       "replicas": world, "step": "eager launches (no graph)",
                       "l2": "2.3 GB of BF16 weights streamed per step exceed L2"},
            "regions_eager_ms_per_step": {name: ms / profile_steps for name, (ms, _) in regions.items()},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
                         "frac": achieved / tensor_peak, "traffic": None, "peak_source": peak_source,
                         "kernel": "hybrid_attention_umma_kernel (one attention layer; tcgen05 / TMEM)",
                         "algorithmic_flops_per_launch": attention_flops},
            "cpu_baseline": cpu,
            "e2e": {"value": batch.num_tokens * e2e_steps * world / (e2e_ms * 1e-3), "unit": "tok/s",
                    "h2d_bytes_per_step": int(token_ids.nbytes), "d2h_bytes_per_step": 4 * batch.num_segments,
                    "steps": e2e_steps},
            "gpu_launches": graph_free_launches * steps,
            "reference_kernels_same_gpu": reference_kernels, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    executor.close()
    blaslt.close()
    if world > 1:
        dist.destroy_process_group()


def prefill_cpu_sample(model, batch, token_ids):
    """CPU oracle on a small mixed step of the same kind (one 64-token chunk on a 192-token prefix)."""
    from oracle import step_oracle
    from lfm25_inference_b200 import workloads
    from oracle import oracle
    oracle.use_all_cores()
    host = step_oracle.HostModel(model)
    small = workloads.MixedStepBatch(batch.num_pages, batch.block_tables[:1].copy(), np.array([192]), np.array([64]),
                                     np.zeros(1, dtype=np.uint32))
    for layer in host.layers:
        if "conv_state" in layer:
            layer["conv_state"] = np.ascontiguousarray(layer["conv_state"][:1])
    begin = time.perf_counter()
    step_oracle.ragged_step(host, token_ids[:64], small, False)
    seconds = time.perf_counter() - begin
    return {"value": 64 / seconds, "unit": "tok/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": "one mixed step with one 64-token chunk on a 192-token prefix (16 layers, BF16), once"}


# ------------------------------------------------------------------------------------ serving trace (config 4)

SERVING_METRIC = "serving generated tok/s (continuous batching over a Poisson trace, 64 request slots)"
SERVING_WORKLOAD = "config4-poisson-trace-prompt-lognormal512-output-u64-512-shared-prefix256"


def serving_trace(seed, count, rate_per_s):
    """BASELINE config 4 as seeded synthetic requests: Poisson arrivals (exponential gaps), prompt length
    round(exp(N(ln 512, 1.0))) clipped to [16, 8192] (the spread 1.0 is an assumption of this build: the source names
    only the median), uniform token ids, output length U{64..512}, and half of the requests starting with one fixed
    256-token prefix."""
    from lfm25_inference_b200 import model as lfm_model
    from lfm25_inference_b200 import serving
    rng = np.random.default_rng(seed)
    shared = rng.integers(0, lfm_model.VOCAB, size=256).astype(np.uint32)
    arrivals = np.cumsum(rng.exponential(1.0 / rate_per_s, size=count))
    requests = []
    for index in range(count):
        length = int(np.clip(round(float(np.exp(rng.normal(np.log(512.0), 1.0)))), 16, 8192))
        prompt = rng.integers(0, lfm_model.VOCAB, size=length).astype(np.uint32)
        if rng.random() < 0.5:
            prompt = np.concatenate([shared, prompt])[:8192]
        requests.append(serving.Request(index, prompt, int(rng.integers(64, 513)), int(arrivals[index] * 1e6)))
    return requests


def run_dispatched_serving_arm(arguments, rank, world):
    """Config 4 over replicas: one engine per GPU, one trace for the whole job, a front on rank 0 that assigns every
    request at its arrival time with the library's dispatcher (prefix-hash affinity, bounded imbalance).  The only
    channel between the processes is a host key-value store; no GPU collective runs.  `value` = tokens generated by
    all replicas / time from the start of the trace until the last replica drained."""
    import threading
    import torch
    import torch.distributed as dist

    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("gloo")                 # host-side control plane only: barrier, store, gather
        store = dist.PrefixStore("lfm25-serving/", dist.distributed_c10d._get_default_store())
    else:
        store = dist.HashStore()
    entry.load_package()
    from lfm25_inference_b200 import model as lfm_model
    from lfm25_inference_b200 import serving

    slots, max_sequence = 64, 8192 + 512 + 16
    pages = slots * ((max_sequence + 15) // 16) // 2 + 4096
    stream = torch.cuda.Stream(device=device)
    with torch.cuda.stream(stream):
        model = lfm_model.RandomModel(4, device, pages, slots)          # replicas hold the same weights
        engine = serving.ServingEngine(model, device, max_slots=slots, max_sequence_tokens=max_sequence,
                                       max_prefill_tokens=512, radix_pages=4096, checkpoint_capacity=128,
                                       use_fp8=not arguments.no_fp8, admission_control=arguments.admission_control)
        engine.calibrate()
        for _ in range(max(arguments.warmup, 1)):
            serving.run_trace(engine, serving_trace(100 + rank, 8, 1000.0))
        before = engine.snapshot()
        trace = serving_trace(4, arguments.requests * world, arguments.rate * world)     # the same on every rank
        if world > 1:
            dist.barrier()
        if rank == 0:
            store.set("origin", repr(time.time() + 0.25))
        origin = float(store.get("origin").decode())
        front_result = {}
        front = None
        if rank == 0:
            front = threading.Thread(target=lambda: front_result.update(serving.run_front(store, world, trace, origin)))
            front.start()
        with ClockSampler(local_rank) as sampler:
            result = serving.run_replica(engine, store, rank, trace, origin)
        clocks = sampler.summary()
        if front is not None:
            front.join()
        after = engine.snapshot()
    result["stats"] = {name: after["stats"][name] - before["stats"][name] for name in before["stats"]}
    result["prefix_cache"] = {name: after["prefix_cache"][name] - before["prefix_cache"][name]
                              for name in ("hits", "misses")}
    result["clocks"] = clocks
    gathered = [result]
    if world > 1:
        gathered = [None] * world if rank == 0 else None
        dist.gather_object(result, gathered, dst=0)
    if rank == 0:
        print(json.dumps(dispatched_serving_line(arguments, world, trace, gathered, front_result)), flush=True)
    engine.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def dispatched_serving_line(arguments, world, trace, gathered, front_result):
    """The JSON line of the dispatched serving run from the replicas' records (host arithmetic only)."""
    records = [record for replica in gathered for record in replica["requests"]]
    finished = [record for record in records if not record["rejected"] and record["generated"] > 0]
    rejected = [record for record in records if record["rejected"]]
    makespan_ms = max(replica["drained_us"] for replica in gathered) / 1e3
    generated = sum(record["generated"] for record in finished)
    prompt_tokens = sum(record["prompt_len"] for record in finished)
    ttft = np.array([record["ttft_us"] for record in finished]) / 1e3
    tpot = np.array([record["tpot_us"] for record in finished if record["tpot_us"] > 0]) / 1e3
    hits = sum(replica["prefix_cache"]["hits"] for replica in gathered)
    misses = sum(replica["prefix_cache"]["misses"] for replica in gathered)
    reused = sum(replica["stats"]["reused_prompt_tokens"] for replica in gathered)
    steps = sum(replica["stats"]["steps"] for replica in gathered)
    value = generated / (makespan_ms * 1e-3)
    per_replica = []
    for replica in gathered:
        mine = [record for record in replica["requests"] if not record["rejected"]]
        per_replica.append({
            "replica": replica["replica"], "requests": len(replica["requests"]),
            "generated_tokens": sum(record["generated"] for record in mine),
            "drained_ms": replica["drained_us"] / 1e3, "steps": replica["stats"]["steps"],
            "mixed_steps": replica["stats"]["mixed_steps"],
            "gpu_busy_frac": replica["stats"]["gpu_ms"] / max(replica["drained_us"] / 1e3, 1e-9),
            "prefix_hits": replica["prefix_cache"]["hits"], "prefix_misses": replica["prefix_cache"]["misses"],
            "sm_mhz": replica["clocks"].get("sm_mhz"), "clock_reasons": replica["clocks"].get("reasons")})
    return {
        "metric": SERVING_METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": 1,
        "warmup": arguments.warmup, "ms_per_step": makespan_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if arguments.no_fp8 else "bf16+e4m3", "data": "synthetic",
        "config": {"workload": SERVING_WORKLOAD + "-dispatched", "requests": len(trace),
                   "rate_per_s": arguments.rate * world, "request_slots_per_replica": 64,
                   "maximum_prefill_tokens": 512, "page_size": 16, "prompt_sigma": 1.0, "replicas": world,
                   "dispatch": "one trace, front on rank 0, lfm25_dispatcher_assign_bounded (prefix hash of the first "
                               "256 prompt tokens, slack 8192 tokens), host key-value store, no collective",
                   "step": "native engine loop per replica, one host sync per step"},
        "requests_per_s": len(finished) / (makespan_ms * 1e-3),
        "admission_control": bool(arguments.admission_control), "rejected_requests": len(rejected),
        "prompt_tokens": prompt_tokens, "generated_tokens": generated,
        "ttft_p50_ms": float(np.percentile(ttft, 50)), "ttft_p95_ms": float(np.percentile(ttft, 95)),
        "tpot_p50_ms": float(np.percentile(tpot, 50)), "tpot_p95_ms": float(np.percentile(tpot, 95)),
        "engine_steps": steps,
        "prefix_cache": {"hits": hits, "misses": misses, "hit_rate": hits / max(hits + misses, 1),
                         "reused_prompt_tokens": reused, "reused_frac": reused / max(prompt_tokens, 1)},
        "per_replica": per_replica,
        "front": {"handed": front_result.get("handed"),
                  "outstanding_tokens_at_end": front_result.get("outstanding_tokens"),
                  "failed_replicas": front_result.get("failed_replicas"),
                  "redispatched_requests": len(front_result.get("redispatched_requests") or []),
                  "unfinished_requests": len(front_result.get("unfinished_requests") or [])},
        "roofline": None, "cpu_baseline": None,
        "e2e": {"value": value, "unit": "tok/s",
                "h2d_bytes_per_step": 4 * (prompt_tokens + generated) * 3 // max(steps, 1),
                "d2h_bytes_per_step": 4 * 64, "steps": steps},
        "gpu_launches": None, "clocks": gathered[0]["clocks"],
    }


def run_serving_arm(arguments, rank, world):
    """One "step" = the whole trace.  `value` = generated tokens / makespan, measured end to end through the serving
    loop (token ids in host memory in, sampled ids in host memory out, every step synchronised), so `e2e` is the same
    number.  Each rank serves its own trace (replicas)."""
    import torch
    import torch.distributed as dist

    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    entry.load_package()
    from lfm25_inference_b200 import model as lfm_model
    from lfm25_inference_b200 import serving

    slots, max_sequence = 64, 8192 + 512 + 16
    pages = slots * ((max_sequence + 15) // 16) // 2 + 4096      # half of the worst case plus the radix budget
    stream = torch.cuda.Stream(device=device)
    with torch.cuda.stream(stream):
        model = lfm_model.RandomModel(4 + rank, device, pages, slots)
        engine = serving.ServingEngine(model, device, max_slots=slots, max_sequence_tokens=max_sequence,
                                       max_prefill_tokens=512, radix_pages=4096, checkpoint_capacity=128,
                                       use_fp8=not arguments.no_fp8,
                                       admission_control=arguments.admission_control)
        engine.calibrate()
        for _ in range(max(arguments.warmup, 1)):                   # short warm-up traces (plans, attributes)
            serving.run_trace(engine, serving_trace(100 + rank, 8, 1000.0))
        if world > 1:
            dist.barrier()
        with ClockSampler(local_rank) as sampler:
            result = serving.run_trace(engine, serving_trace(4 + rank, arguments.requests, arguments.rate))
        clocks = sampler.summary()
        makespan_ms = result["makespan_us"] / 1e3
    (makespan_ms,) = max_over_ranks([makespan_ms], device, world)
    if rank == 0:
        rejected = [entry_ for entry_ in result["requests"] if entry_["rejected"]]
        finished = [entry_ for entry_ in result["requests"] if not entry_["rejected"]]
        reasons = {}
        for entry_ in rejected:
            reasons[entry_["rejected"]] = reasons.get(entry_["rejected"], 0) + 1
        ttft = np.array([entry_["ttft_us"] for entry_ in finished]) / 1e3
        tpot = np.array([entry_["tpot_us"] for entry_ in finished if entry_["tpot_us"] > 0]) / 1e3
        generated = sum(entry_["generated"] for entry_ in finished)
        prompt_tokens = sum(entry_["prompt_len"] for entry_ in finished)
        stats, prefix = result["stats"], result["prefix_cache"]
        value = generated * world / (makespan_ms * 1e-3)
        line = {
            "metric": SERVING_METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": 1,
            "warmup": arguments.warmup, "ms_per_step": makespan_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if arguments.no_fp8 else "bf16+e4m3", "data": "synthetic",
            "config": {"workload": SERVING_WORKLOAD, "requests": arguments.requests, "rate_per_s": arguments.rate,
                       "request_slots": slots, "maximum_prefill_tokens": 512, "page_size": 16,
                       "prompt_sigma": 1.0, "replicas": world, "step": "native engine loop, eager launches, one host sync per step"},
            "requests_per_s": len(finished) * world / (makespan_ms * 1e-3),
            "admission_control": bool(arguments.admission_control), "rejected_requests": len(rejected),
            "rejected_by_reason": reasons,
            "prompt_tokens": prompt_tokens, "generated_tokens": generated,
            "ttft_p50_ms": float(np.percentile(ttft, 50)), "ttft_p95_ms": float(np.percentile(ttft, 95)),
            "tpot_p50_ms": float(np.percentile(tpot, 50)), "tpot_p95_ms": float(np.percentile(tpot, 95)),
            "engine_steps": stats["steps"], "mixed_steps": stats["mixed_steps"], "decode_steps": stats["decode_steps"],
            "gpu_busy_frac": stats["gpu_ms"] / makespan_ms,
            "prefix_cache": {"hits": prefix["hits"], "misses": prefix["misses"],
                             "reused_prompt_tokens": stats["reused_prompt_tokens"],
                             "reused_frac": stats["reused_prompt_tokens"] / max(prompt_tokens, 1)},
            "cost_curves_ms": engine.predicted_ms(),
            "roofline": None, "cpu_baseline": None,
            "e2e": {"value": value, "unit": "tok/s",
                    "h2d_bytes_per_step": 4 * (prompt_tokens + generated) * 3 // max(stats["steps"], 1),
                    "d2h_bytes_per_step": 4 * slots, "steps": stats["steps"]},
            "gpu_launches": None, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    engine.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    arguments = parse_arguments()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if arguments.workload == "step":
        if arguments.impl == "reference":
            run_step_reference_arm(arguments, rank)
        else:
            run_step_arm(arguments, rank, world)
        return
    if arguments.workload == "gemm":
        if arguments.impl == "reference":
            raise SystemExit("--impl reference times the decode workloads")
        run_gemm_arm(arguments, rank, world)
        return
    if arguments.workload == "serving":
        if arguments.impl == "reference":
            raise SystemExit("--impl reference times the decode workloads")
        if arguments.dispatch:
            run_dispatched_serving_arm(arguments, rank, world)
        else:
            run_serving_arm(arguments, rank, world)
        return
    if arguments.workload == "prefill":
        if arguments.impl == "reference":
            raise SystemExit("--impl reference times the decode workloads; the prefill line carries its own cpu_baseline")
        run_prefill_arm(arguments, rank, world)
        return
    if arguments.impl == "reference":
        run_reference_arm(arguments, rank)
        return
    run_gpu_arm(arguments, rank, world)


if __name__ == "__main__":
    main()

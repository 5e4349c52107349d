"""The multi-GPU path is N independent replicas: the only cross-rank step is the timing reduction (maximum over
ranks) that turns per-replica times into whole-job throughput.  Checked here with two gloo ranks on CPU, together
with the dispatcher that spreads requests over the replicas."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    # rank 1 is the slow replica: its times must define the job on every rank
    mine = [10.0 + 5.0 * rank, 100.0 - 20.0 * rank]
    reduced = bench.max_over_ranks(mine, torch.device("cpu"), world)
    dist.barrier()
    results[rank] = (reduced, bench.aggregate_throughput(128 * 4, world, reduced[0]))
    dist.destroy_process_group()


def test_two_replicas_report_the_slowest_time_and_the_summed_throughput():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
    for rank in range(world):
        reduced, throughput = results[rank]
        assert reduced == [15.0, 100.0]
        assert throughput == pytest.approx(128 * 4 * 2 / 15e-3)


def test_single_replica_needs_no_process_group():
    import bench
    assert bench.max_over_ranks([3.0, 4.0], torch.device("cpu"), 1) == [3.0, 4.0]
    assert bench.aggregate_throughput(64, 1, 2.0) == pytest.approx(32000.0)


class _FakeEngine:
    """The engine's interface with no GPU behind it: every active request yields one token per step."""

    def __init__(self, step_seconds=0.0):
        self.waiting, self.running, self.step_seconds = [], {}, step_seconds

    def submit(self, request):
        self.waiting.append(request)

    def queued(self):
        return len(self.waiting)

    def active(self):
        return len(self.running)

    def step(self, now_us):
        if self.step_seconds:
            import time
            time.sleep(self.step_seconds)
        for request in self.waiting:
            self.running[request.request_id] = [request, 0]
        self.waiting = []
        events = []
        for request_id in list(self.running):
            request, produced = self.running[request_id]
            produced += 1
            finished = produced == request.max_new_tokens
            events.append((request_id, 7, finished, now_us, 0, 0))
            if finished:
                del self.running[request_id]
            else:
                self.running[request_id][1] = produced
        return events, 0.0


def _dispatch_trace():
    import numpy as np
    from lfm25_inference_b200 import serving
    rng = np.random.default_rng(11)
    shared = rng.integers(0, 65536, size=256).astype(np.uint32)
    requests = []
    for index in range(24):
        prompt = rng.integers(0, 65536, size=int(rng.integers(16, 600))).astype(np.uint32)
        if index % 2 == 0:
            prompt = np.concatenate([shared, prompt])
        requests.append(serving.Request(index, prompt, int(rng.integers(2, 9)), index * 4000))
    return requests


def _dispatch_rank_main(rank, world, port, results):
    import threading
    import time
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as entry
    entry.load_package()
    from lfm25_inference_b200 import serving
    store = dist.PrefixStore("trace/", dist.distributed_c10d._get_default_store())
    trace = _dispatch_trace()
    dist.barrier()
    if rank == 0:
        store.set("origin", repr(time.time() + 0.05))
    origin = float(store.get("origin").decode())
    front_result = {}
    front = None
    if rank == 0:
        front = threading.Thread(target=lambda: front_result.update(serving.run_front(store, world, trace, origin,
                                                                                      slack_tokens=1500)))
        front.start()
    mine = serving.run_replica(_FakeEngine(), store, rank, trace, origin)
    if front is not None:
        front.join()
    dist.barrier()
    done = [int(store.add(f"done/{replica}", 0)) for replica in range(world)]
    results[rank] = (mine, dict(front_result), done)
    dist.destroy_process_group()


def test_one_trace_is_dispatched_over_two_replicas():
    """The front on rank 0 hands a single trace out over two replica processes through the host store: every request
    is served exactly once, on the replica the front chose, each replica reports back what it finished, and the
    requests that share a prefix stay together until their home replica is too far ahead of the other."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    from lfm25_inference_b200 import serving
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    port = 31500 + os.getpid() % 2000
    mp.spawn(_dispatch_rank_main, args=(world, port, results), nprocs=world, join=True)
    trace = _dispatch_trace()
    front = results[0][1]
    served = {}
    for rank in range(world):
        mine, _, done = results[rank]
        assert mine["replica"] == rank
        for record in mine["requests"]:
            assert record["request_id"] not in served
            served[record["request_id"]] = rank
            request = trace[record["request_id"]]
            assert record["generated"] == request.max_new_tokens and record["rejected"] is None
            assert record["ttft_us"] is not None and record["ttft_us"] >= 0
        assert done[rank] == sum(serving.estimated_tokens(trace[record["request_id"]]) for record in mine["requests"])
    assert served == front["assignment"] and len(served) == len(trace)
    assert front["handed"] == [sum(1 for rank in served.values() if rank == replica) for replica in range(world)]
    assert min(front["handed"]) >= 4                               # both replicas worked
    shared_home = serving.prefix_hash(trace[0].prompt) % world
    shared_placed = [served[index] for index in range(0, len(trace), 2)]
    assert shared_placed.count(shared_home) > len(shared_placed) // 2


class _ReplicaGone(Exception):
    pass


class _DyingEngine(_FakeEngine):
    """Serves a few steps, then fails for good (the host-side stand-in for a replica that is lost)."""

    def __init__(self, steps_before_failure, step_seconds):
        super().__init__(step_seconds)
        self.remaining = steps_before_failure

    def step(self, now_us):
        if self.remaining == 0:
            raise _ReplicaGone()
        self.remaining -= 1
        return super().step(now_us)


def _failure_trace():
    import numpy as np
    from lfm25_inference_b200 import serving
    rng = np.random.default_rng(12)
    return [serving.Request(index, rng.integers(0, 65536, size=int(rng.integers(16, 200))).astype(np.uint32), 30,
                            index * 25000) for index in range(40)]


def _failure_rank_main(rank, world, port, results):
    import threading
    import time
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as entry
    entry.load_package()
    from lfm25_inference_b200 import serving
    store = dist.PrefixStore("failure/", dist.distributed_c10d._get_default_store())
    trace = _failure_trace()
    dist.barrier()
    if rank == 0:
        store.set("origin", repr(time.time() + 0.05))
    origin = float(store.get("origin").decode())
    front_result = {}
    front = None
    if rank == 0:
        front = threading.Thread(target=lambda: front_result.update(
            serving.run_front(store, world, trace, origin, failure_timeout_s=0.3)))
        front.start()
    engine = _FakeEngine(0.004) if rank == 0 else _DyingEngine(20, 0.004)      # replica 1 lives for 80 ms
    mine = None
    try:
        mine = serving.run_replica(engine, store, rank, trace, origin)
    except _ReplicaGone:
        pass                                # the replica is gone: no more signs of life, nothing reported
    if front is not None:
        front.join()
    results[rank] = (mine, dict(front_result))
    dist.barrier()
    dist.destroy_process_group()


def test_front_stops_using_a_replica_that_gives_no_sign_of_life():
    """Failure detection and recovery on the host, no GPU involved: replica 1 fails after a few steps (an exception
    in its loop), its heartbeat in the store goes stale, the front marks it failed in the dispatcher after the
    timeout, hands what it had not finished and every later request to the surviving replica, and the trace ends
    with every request served."""
    sys.path.insert(0, ROOT)
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    port = 33500 + os.getpid() % 2000
    mp.spawn(_failure_rank_main, args=(world, port, results), nprocs=world, join=True)
    trace = _failure_trace()
    survivor, front = results[0]
    assert results[1][0] is None
    assert front["failed_replicas"] == [1]
    # whatever the lost replica had been handed and not finished went to the survivor; in the end every request
    # has been served there in full (the ones that started on the lost replica start over)
    assert front["redispatched_requests"] and front["unfinished_requests"] == []
    assignment = front["assignment"]
    assert all(replica == 0 for replica in assignment.values())
    assert all(assignment[request.request_id] == 0 for request in trace[-10:])
    served = {record["request_id"] for record in survivor["requests"] if record["generated"] == 30}
    assert served == {request.request_id for request in trace}
    assert set(front["redispatched_requests"]) <= served


def test_dispatched_serving_line_adds_up_the_replicas():
    """The line of the dispatched serving run from the replicas' records (host arithmetic only): tokens and requests
    are summed over the replicas, the makespan is the slowest replica's, percentiles are taken over all requests."""
    sys.path.insert(0, ROOT)
    import argparse
    import numpy as np
    import bench
    from lfm25_inference_b200 import serving

    def record(request_id, replica, generated, ttft_us, tpot_us, rejected=None):
        return {"request_id": request_id, "prompt_len": 100, "arrival_us": 0, "generated": generated,
                "ttft_us": ttft_us, "tpot_us": tpot_us, "last_token_us": 0, "reused_tokens": 0, "rejected": rejected,
                "replica": replica}

    clocks = {"sm_mhz": 1965.0, "sm_max_mhz": 1965.0, "reasons": []}
    stats = {"steps": 10, "mixed_steps": 4, "decode_steps": 6, "gpu_ms": 900.0, "reused_prompt_tokens": 256,
             "generated_tokens": 0, "prefill_tokens": 0}
    gathered = [
        {"replica": 0, "requests": [record(0, 0, 10, 1000, 2000.0), record(1, 0, 30, 3000, 4000.0)],
         "drained_us": 1_000_000, "stats": dict(stats), "prefix_cache": {"hits": 1, "misses": 1}, "clocks": clocks},
        {"replica": 1, "requests": [record(2, 1, 20, 2000, 3000.0), record(3, 1, 0, None, 0.0, rejected="slots")],
         "drained_us": 2_000_000, "stats": dict(stats), "prefix_cache": {"hits": 0, "misses": 2}, "clocks": clocks},
    ]
    trace = [serving.Request(index, np.zeros(100, dtype=np.uint32), 30, 0) for index in range(4)]
    arguments = argparse.Namespace(warmup=1, rate=2.0, no_fp8=False, admission_control=True)
    front = {"handed": [2, 2], "outstanding_tokens": [0, 0], "failed_replicas": [], "redispatched_requests": [],
             "unfinished_requests": []}
    line = bench.dispatched_serving_line(arguments, 2, trace, gathered, front)
    assert line["n_gpus"] == 2 and line["ms_per_step"] == 2000.0
    assert line["generated_tokens"] == 60 and line["value"] == pytest.approx(30.0)        # 60 tokens in 2 s
    assert line["rejected_requests"] == 1 and line["requests_per_s"] == pytest.approx(1.5)
    assert line["ttft_p50_ms"] == pytest.approx(2.0) and line["tpot_p50_ms"] == pytest.approx(3.0)
    assert line["prefix_cache"]["hits"] == 1 and line["prefix_cache"]["misses"] == 3
    assert [entry["requests"] for entry in line["per_replica"]] == [2, 2]
    assert line["front"]["redispatched_requests"] == 0 and line["config"]["replicas"] == 2

"""Continuous-batching serving over the C ABI.

The GPU-owner loop itself -- request slots, admission with prefix reuse, step planning, the step's device metadata,
mixed prefill / decode steps, token bookkeeping -- is native (`csrc/serving_engine.cu`, `lfm25_engine_*`, the
counterpart of the reference's src/engine/serving/radix_owner.rs).  This module is the thin front of it that the tests
and the benchmark use: it feeds requests in arrival order, calls `lfm25_engine_step` until the trace is drained, and
turns the token events into per-request latency records.  Sampling is greedy; the model is whatever `RandomModel`
the caller built.
"""
from __future__ import annotations

import ctypes
import hashlib
import time
from dataclasses import dataclass

import numpy as np

from . import _abi, ops
from . import model as lfm_model
from ._abi import check, library


# lfm25_engine_event.rejected (include/lfm25_b200.h, LFM25_REJECT_*)
REJECT_REASONS = {1: "sequence_capacity", 2: "prompt_limit", 3: "decode_budget", 4: "ttft", 5: "slots", 6: "kv_pages"}


@dataclass
class Request:
    request_id: int
    prompt: np.ndarray               # uint32
    max_new_tokens: int
    arrival_us: int


class ServingEngine:
    """One engine per GPU, driven from one host thread (the reference's GPU-owner thread)."""

    def __init__(self, model: lfm_model.RandomModel, device, max_slots: int = 64, max_sequence_tokens: int = 8704,
                 max_prefill_tokens: int = 512, radix_pages: int = 4096, checkpoint_capacity: int = 64,
                 use_fp8: bool = True, ttft_slo_us: int = 400_000, tpot_slo_us: int = 50_000,
                 step_budget_ms: float = 40.0, admission_control: bool = False, interactive_prompt_limit: int = 0):
        """`admission_control`: decide every queued request at the next step, admitting it or rejecting it with a
        reason (the reference's admit_request_radix, src/engine/serving/radix_owner.rs:549-708); off, a request that
        does not fit yet waits in the queue."""
        self.model, self.device, self.max_slots = model, device, max_slots
        self.blaslt = ops.BlasLt()
        self.blaslt.bind_current_stream()
        config = _abi.EngineConfig(max_slots, max_sequence_tokens, max_prefill_tokens, radix_pages,
                                   checkpoint_capacity, int(use_fp8), ttft_slo_us, tpot_slo_us, step_budget_ms,
                                   int(admission_control), interactive_prompt_limit)
        self._handle = ctypes.c_void_p()
        check(library().lfm25_engine_create(self.blaslt._handle, model.struct, ctypes.byref(config),
                                            ctypes.byref(self._handle)))
        self._capacity = 2 * max_slots
        self._events = (_abi.EngineEvent * self._capacity)()
        self._count = ctypes.c_size_t(0)
        self._gpu_ms = ctypes.c_float(0.0)

    def calibrate(self) -> None:
        """Measures the planner's cost curves on the idle engine (once, before the first step)."""
        check(library().lfm25_engine_calibrate(self._handle))

    def predicted_ms(self) -> dict:
        """A few points of the calibrated cost curves, for reports."""
        cost = library().lfm25_engine_cost_model(self._handle)
        decode = {batch: float(library().lfm25_cost_model_predict_decode_ms(cost, batch, 2048, 1))
                  for batch in (1, 8, 32, 64)}
        prefill = {tokens: float(library().lfm25_cost_model_predict_prefill_ms(cost, tokens))
                   for tokens in (16, 64, 128, 256, 512)}
        return {"decode_ms_at_context_2048": decode, "prefill_ms": prefill}

    def submit(self, request: Request) -> None:
        prompt = np.ascontiguousarray(request.prompt, dtype=np.uint32)
        check(library().lfm25_engine_submit(self._handle, request.request_id,
                                            prompt.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), prompt.size,
                                            request.max_new_tokens, request.arrival_us))

    def step(self, now_us: int):
        """Admits, plans and runs one step.  Returns (events, gpu_ms); an event is
        (request_id, token, finished, time_us, reused_tokens, rejected): `rejected` is 0 for a token and one of the
        REJECT_* reasons for a request that admission control turned away."""
        check(library().lfm25_engine_step(self._handle, now_us, self._events, self._capacity,
                                          ctypes.byref(self._count), ctypes.byref(self._gpu_ms)))
        events = [(int(e.request_id), int(e.token), bool(e.finished), int(e.time_us), int(e.reused_tokens),
                   int(e.rejected)) for e in self._events[:self._count.value]]
        return events, float(self._gpu_ms.value)

    def active(self) -> int:
        return int(library().lfm25_engine_active(self._handle))

    def queued(self) -> int:
        return int(library().lfm25_engine_queued(self._handle))

    def snapshot(self) -> dict:
        stats, pool, prefix = _abi.EngineStats(), _abi.KvPoolSnapshot(), _abi.PrefixCacheSnapshot()
        library().lfm25_engine_get_stats(self._handle, ctypes.byref(stats), ctypes.byref(pool), ctypes.byref(prefix))

        def fields(struct):
            return {name: getattr(struct, name) for name, _ in struct._fields_}

        return {"stats": fields(stats), "pool": fields(pool), "prefix_cache": fields(prefix)}

    def close(self) -> None:
        if self._handle:
            library().lfm25_engine_destroy(self._handle)
            self._handle = None
        self.blaslt.close()


def run_trace(engine: ServingEngine, requests: list[Request]) -> dict:
    """Drives the engine over a list of requests.  The clock is the wall clock of this process since the call,
    jumped forward to the next arrival whenever the engine is idle.  Returns per-request records (time to first
    token, mean time per output token, tokens) and the engine's counters for the trace."""
    before = engine.snapshot()["stats"]
    pending = sorted(requests, key=lambda request: request.arrival_us)
    records = {request.request_id: {"request_id": request.request_id, "prompt_len": len(request.prompt),
                                    "arrival_us": request.arrival_us, "times_us": [], "tokens": [],
                                    "reused_tokens": 0, "rejected": None} for request in pending}
    origin = time.perf_counter()
    skipped_us = 0
    cursor = 0
    idle_rounds = 0
    while cursor < len(pending) or engine.queued() or engine.active():
        now_us = int((time.perf_counter() - origin) * 1e6) + skipped_us
        if not engine.queued() and not engine.active() and cursor < len(pending) and \
                pending[cursor].arrival_us > now_us:
            skipped_us += pending[cursor].arrival_us - now_us          # idle: jump to the next arrival
            now_us = pending[cursor].arrival_us
        while cursor < len(pending) and pending[cursor].arrival_us <= now_us:
            engine.submit(pending[cursor])
            cursor += 1
        events, _ = engine.step(now_us)
        for request_id, token, _, time_us, reused, rejected in events:
            record = records[request_id]
            if rejected:
                record["rejected"] = REJECT_REASONS.get(rejected, str(rejected))
                continue
            record["times_us"].append(time_us)
            record["tokens"].append(token)
            record["reused_tokens"] = reused
        idle_rounds = 0 if (events or engine.active()) else idle_rounds + 1
        if idle_rounds > 1000:
            raise RuntimeError("the engine makes no progress: a queued request does not fit the page pool")
    makespan_us = int((time.perf_counter() - origin) * 1e6) + skipped_us
    finished = []
    for record in records.values():
        times = record.pop("times_us")
        gaps = np.diff(times) if len(times) > 1 else np.array([])
        record["generated"] = len(record["tokens"])
        record["ttft_us"] = times[0] - record["arrival_us"] if times else None
        record["tpot_us"] = float(gaps.mean()) if gaps.size else 0.0
        finished.append(record)
    after = engine.snapshot()
    stats = {name: after["stats"][name] - before[name] for name in before}
    return {"makespan_us": makespan_us, "wall_s": time.perf_counter() - origin, "requests": finished, "stats": stats,
            "prefix_cache": after["prefix_cache"], "pool": after["pool"]}


# ------------------------------------------------------------------------------ one trace over several replicas
#
# One process per GPU, each with its own engine; one front (a thread of rank 0) that walks a single trace in real
# time and hands every request, at its arrival time, to a replica chosen by the library's dispatcher (least
# outstanding tokens, prefix-hash affinity with bounded imbalance).  Requests travel as indices into the trace, which
# every process builds from the same seed; the channel is a key-value store of the host (torch.distributed's store:
# no GPU collective anywhere).  Keys: "n/<replica>" = requests handed to the replica so far, "q/<replica>/<k>" = index
# of the k-th of them, "done/<replica>" = tokens the replica has finished with (prompt + generated of completed or
# rejected requests), "fin/<replica>" and "f/<replica>/<k>" = how many requests it has finished and which,
# "beat/<replica>" = wall-clock time of the replica's last sign of life, "closed" = set by the front once every
# request of the trace is finished.  A replica whose last sign of life is older than the front's timeout is marked
# failed in the dispatcher (lfm25_dispatcher_mark_failed) and gets no further requests; what it had been handed and
# has not reported finished is handed out again to the others.

HEARTBEAT_PERIOD_S = 0.1

PREFIX_HASH_TOKENS = 256


def prefix_hash(prompt: np.ndarray, tokens: int = PREFIX_HASH_TOKENS):
    """64-bit digest of the first `tokens` prompt ids; None for a shorter prompt (nothing worth an affinity)."""
    if len(prompt) < tokens:
        return None
    data = np.ascontiguousarray(prompt[:tokens], dtype=np.uint32).tobytes()
    return int.from_bytes(hashlib.blake2b(data, digest_size=8).digest(), "little")


def estimated_tokens(request: Request) -> int:
    return int(len(request.prompt) + request.max_new_tokens)


def run_front(store, replicas: int, requests: list[Request], origin_s: float, slack_tokens: int = 8192,
              clock=time.time, sleep=time.sleep, failure_timeout_s: float = 5.0, watch_period_s: float = 0.02) -> dict:
    """Hands out `requests` in arrival order, each at origin_s + arrival, keeps watching until every request is
    finished, and returns the assignment {request_id: replica} with the dispatcher's view of the loads at the end.
    A replica that has given no sign of life for `failure_timeout_s` is marked failed and left out from then on;
    what it had been handed and has not reported finished is handed out again to the replicas that live (the
    request starts over there; its arrival time stays)."""
    from .cache import Dispatcher
    dispatcher = Dispatcher(replicas)
    seen_done = [0] * replicas
    seen_finished = [0] * replicas
    handed = [[] for _ in range(replicas)]          # request indices per replica, in hand-out order
    finished = set()
    failed = []
    redispatched = []
    assignment = {}
    hashes = [prefix_hash(request.prompt) for request in requests]
    state = {"nobody_left": False}

    def hand_out(index: int) -> None:
        request = requests[index]
        replica = dispatcher.assign(estimated_tokens(request), prefix_hash=hashes[index], slack_tokens=slack_tokens)
        store.set(f"q/{replica}/{len(handed[replica])}", str(index))
        handed[replica].append(index)
        store.add(f"n/{replica}", 1)
        assignment[request.request_id] = replica

    def look() -> None:
        """Completions and signs of life reported since the last look; failures found are handled here."""
        now = clock()
        for replica in range(replicas):
            if replica in failed:
                continue
            done = int(store.add(f"done/{replica}", 0))
            if done > seen_done[replica]:
                dispatcher.complete(replica, done - seen_done[replica])
                seen_done[replica] = done
            count = int(store.add(f"fin/{replica}", 0))
            while seen_finished[replica] < count:
                finished.add(int(store.get(f"f/{replica}/{seen_finished[replica]}")))
                seen_finished[replica] += 1
            if store.check([f"beat/{replica}"]):
                last_beat = float(store.get(f"beat/{replica}").decode())
            else:
                last_beat = origin_s                             # a replica that never reported counts from the start
            if now - last_beat > failure_timeout_s:
                if len(failed) + 1 == replicas:
                    state["nobody_left"] = True                  # the last replica is gone too: nothing to hand to
                    continue
                dispatcher.mark_failed(replica)
                failed.append(replica)
                for index in handed[replica]:
                    if index not in finished:
                        redispatched.append(requests[index].request_id)
                        hand_out(index)

    order = sorted(range(len(requests)), key=lambda index: requests[index].arrival_us)
    for index in order:
        wait = origin_s + requests[index].arrival_us * 1e-6 - clock()
        while wait > 0:                                          # keep looking while waiting for the next arrival
            sleep(min(wait, watch_period_s))
            look()
            wait = origin_s + requests[index].arrival_us * 1e-6 - clock()
        look()
        if state["nobody_left"]:
            break
        hand_out(index)
    while len(finished) < len(requests) and not state["nobody_left"]:     # all handed out: wait for the results
        sleep(watch_period_s)
        look()
    store.set("closed", "1")
    return {"assignment": assignment, "handed": [len(indices) for indices in handed], "failed_replicas": failed,
            "redispatched_requests": redispatched,
            "unfinished_requests": sorted(requests[index].request_id for index in range(len(requests))
                                          if index not in finished),
            "outstanding_tokens": [dispatcher.load(replica) for replica in range(replicas)]}


def run_replica(engine, store, replica: int, requests: list[Request], origin_s: float, clock=time.time,
                idle_sleep_s: float = 0.0002) -> dict:
    """The loop of one replica: takes the requests the front has handed to it, steps its engine in real time and
    reports finished tokens back.  `engine` needs submit / step / active / queued (a ServingEngine)."""
    records = {}
    taken = 0
    reported = 0
    closed = False
    first_step_us = None
    busy_until_us = 0
    last_beat = 0.0
    while True:
        if clock() - last_beat >= HEARTBEAT_PERIOD_S:
            last_beat = clock()
            store.set(f"beat/{replica}", repr(last_beat))
        count = int(store.add(f"n/{replica}", 0))
        while taken < count:
            index = int(store.get(f"q/{replica}/{taken}"))
            request = requests[index]
            taken += 1
            records[request.request_id] = {"request_id": request.request_id, "index": index,
                                           "prompt_len": len(request.prompt),
                                           "arrival_us": request.arrival_us, "times_us": [], "tokens": 0,
                                           "reused_tokens": 0, "rejected": None, "replica": replica,
                                           "estimated_tokens": estimated_tokens(request)}
            engine.submit(request)
        if not engine.queued() and not engine.active():
            if closed:
                # one more look at the queue after seeing "closed": the front sets it after its last hand-out
                if int(store.add(f"n/{replica}", 0)) == taken:
                    break
                continue
            closed = store.check(["closed"])
            time.sleep(idle_sleep_s)
            continue
        now_us = int((clock() - origin_s) * 1e6)
        if first_step_us is None:
            first_step_us = now_us
        events, _ = engine.step(now_us)
        if events:
            busy_until_us = int((clock() - origin_s) * 1e6)
        finished_tokens = 0
        finished_now = []
        for request_id, _, finished, time_us, reused, rejected in events:
            record = records[request_id]
            if rejected:
                record["rejected"] = REJECT_REASONS.get(rejected, str(rejected))
                finished_tokens += record["estimated_tokens"]
                finished_now.append(record["index"])
                continue
            record["times_us"].append(time_us)
            record["tokens"] += 1
            record["reused_tokens"] = reused
            if finished:
                finished_tokens += record["estimated_tokens"]
                finished_now.append(record["index"])
        if finished_tokens:
            store.add(f"done/{replica}", finished_tokens)
        for index in finished_now:                      # which requests are finished: what the front re-dispatches by
            store.set(f"f/{replica}/{reported}", str(index))
            reported += 1
        if finished_now:
            store.add(f"fin/{replica}", len(finished_now))
    last_us = busy_until_us          # when this replica produced its last token (it then idles until the trace closes)
    out = []
    for record in records.values():
        times = record.pop("times_us")
        gaps = np.diff(times) if len(times) > 1 else np.array([])
        record["generated"] = record.pop("tokens")
        record["ttft_us"] = int(times[0] - record["arrival_us"]) if times else None
        record["last_token_us"] = int(times[-1]) if times else None
        record["tpot_us"] = float(gaps.mean()) if gaps.size else 0.0
        out.append(record)
    return {"replica": replica, "requests": out, "first_step_us": first_step_us, "drained_us": last_us}

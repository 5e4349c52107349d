"""Host logic of the path (no GPU): the reference's unit tests for the page allocator, the block tables and the
decode scheduler re-expressed against the C ABI, plus the replica dispatcher with a replica failure injected on
the host."""
import numpy as np
import pytest

from lfm25_inference_b200 import Lfm25Error, _abi
from lfm25_inference_b200.cache import (Dispatcher, FixedBlockTables, KvAllocationError, KvPageAllocator,
                                        schedule_decode)

UNASSIGNED = 0xFFFFFFFF


def test_allocator_grows_incrementally_and_reclaims_pages():
    # src/cache/allocator.rs:231-245
    allocator = KvPageAllocator(8, 16)
    reserved = allocator.try_reserve_tokens(64)
    assert reserved == 4
    table = np.full(4, UNASSIGNED, dtype=np.uint32)
    assert allocator.grow_sequence(0, 17, table) == 2
    assert table[:2].tolist() == [0, 1]                       # a fresh pool hands out 0, 1, 2, ...
    assert allocator.snapshot()["allocated_pages"] == 2
    assert allocator.grow_sequence(17, 48, table) == 1
    allocator.release_sequence(48, table)
    allocator.release_reservation(reserved)
    assert allocator.snapshot()["free_pages"] == 8
    assert np.all(table == UNASSIGNED)
    assert allocator.snapshot()["peak_allocated_pages"] == 3


def test_reservation_prevents_collective_growth_oom():
    # src/cache/allocator.rs:247-256
    allocator = KvPageAllocator(4, 16)
    assert allocator.try_reserve_tokens(48) == 3
    with pytest.raises(KvAllocationError) as error:
        allocator.try_reserve_tokens(32)
    assert error.value.code == _abi.KV_LOGICAL_RESERVATION_EXHAUSTED
    with pytest.raises(KvAllocationError) as error:
        allocator.try_reserve_tokens(0)
    assert error.value.code == _abi.KV_SEQUENCE_CAPACITY_EXCEEDED


def test_cached_page_survives_request_release_and_can_be_shared():
    # src/cache/allocator.rs:258-275
    allocator = KvPageAllocator(4, 16)
    reserved = allocator.try_reserve_tokens(16)
    first = np.full(1, UNASSIGNED, dtype=np.uint32)
    allocator.grow_sequence(0, 16, first)
    page = int(first[0])
    allocator.pin_cached_pages([page])
    allocator.release_sequence(16, first)
    allocator.release_reservation(reserved)
    assert allocator.snapshot()["allocated_pages"] == 1 and allocator.snapshot()["cached_pages"] == 1
    allocator.retain_pages([page])
    second = np.array([page], dtype=np.uint32)
    allocator.release_sequence(16, second)
    assert allocator.snapshot()["allocated_pages"] == 1


def test_cached_pages_reduce_future_private_reservation_capacity():
    # src/cache/allocator.rs:277-292
    allocator = KvPageAllocator(4, 16)
    reserved = allocator.try_reserve_tokens(16)
    table = np.full(1, UNASSIGNED, dtype=np.uint32)
    allocator.grow_sequence(0, 16, table)
    allocator.pin_cached_pages([int(table[0])])
    allocator.release_sequence(16, table)
    allocator.release_reservation(reserved)
    assert allocator.try_reserve_pages(3) == 3
    with pytest.raises(KvAllocationError):
        allocator.try_reserve_pages(1)


def test_allocator_error_paths():
    allocator = KvPageAllocator(2, 16)
    table = np.full(4, UNASSIGNED, dtype=np.uint32)
    with pytest.raises(KvAllocationError) as error:
        allocator.grow_sequence(0, 48, table)                 # 3 pages from a pool of 2
    assert error.value.code == _abi.KV_PHYSICAL_PAGES_EXHAUSTED
    assert np.all(table == UNASSIGNED) and allocator.snapshot()["free_pages"] == 2
    with pytest.raises(KvAllocationError) as error:
        allocator.grow_sequence(32, 16, table)                # shrinking
    assert error.value.code == _abi.KV_SEQUENCE_CAPACITY_EXCEEDED
    with pytest.raises(KvAllocationError) as error:
        allocator.grow_sequence(0, 16 * 5, table)             # beyond the table
    assert error.value.code == _abi.KV_SEQUENCE_CAPACITY_EXCEEDED
    with pytest.raises(KvAllocationError):
        allocator.retain_pages([1])                           # a free page cannot be retained
    with pytest.raises(KvAllocationError):
        allocator.pin_cached_pages([7])                       # out of range
    allocator.grow_sequence(0, 16, table)
    stale = table.copy()
    allocator.release_sequence(16, table)
    allocator.release_sequence(16, stale)                     # double release: the page is not pushed twice
    assert allocator.snapshot()["free_pages"] == 2
    with pytest.raises(Lfm25Error):
        KvPageAllocator(0, 16)


def test_tables_have_stable_disjoint_slot_ranges():
    # src/cache/block_table.rs:46-54
    tables = FixedBlockTables(3, 4)
    tables.slot(1)[2] = 7
    assert tables.slot(1)[2] == 7
    assert np.all(tables.slot(0) == UNASSIGNED)
    assert tables.as_array().size == 12 and tables.as_array()[1, 2] == 7
    with pytest.raises(Lfm25Error, match="out of range"):
        tables.slot(3)
    with pytest.raises(Lfm25Error):
        FixedBlockTables(0, 4)


def test_allocator_fills_block_tables_for_a_batch():
    """The pairing the model cache uses (src/model/lfm2_base.rs:338-380): grow each sequence by one token per step
    and derive the physical slot from its table row."""
    allocator = KvPageAllocator(64, 16)
    tables = FixedBlockTables(4, 8)
    lengths = [0, 0, 0, 0]
    for step in range(40):
        for slot in range(4):
            allocator.grow_sequence(lengths[slot], lengths[slot] + 1, tables.slot(slot))
            lengths[slot] += 1
    table = tables.as_array()
    assert np.all(table[:, :3] != UNASSIGNED) and np.all(table[:, 3:] == UNASSIGNED)
    assert len(set(table[:, :3].reshape(-1).tolist())) == 12   # no page is shared
    assert allocator.snapshot()["allocated_pages"] == 12


def test_schedule_decode_orders_by_deadline():
    # src/scheduler/planner.rs:80-113: every decoding slot, earliest next-token deadline first
    phases = [_abi.PHASE_DECODING, _abi.PHASE_FREE, _abi.PHASE_DECODING, _abi.PHASE_QUEUED_PREFILL,
              _abi.PHASE_DECODING, _abi.PHASE_DECODING]
    deadlines = [900, 0, 300, 100, 50, 300]
    contexts = [10, 999, 4000, 9999, 7, 12]
    slots, maximum = schedule_decode(phases, deadlines, contexts, now_us=100)
    assert slots.tolist() == [4, 2, 5, 0]                     # slot 4 is already late (slack saturates at 0)
    assert maximum == 4000                                    # only decoding slots count
    slots, maximum = schedule_decode([_abi.PHASE_FREE] * 3, [0] * 3, [5] * 3, now_us=0)
    assert slots.size == 0 and maximum == 1


def test_dispatcher_balances_and_survives_a_replica_failure():
    dispatcher = Dispatcher(4)
    placed = [dispatcher.assign(100) for _ in range(8)]
    assert sorted(placed) == [0, 0, 1, 1, 2, 2, 3, 3]         # least loaded, ties to the lowest index
    assert [dispatcher.load(r) for r in range(4)] == [200] * 4
    # requests sharing a prefix keep going to the replica the prefix hashes to
    home = 1234567 % 4
    assert {dispatcher.assign(50, prefix_hash=1234567) for _ in range(5)} == {home}
    dispatcher.complete(home, 250)
    assert dispatcher.load(home) == 200
    # failure injected on the host: the replica stops receiving work, its prefix traffic falls back to least-loaded
    dispatcher.mark_failed(home)
    after = [dispatcher.assign(10, prefix_hash=1234567) for _ in range(6)]
    assert home not in after and len(set(after)) == 3
    for replica in range(4):
        dispatcher.mark_failed(replica)
    with pytest.raises(Lfm25Error, match="no live replica"):
        dispatcher.assign(1)


def test_dispatcher_bounded_affinity_spills_to_the_idlest_replica():
    """lfm25_dispatcher_assign_bounded: the prefix's home keeps a request while it is at most `slack` tokens busier
    than the idlest replica, then the idlest one takes it; requests without a prefix go to the idlest replica."""
    dispatcher = Dispatcher(4)
    home = 1234567 % 4
    placed = [dispatcher.assign(100, prefix_hash=1234567, slack_tokens=250) for _ in range(3)]
    assert placed == [home] * 3 and dispatcher.load(home) == 300
    spilled = dispatcher.assign(100, prefix_hash=1234567, slack_tokens=250)
    assert spilled != home and dispatcher.load(spilled) == 100
    assert dispatcher.assign(10, slack_tokens=250) not in (home, spilled)
    dispatcher.complete(home, 300)
    assert dispatcher.assign(100, prefix_hash=1234567, slack_tokens=250) == home
    dispatcher.mark_failed(home)
    assert dispatcher.assign(100, prefix_hash=1234567, slack_tokens=250) != home


def test_pages_short_reports_a_shortage_before_any_row_changes():
    """A pool too small for a whole step: lfm25_kv_allocator_pages_short names the shortage while the block tables
    and the pool are untouched; growing the sequences one by one instead would have changed the first rows before
    failing on a later one.  (The serving engine asks this before it grows the sequences of a step.)"""
    allocator = KvPageAllocator(6, 16)
    tables = FixedBlockTables(3, 4)
    current, target = [0, 0, 0], [33, 33, 33]                # 3 pages each: 9 > 6
    assert allocator.pages_short(current, target) == 3
    assert allocator.snapshot()["free_pages"] == 6
    assert (tables.as_array() == 0xFFFFFFFF).all()
    assert allocator.pages_short(current[:2], target[:2]) == 0
    assert allocator.pages_short([16], [17]) == 0 and allocator.pages_short([16], [16]) == 0
    with pytest.raises(KvAllocationError):
        allocator.pages_short([32], [16])                    # a target below the current length
    # one by one: the first two rows grow, the third fails -- the state the engine's pre-check avoids
    assert allocator.grow_sequence(0, 33, tables.slot(0)) == 3
    assert allocator.grow_sequence(0, 33, tables.slot(1)) == 3
    with pytest.raises(KvAllocationError):
        allocator.grow_sequence(0, 33, tables.slot(2))
    assert allocator.pages_short([33, 33, 0], [33, 34, 16]) == 1

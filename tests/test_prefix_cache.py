"""The radix prefix index (host-only, src/cache/radix.rs) restated from the reference's own tests
(src/cache/radix.rs:289-350) plus the allocator hand-over a serving loop performs; the checkpoint pool's device
copies are in the GPU part."""
import numpy as np
import pytest

from lfm25_inference_b200 import cache
from lfm25_inference_b200._abi import Lfm25Error


def tokens(pages):
    return np.arange(pages * 16, dtype=np.uint32)


def test_longest_match_stops_at_deepest_checkpoint():
    # src/cache/radix.rs:297-323
    radix = cache.PageRadixCache(16, 16)
    sequence = tokens(4)
    assert radix.can_publish(sequence, 32)
    assert list(radix.insert_checkpoint(sequence, 32, [4, 5], 7)) == [4, 5]
    assert radix.can_publish(sequence, 64)
    assert list(radix.insert_checkpoint(sequence, 64, [99, 98, 6, 7], 8)) == [6, 7]
    matched, slot, pages = radix.longest_checkpoint(sequence, 63)
    assert (matched, slot, list(pages)) == (32, 7, [4, 5])
    matched, slot, pages = radix.longest_checkpoint(sequence, 64)
    assert (matched, slot, list(pages)) == (64, 8, [4, 5, 6, 7])
    radix.close()


def test_refresh_probe_does_not_change_admission_statistics():
    # src/cache/radix.rs:325-337
    radix = cache.PageRadixCache(16, 16)
    sequence = tokens(2)
    radix.insert_checkpoint(sequence, 32, [1, 2], 3)
    assert radix.probe_checkpoint(sequence, 32) is not None
    snapshot = radix.snapshot()
    assert (snapshot["hits"], snapshot["misses"], snapshot["matched_tokens"]) == (0, 0, 0)
    radix.close()


def test_page_budget_counts_only_new_radix_nodes():
    # src/cache/radix.rs:339-349
    radix = cache.PageRadixCache(16, 3)
    sequence = tokens(4)
    radix.insert_checkpoint(sequence, 32, [1, 2], 1)
    assert radix.can_publish(sequence, 48)
    radix.insert_checkpoint(sequence, 48, [9, 9, 3], 2)
    assert not radix.can_publish(sequence, 64)
    assert radix.snapshot()["cached_pages"] == 3
    radix.close()


def test_statistics_misses_and_branching_prefixes():
    radix = cache.PageRadixCache(16, 64)
    shared = tokens(2)
    first = np.concatenate([shared, np.full(16, 7, dtype=np.uint32)])
    second = np.concatenate([shared, np.full(16, 9, dtype=np.uint32)])
    assert radix.longest_checkpoint(first, 48) is None                 # empty index: a miss
    assert radix.longest_checkpoint(first[:15], 15) is None            # shorter than a page: a miss
    radix.insert_checkpoint(first, 48, [10, 11, 12], 0)
    # a node without a checkpoint on the path does not count as a hit
    assert radix.longest_checkpoint(second, 48) is None
    # the sibling branch reuses the two shared pages: only its own third page is new
    assert list(radix.insert_checkpoint(second, 48, [10, 11, 20], 1)) == [20]
    matched, slot, pages = radix.longest_checkpoint(second, 1000)
    assert (matched, slot, list(pages)) == (48, 1, [10, 11, 20])
    snapshot = radix.snapshot()
    assert snapshot == {"nodes": 5, "cached_pages": 4, "checkpoints": 2, "hits": 1, "misses": 3,
                        "matched_tokens": 48}
    radix.close()


def test_insert_errors():
    radix = cache.PageRadixCache(16, 4)
    sequence = tokens(3)
    with pytest.raises(Lfm25Error, match="cannot be empty"):
        radix.insert_checkpoint(sequence, 0, [], 0)
    with pytest.raises(Lfm25Error, match="exceeds token input"):
        radix.insert_checkpoint(sequence, 64, [1, 2, 3, 4], 0)
    with pytest.raises(Lfm25Error, match="page aligned"):
        radix.insert_checkpoint(sequence, 20, [1], 0)
    with pytest.raises(Lfm25Error, match="page count mismatch"):
        radix.insert_checkpoint(sequence, 32, [1], 0)
    radix.insert_checkpoint(sequence, 32, [1, 2], 0)
    with pytest.raises(Lfm25Error, match="cannot be published"):
        radix.insert_checkpoint(sequence, 32, [1, 2], 1)               # already checkpointed
    with pytest.raises(Lfm25Error, match="positive page budget"):
        cache.PageRadixCache(16, 0)
    radix.close()


def test_published_pages_survive_their_sequence_in_the_allocator():
    """The hand-over of src/engine/serving/radix_owner.rs:464-547: pages indexed by the radix tree are pinned, so
    releasing the sequence that produced them returns only its unshared pages; a later request retains the cached
    pages instead of allocating new ones."""
    allocator = cache.KvPageAllocator(8)
    tables = cache.FixedBlockTables(2, 4)
    radix = cache.PageRadixCache(16, 8)
    prompt = tokens(3)
    allocator.try_reserve_tokens(48)
    allocator.grow_sequence(0, 40, tables.slot(0))                    # three pages: 0, 1, 2
    owned = tables.slot(0)[:3].copy()
    fresh = radix.insert_checkpoint(prompt, 32, owned[:2], 0)
    allocator.pin_cached_pages(fresh)
    allocator.release_sequence(40, tables.slot(0))
    assert allocator.snapshot()["free_pages"] == 6                    # the two cached pages stay out of the pool
    matched, _, pages = radix.longest_checkpoint(prompt, 47)
    assert matched == 32 and list(pages) == list(owned[:2])
    allocator.retain_pages(pages)
    tables.slot(1)[:2] = pages
    allocator.try_reserve_tokens(48)
    allocator.grow_sequence(32, 48, tables.slot(1))
    assert tables.slot(1)[2] not in pages
    radix.close()

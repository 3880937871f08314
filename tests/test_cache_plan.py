"""The cache's bookkeeping and the step plan (no GPU): no slot or page lost, held twice
or freed twice; groups with storage of their own; rings; fixed-size state."""
import random

import pytest
import torch

from kidi_b200 import ErrorCode, KidiError, StepBatch
from kidi_b200.cache.allocator import IdAllocator
from kidi_b200.cache.sequence_cache import KVRequest, SequenceCache, StateRequest
from kidi_b200.engine.plan import build_plan

CPU = torch.device("cpu")


def make_cache(max_tokens=1024, requests=None, max_positions=512, **options):
    requests = requests if requests is not None else [[KVRequest(2, 16)], [KVRequest(2, 16, 100)], [KVRequest(2, 16)]]
    return SequenceCache(requests, max_tokens=max_tokens, max_positions=max_positions, dtype=torch.float32,
                         device=CPU, **options)


def test_allocator_refuses_double_free_and_exhaustion():
    pool = IdAllocator(3, "slot")
    held = [pool.acquire() for _ in range(3)]
    assert sorted(held) == [0, 1, 2]
    with pytest.raises(KidiError):
        pool.acquire()
    pool.release(held[1])
    with pytest.raises(KidiError):
        pool.release(held[1])            # freed twice
    with pytest.raises(KidiError):
        pool.release(7)                  # never existed
    assert pool.acquire() == held[1]     # a freed slot is used again at once
    pool.check()


def test_groups_have_storage_of_their_own():
    cache = make_cache()
    assert len(cache.kv_groups) == 2     # full history (two layers) and a window of 100 (one layer)
    full, ring = cache.kv_groups
    assert full.keys.shape == (2, 16, 2, 64, 16) and full.ring_pages == 0
    assert ring.keys.shape[0] == 1 and ring.ring_pages == 2 and ring.pages_per_sequence == 2
    assert cache.views(0)[0].group is full and cache.views(2)[0].group is full
    assert cache.views(0)[0].index == 0 and cache.views(2)[0].index == 1
    assert cache.views(1)[0].group is ring
    assert cache.bytes() == 2 * full.keys.numel() * 4 + 2 * ring.keys.numel() * 4


def test_pages_follow_lengths_and_come_back():
    cache = make_cache(max_tokens=640)
    a, b = cache.acquire(), cache.acquire()
    cache.reserve([(a, 65), (b, 300)])
    cache.commit([(a, 65), (b, 300)])
    full, ring = cache.kv_groups
    assert len(full.pages[a]) == 2 and len(full.pages[b]) == 5
    assert len(ring.pages[a]) == 2 and len(ring.pages[b]) == 2   # a ring holds ceil(100/64) pages at most
    assert (full.table_host[b, :5] == full.pages[b]).all()
    cache.check()
    assert cache.held_tokens() == 128 + 320
    with pytest.raises(KidiError) as caught:                      # four more pages are not there (three are)
        cache.reserve([(a, 65 + 4 * 64)])
    assert caught.value.code == ErrorCode.RUNTIME and "cache is full" in caught.value.message
    assert len(full.pages[a]) == 2                                # all or nothing
    cache.release(b)
    cache.reserve([(a, 400)])
    cache.check()
    with pytest.raises(KidiError):
        cache.release(b)                                          # released twice
    with pytest.raises(KidiError):
        cache.reserve([(b, 10)])                                  # not held
    with pytest.raises(KidiError):
        cache.reserve([(a, 513)])                                 # beyond the positional capacity
    cache.release(a)
    assert not cache.slots.held and full.pool.free_count == full.n_pages and ring.pool.free_count == ring.n_pages


def test_random_traffic_loses_nothing():
    generator = random.Random(0)
    cache = make_cache(max_tokens=2048)
    live = {}
    for _ in range(600):
        action = generator.random()
        if action < 0.3 and cache.slots.free_count:
            live[cache.acquire()] = 0
        elif action < 0.75 and live:
            slot = generator.choice(list(live))
            target = min(512, live[slot] + generator.randint(1, 130))
            if cache.can_hold([(slot, target)]):
                cache.reserve([(slot, target)])
                cache.commit([(slot, target)])
                live[slot] = target
        elif live:
            slot = generator.choice(list(live))
            cache.release(slot)
            del live[slot]
        cache.check()
        assert cache.held_tokens() <= cache.max_tokens
    for slot in list(live):
        cache.release(slot)
    cache.check()
    assert all(group.pool.free_count == group.n_pages for group in cache.kv_groups)


def test_fixed_size_state_is_zeroed_when_a_slot_is_handed_out():
    cache = make_cache(requests=[[KVRequest(1, 16), StateRequest((3, 4))], [StateRequest((3, 4))], []])
    # 16 slots and, as the last row, the padding slot's (what padding sequences of a captured step carry).
    assert len(cache.state_groups) == 1 and cache.state_groups[0].storage.shape == (2, 17, 3, 4)
    assert cache.padding_slot == 16 and cache.kv_groups[0].table.shape[0] == 17
    slot = cache.acquire()
    kv_view, state = cache.views(0)
    assert state.shape == (17, 3, 4) and cache.views(2) == []
    with pytest.raises(KidiError):
        cache.release(cache.padding_slot)          # never handed out, so never given back
    state[slot].fill_(5.0)
    cache.views(1)[0][slot].fill_(7.0)
    cache.release(slot)
    again = cache.acquire()
    assert again == slot and float(state[slot].abs().sum()) == 0.0 and float(cache.views(1)[0][slot].abs().sum()) == 0.0


def test_an_entry_can_read_an_earlier_entry_s_cache():
    cache = make_cache(requests=[[KVRequest(2, 16)], [KVRequest(2, 16)], [KVRequest(2, 16)]], cache_from=[None, 0, None])
    assert len(cache.kv_groups) == 1 and cache.kv_groups[0].keys.shape[0] == 2   # entry 1 owns no storage
    assert cache.views(1)[0] is cache.views(0)[0]
    assert cache.views(2)[0].index == 1
    with pytest.raises(KidiError):
        SequenceCache([[KVRequest(2, 16)], [KVRequest(2, 16)]], max_tokens=64, max_positions=64, dtype=torch.float32,
                      device=CPU, cache_from=[1, None]).views(0)


def test_rewind():
    cache = make_cache(requests=[[KVRequest(2, 16)]])
    slot = cache.acquire()
    cache.reserve([(slot, 200)])
    cache.commit([(slot, 200)])
    cache.rewind(slot, 70)
    assert cache.length(slot) == 70 and len(cache.kv_groups[0].pages[slot]) == 2
    cache.check()
    with pytest.raises(KidiError):
        cache.rewind(slot, 71)


def test_rewind_with_fixed_size_state_takes_a_snapshot():
    cache = make_cache(requests=[[KVRequest(1, 16), StateRequest((2, 3))], [StateRequest((2, 3))]])
    slot, other = cache.acquire(), cache.acquire()
    state = [cache.views(0)[1], cache.views(1)[0]]
    cache.reserve([(slot, 100)])
    cache.commit([(slot, 100)])
    state[0][slot].fill_(1.0)
    state[1][slot].fill_(2.0)
    state[0][other].fill_(9.0)
    saved = cache.snapshot_state(slot)                      # the state after 100 tokens
    cache.reserve([(slot, 180)])
    cache.commit([(slot, 180)])
    state[0][slot].fill_(3.0)
    state[1][slot].fill_(4.0)
    with pytest.raises(KidiError):
        cache.rewind(slot, 100)                             # state cannot be computed backwards
    with pytest.raises(KidiError):
        cache.rewind(slot, 90, state=saved)                 # the snapshot is of another length
    with pytest.raises(KidiError):
        cache.rewind(other, 0, state=saved)                 # and of another slot
    cache.rewind(slot, 100, state=saved)
    assert cache.length(slot) == 100 and len(cache.kv_groups[0].pages[slot]) == 2
    assert float(state[0][slot].mean()) == 1.0 and float(state[1][slot].mean()) == 2.0
    assert float(state[0][other].mean()) == 9.0             # nobody else's state moved
    cache.check()


def test_the_budget_counts_whole_pages():
    cache = make_cache(max_tokens=130, requests=[[KVRequest(1, 16)]])
    assert cache.max_tokens == 192 and cache.n_slots == 3
    slots = [cache.acquire() for _ in range(3)]
    cache.reserve([(slot, 1) for slot in slots])          # three sequences of one token hold three pages
    with pytest.raises(KidiError):
        cache.reserve([(slots[0], 65)])


# ------------------------------------------------------------------------ plan
def test_plan_tables():
    batch = StepBatch(slots=[4, 2, 9], tokens=[[5, 6, 7], [8], [1, 2]], want=[[0, 2], [], [1]])
    plan = build_plan(batch, starts=[10, 0, 63], vocab_size=20)
    assert plan.n_rows == 6 and plan.n_seqs == 3 and plan.n_want == 3
    assert plan.tokens.tolist() == [5, 6, 7, 8, 1, 2]
    assert plan.row_seq.tolist() == [0, 0, 0, 1, 2, 2]
    assert plan.row_pos.tolist() == [10, 11, 12, 0, 63, 64]
    assert plan.seq_slot.tolist() == [4, 2, 9] and plan.seq_row0.tolist() == [0, 3, 4]
    assert plan.want_rows.tolist() == [0, 2, 5]
    assert plan.max_new == 3 and plan.max_total == 65 and not plan.is_decode
    packed, offsets = plan.packed(), plan.offsets()
    for name, (begin, size) in offsets.items():
        assert begin % 4 == 0 and (packed[begin:begin + size] == getattr(plan, name)).all()
    last = build_plan(StepBatch([0, 1], [[3], [4]]), [5, 9], 20)
    assert last.is_decode and last.want_rows.tolist() == [0, 1]


@pytest.mark.parametrize("batch,starts", [
    (StepBatch([], []), []),
    (StepBatch([1, 1], [[1], [2]]), [0, 0]),                 # a slot twice
    (StepBatch([1], [[]]), [0]),                             # no token
    (StepBatch([1], [[20]]), [0]),                           # token outside the vocabulary
    (StepBatch([1], [[-1]]), [0]),
    (StepBatch([1], [[1, 2]], [[2]]), [0]),                  # wanted place outside the new tokens
    (StepBatch([1, 2], [[1], [2]], [[0]]), [0, 0]),          # want for one sequence only
])
def test_plan_validation(batch, starts):
    with pytest.raises(KidiError) as caught:
        build_plan(batch, starts, vocab_size=20)
    assert caught.value.code == ErrorCode.INVALID_ARGUMENT


def test_values_of_a_page_are_cleared_when_it_is_handed_out_again():
    """What a sequence left in its pages must not reach the next one that gets them: rows past
    the next sequence's end are read with their page. Fresh pages are zero from the start and
    are not cleared again."""
    import torch
    from kidi_b200.cache.sequence_cache import KVRequest, SequenceCache
    cache = SequenceCache([[KVRequest(2, 16)], [KVRequest(2, 16)]], max_tokens=256, max_positions=256,
                          dtype=torch.float32, device=torch.device("cpu"), page_size=64)
    group = cache.kv_groups[0]
    first = cache.acquire()
    cache.reserve([(first, 130)])                       # three pages
    pages = list(group.pages[first])
    assert len(pages) == 3 and float(group.values.abs().sum()) == 0.0
    group.values[:, pages] = float("nan")
    group.keys[:, pages] = float("nan")
    cache.commit([(first, 130)])
    cache.release(first)
    second = cache.acquire()
    cache.reserve([(second, 70)])                       # two of the used pages come back
    again = group.pages[second]
    assert set(again) <= set(pages)
    assert torch.isfinite(group.values[:, again]).all() and float(group.values[:, again].abs().sum()) == 0.0
    left = [page for page in pages if page not in again]
    assert torch.isnan(group.values[:, left]).all()     # a page nobody holds is not touched
    cache.reserve([(second, 256)])                      # the third used page and a fresh one
    assert torch.isfinite(group.values[:, group.pages[second]]).all()
    cache.check()

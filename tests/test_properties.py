"""Property-based checks (hypothesis) of the pure host-side pieces: assignment splitters and the cache directory."""
from hypothesis import given, settings
from hypothesis import strategies as st

from dlslime_b200._slime_c import Assignment, cache, nsplit_assign_by_step, split_assign_by_max_length, split_assign_by_step

assignments = st.lists(
    st.builds(Assignment, st.integers(0, 7), st.integers(0, 7), st.integers(0, 1 << 40), st.integers(0, 1 << 40), st.integers(0, 1 << 22)),
    min_size=0, max_size=12)


@settings(max_examples=150, deadline=None)
@given(assignments, st.integers(1, 1 << 21))
def test_split_by_max_length_covers_every_byte_once_in_order(batch, max_len):
    out = split_assign_by_max_length(batch, max_len)
    assert all(x.length <= max_len or x.length == 0 for x in out)
    it = iter(out)
    for a in batch:  # pieces of one assignment are contiguous on both sides, in order, and add up
        if a.length <= max_len:
            assert next(it).to_tuple() == a.to_tuple()
            continue
        covered = 0
        while covered < a.length:
            p = next(it)
            assert (p.mr_key, p.remote_mr_key) == (a.mr_key, a.remote_mr_key)
            assert (p.target_offset, p.source_offset) == (a.target_offset + covered, a.source_offset + covered)
            assert 0 < p.length <= max_len
            covered += p.length
        assert covered == a.length
    assert next(it, None) is None


@settings(max_examples=100, deadline=None)
@given(assignments, st.integers(1, 16))
def test_split_by_step_and_nsplit_keep_order_and_group_sizes(batch, k):
    groups = split_assign_by_step(batch, k)
    flat = [x.to_tuple() for g in groups for x in g]
    assert flat == [a.to_tuple() for a in batch]
    assert all(len(g) == k for g in groups[:-1]) and all(0 < len(g) <= k for g in groups)
    parts = nsplit_assign_by_step(batch, k)
    assert [x.to_tuple() for g in parts for x in g] == [a.to_tuple() for a in batch]
    assert len(parts) <= k
    if batch:
        step = -(-len(batch) // k)
        assert all(len(g) == step for g in parts[:-1])


ops = st.lists(st.one_of(
    st.tuples(st.just("store"), st.sampled_from(["a", "b", "c"]), st.lists(st.integers(1, 700 * 1024), min_size=1, max_size=4)),
    st.tuples(st.just("delete"), st.integers(0, 30)),
), min_size=1, max_size=40)


@settings(max_examples=100, deadline=None)
@given(ops)
def test_cache_directory_never_hands_a_slab_out_twice(program):
    slab, total = 128 * 1024, 24
    srv = cache.CacheServer(slab_size=slab, memory_size=total * slab)
    live = {}  # (peer, version) -> slab ids
    last_version = 0
    for op in program:
        if op[0] == "store":
            _, peer, lengths = op
            need = sum(-(-n // slab) for n in lengths)
            free_before = srv.stats().free_slabs
            try:
                m = srv.store_assignments(peer, [Assignment(1, 2, 0, 0, n) for n in lengths])
            except RuntimeError:
                assert need > free_before  # refused only when the pool really is too small ...
                assert srv.stats().free_slabs == free_before  # ... and nothing leaks on refusal
                continue
            assert need <= free_before and len(m.slab_ids) == need
            assert m.version > last_version  # versions only grow
            last_version = m.version
            in_use = {s for ids in live.values() for s in ids}
            assert not in_use & set(m.slab_ids) and len(set(m.slab_ids)) == need
            assert all(0 <= s < total for s in m.slab_ids)
            assert [x.source_offset for x in m.assignments] == [s * slab for s in m.slab_ids]
            assert sum(x.length for x in m.assignments) == sum(lengths) == m.total_bytes()
            live[(peer, m.version)] = list(m.slab_ids)
        else:
            keys = sorted(live)
            if not keys:
                continue
            peer, version = keys[op[1] % len(keys)]
            assert srv.delete_assignments(peer, version) is True
            assert srv.delete_assignments(peer, version) is False
            del live[(peer, version)]
        stt = srv.stats()
        used = sum(len(v) for v in live.values())
        assert (stt.used_slabs, stt.free_slabs) == (used, total - used)
        assert stt.num_assignment_entries == len(live)
    for peer, version in list(live):
        assert srv.delete_assignments(peer, version)
    assert srv.stats().free_slabs == total

"""DLSlimeCache directory semantics (slab math, reuse order, errors), pinned like the reference's
``tests/python/test_cache_v0.py`` pins them."""
import pytest

from dlslime_b200._slime_c import Assignment, cache

K = 1024


def test_defaults():
    s = cache.CacheServer()
    assert (s.slab_size(), s.memory_size(), s.num_slabs()) == (256 * K, 0, 0)


def test_fixed_pool_and_validation():
    s = cache.CacheServer(slab_size=128 * K, memory_size=512 * K)
    st = s.stats()
    assert (st.num_slabs, st.used_slabs, st.free_slabs) == (4, 0, 4)
    with pytest.raises(ValueError, match="multiple of slab_size"):
        cache.CacheServer(slab_size=128 * K, memory_size=300 * K)
    for bad in (128 * K - 1, 1024 ** 3 + 1):
        with pytest.raises(ValueError, match=r"\[128K, 1G\]"):
            cache.CacheServer(slab_size=bad)


def test_full_pool_rejects_then_reuses_last_freed_slab_first():
    s = cache.CacheServer(slab_size=128 * K, memory_size=256 * K)
    m = s.store_assignments("a", [Assignment(1, 2, 0, 0, 256 * K)])
    assert m.slab_ids == [0, 1] and [x.source_offset for x in m.assignments] == [0, 128 * K]
    with pytest.raises(RuntimeError, match="not enough preallocated cache slabs"):
        s.store_assignments("b", [Assignment(1, 2, 0, 0, 1)])
    assert s.delete_assignments("a", m.version) is True and s.stats().free_slabs == 2
    assert s.store_assignments("b", [Assignment(1, 2, 0, 0, 1)]).slab_ids == [1]


def test_store_query_roundtrip_and_miss():
    s = cache.CacheServer()
    m = s.store_assignments("a", [Assignment(11, 22, 0, 1024, 4096), Assignment(11, 22, 4096, 8192, 2048)])
    assert (m.peer_agent_id, m.version, m.total_bytes()) == ("a", 1, 6144)
    got = s.query_assignments("a", 1)
    assert [(x.mr_key, x.remote_mr_key, x.target_offset, x.length) for x in got.assignments] == [(11, 22, 0, 4096), (11, 22, 4096, 2048)]
    assert s.query_assignments("a", 2) is None and s.query_assignments("b", 1) is None


def test_splitting_into_slabs():
    slab = 256 * K
    s = cache.CacheServer(slab_size=slab, memory_size=4 * slab)
    m = s.store_assignments("a", [Assignment(1, 2, 10, 20, 2 * slab + 123)])
    assert m.slab_ids == [0, 1, 2]
    assert [(x.target_offset, x.source_offset, x.length) for x in m.assignments] == [(10, 0, slab), (10 + slab, slab, slab), (10 + 2 * slab, 2 * slab, 123)]


def test_stats_delete_clear_and_empty_peer():
    s = cache.CacheServer(slab_size=128 * K, memory_size=1024 * K)
    m0 = s.store_assignments("a", [Assignment(1, 2, 0, 0, 300 * K)])
    s.store_assignments("a", [Assignment(1, 2, 0, 0, 64 * K)])
    s.store_assignments("b", [Assignment(3, 4, 0, 0, 32 * K)])
    st = s.stats()
    assert (st.num_assignment_peers, st.num_assignment_entries, st.num_assignments, st.assignment_bytes, st.used_slabs, st.free_slabs) == (2, 3, 5, 396 * K, 5, 3)
    assert s.delete_assignments("a", m0.version) and not s.delete_assignments("a", m0.version)
    assert s.stats().used_slabs == 2
    with pytest.raises(ValueError, match="peer_agent_id"):
        s.store_assignments("", [Assignment(1, 2, 0, 0, 64)])
    s.clear()
    assert s.stats().num_assignment_entries == 0
    assert s.store_assignments("a", [Assignment(1, 2, 0, 0, 64)]).version == 1


def test_package_level_names_match_the_reference():
    """``dlslime.cache`` in the reference exports the directory as ``CacheServer`` and a few helpers: the same calls work
    on this package (``dlslime/cache/__init__.py:22-45`` in the reference)."""
    import dlslime_b200.cache as pkg

    d = pkg.CacheServer(slab_size=128 * K, memory_size=512 * K)
    assert isinstance(d, cache.CacheServer) and d.num_slabs() == 4
    assert isinstance(pkg.CacheServer(), cache.CacheServer) and isinstance(pkg.CacheServer(128 * K, 256 * K), cache.CacheServer)
    assert pkg.ccache is cache and pkg.CacheDirectory is cache.CacheServer
    assert pkg.assignment_to_tuple(Assignment(1, 2, 3, 4, 5)) == (1, 2, 3, 4, 5)
    assert pkg.resolve_host_for_registration("10.0.0.1") == "10.0.0.1" and pkg.resolve_host_for_registration("0.0.0.0")

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
    from hypothesis import assume

    assume(sum(a.length for a in batch) // max_len < 5000)  # keep the number of pieces (and the run time) small
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


# ------------------------------------------------------------------------------------------------
# the embedded store against a model: strings, hashes and lists with time-to-live on an injected clock
# ------------------------------------------------------------------------------------------------
KEYS = st.sampled_from(["k1", "k2", "k3"])
VALS = st.sampled_from(["a", "b", "c", "dd"])
kv_ops = st.lists(st.one_of(
    st.tuples(st.just("set"), KEYS, VALS, st.sampled_from([-1, 50, 500])),
    st.tuples(st.just("get"), KEYS),
    st.tuples(st.just("del"), KEYS),
    st.tuples(st.just("hset"), KEYS, VALS, VALS),
    st.tuples(st.just("hget"), KEYS, VALS),
    st.tuples(st.just("hdel"), KEYS, VALS),
    st.tuples(st.just("lpush"), KEYS, VALS),
    st.tuples(st.just("rpush"), KEYS, VALS),
    st.tuples(st.just("lpop"), KEYS),
    st.tuples(st.just("rpop"), KEYS),
    st.tuples(st.just("pexpire"), KEYS, st.sampled_from([10, 100, 1000])),
    st.tuples(st.just("tick"), st.sampled_from([1, 9, 60, 600])),
), min_size=1, max_size=60)


class _Model:
    """What Redis does for this subset: one namespace, typed values, a deadline per key, empty containers vanish."""

    def __init__(self):
        self.now, self.d = 1_000_000, {}

    def _live(self, k):
        e = self.d.get(k)
        if e is not None and e[2] is not None and e[2] <= self.now:
            del self.d[k]
            e = None
        return e

    def typed(self, k, kind, create):
        e = self._live(k)
        if e is None:
            if not create:
                return None
            e = self.d[k] = [kind, {} if kind == "hash" else [] if kind == "list" else "", None]
        if e[0] != kind:
            raise TypeError
        return e

    def drop_if_empty(self, k):
        e = self.d.get(k)
        if e is not None and e[0] in ("hash", "list") and not e[1]:
            del self.d[k]


@settings(max_examples=200, deadline=None)
@given(kv_ops)
def test_kv_store_matches_the_model(program):
    import pytest

    from dlslime_b200 import _slime_c

    kv, m = _slime_c.ctrl.KvStore(), _Model()
    kv.set_clock(lambda: m.now)

    def both(model_fn, real_fn):
        """Runs the model first; a type clash there must be a WRONGTYPE error in the store."""
        try:
            want = model_fn()
        except TypeError:
            with pytest.raises(RuntimeError, match="WRONGTYPE"):
                real_fn()
            return
        assert real_fn() == want

    for op in program:
        name, args = op[0], op[1:]
        if name == "tick":
            m.now += args[0]
        elif name == "set":
            k, v, px = args
            m._live(k)
            m.d[k] = ["string", v, None if px < 0 else m.now + px]  # SET replaces any type and clears the deadline
            assert kv.set(k, v, px=px) is True
        elif name == "get":
            both(lambda: (lambda e: None if e is None else e[1])(m.typed(args[0], "string", False)), lambda: kv.get(args[0]))
        elif name == "del":
            want = 1 if m._live(args[0]) is not None else 0
            m.d.pop(args[0], None)
            assert kv.delete(args[0]) == want
        elif name == "hset":
            k, f, v = args

            def mh():
                e = m.typed(k, "hash", True)
                new = 0 if f in e[1] else 1
                e[1][f] = v
                return new
            both(mh, lambda: kv.hset(k, {f: v}))
        elif name == "hget":
            k, f = args
            both(lambda: (lambda e: None if e is None else e[1].get(f))(m.typed(k, "hash", False)), lambda: kv.hget(k, f))
        elif name == "hdel":
            k, f = args

            def mhd():
                e = m.typed(k, "hash", False)
                n = 0 if e is None or f not in e[1] else 1
                if n:
                    del e[1][f]
                    m.drop_if_empty(k)
                return n
            both(mhd, lambda: kv.hdel(k, f))
        elif name in ("lpush", "rpush"):
            k, v = args

            def mp():
                e = m.typed(k, "list", True)
                e[1].insert(0, v) if name == "lpush" else e[1].append(v)
                return len(e[1])
            both(mp, lambda: getattr(kv, name)(k, v))
        elif name in ("lpop", "rpop"):
            k = args[0]

            def mpop():
                e = m.typed(k, "list", False)
                if e is None:
                    return None
                v = e[1].pop(0) if name == "lpop" else e[1].pop()
                m.drop_if_empty(k)
                return v
            both(mpop, lambda: getattr(kv, name)(k))
        elif name == "pexpire":
            k, ms = args
            e = m._live(k)
            if e is not None:
                e[2] = m.now + ms
            assert kv.pexpire(k, ms) is (e is not None)
        # after every step: same set of live keys, same types, same list contents
        live = {k for k in list(m.d) if m._live(k) is not None}
        assert {k for k in ("k1", "k2", "k3") if kv.exists(k)} == live
        assert kv.dbsize() == len(live)
        for k in live:
            assert kv.type(k) == m.d[k][0]
            if m.d[k][0] == "list":
                assert kv.lrange(k, 0, -1) == m.d[k][1] and kv.llen(k) == len(m.d[k][1])
            ttl = kv.pttl(k)
            assert ttl == (-1 if m.d[k][2] is None else m.d[k][2] - m.now)


stream_ops = st.lists(st.one_of(
    st.tuples(st.just("xadd"), st.sampled_from(["s1", "s2"]), VALS, st.sampled_from([0, 0, 3, 5])),
    st.tuples(st.just("xread"), st.sampled_from(["s1", "s2"]), st.integers(0, 12), st.sampled_from([0, 1, 4])),
    st.tuples(st.just("tick"), st.sampled_from([0, 1, 7])),
    st.tuples(st.just("back"), st.sampled_from([1, 5])),  # the clock steps backwards: ids must still grow
), min_size=1, max_size=50)


@settings(max_examples=150, deadline=None)
@given(stream_ops)
def test_streams_keep_order_trim_and_resume(program):
    """Stream ids grow strictly whatever the clock does; MAXLEN keeps the newest entries; a reader that resumes from the
    last id it saw gets exactly the entries added since (the mailbox handshake depends on this)."""
    from dlslime_b200 import _slime_c

    kv = _slime_c.ctrl.KvStore()
    now = [10_000]
    kv.set_clock(lambda: now[0])
    model = {"s1": [], "s2": []}  # (id tuple, id text, fields)
    key_of = lambda text: tuple(int(x) for x in text.split("-"))
    for op in program:
        if op[0] == "tick":
            now[0] += op[1]
        elif op[0] == "back":
            now[0] -= op[1]
        elif op[0] == "xadd":
            _, k, v, maxlen = op
            text = kv.xadd(k, {"f": v}, maxlen=maxlen)
            ident = key_of(text)
            if model[k]:
                assert ident > model[k][-1][0]
            model[k].append((ident, text, {"f": v}))
            if maxlen:
                model[k] = model[k][-maxlen:]
        else:
            _, k, seen, count = op
            entries = model[k]
            last = entries[min(seen, len(entries)) - 1][1] if entries and seen else "0-0"
            want = [(t, f) for i, t, f in entries if i > key_of(last)]
            if count:
                want = want[:count]
            got = kv.xread({k: last}, count, None)
            assert got == ([(k, want)] if want else [])
        for k, entries in model.items():
            assert kv.xlen(k) == len(entries)
            assert kv.xrange(k, "-", "+") == [(t, f) for _, t, f in entries]


pool_ops = st.lists(st.one_of(
    st.tuples(st.just("reg"), st.sampled_from(["a", "b", None]), st.sampled_from([0x1000, 0x2000, 0x3000]), st.sampled_from([64, 128, 4096])),
    st.tuples(st.just("unreg_name"), st.sampled_from(["a", "b", "auto_0x1000", "auto_0x2000", "auto_0x3000"])),
    st.tuples(st.just("unreg_handle"), st.integers(0, 6)),
), min_size=1, max_size=40)


@settings(max_examples=200, deadline=None)
@given(pool_ops)
def test_memory_pool_handles_are_stable_and_regions_only_grow(program):
    """A name identifies its region (registering it again returns the same handle, a larger length grows the region); a
    second name for a pointer that is registered already becomes an alias of that region; a region that moves under one of
    its names loses the automatic name of its old address; unregistering a name removes the region only with its last name, unregistering the handle removes it with all names; handles of live regions are distinct."""
    from dlslime_b200 import _slime_c

    pool = _slime_c.MemoryPool()
    names, regions = {}, {}  # name -> handle; handle -> [addr, length]
    for op in program:
        if op[0] == "reg":
            _, name, addr, length = op
            key = name or f"auto_{addr:#x}"
            h = pool.register_memory_region(addr, length, name)
            by_ptr = next((hh for hh, r in regions.items() if r[0] == addr), None)
            if key in names and name is not None and by_ptr is not None and by_ptr != names[key]:
                assert h == -1  # the name belongs to another region than the one that starts at this address: refused
                continue
            assert h >= 0
            if name is None and by_ptr is not None:  # no name given: the pointer identifies the region, nothing is added
                assert h == by_ptr
                if regions[h][1] < length:
                    regions[h][1] = length
            elif key in names:  # the name wins: same handle, moved and / or grown
                assert h == names[key]
                if regions[h][0] != addr:  # an automatic name says where the region started: it does not survive a move
                    stale = f"auto_{regions[h][0]:#x}"
                    if stale != key and names.get(stale) == h:
                        del names[stale]
                if regions[h][0] != addr or regions[h][1] < length:
                    regions[h] = [addr, length]
            elif by_ptr is not None:  # a new name for a registered pointer: alias
                assert h == by_ptr
                names[key] = h
                if regions[h][1] < length:
                    regions[h][1] = length
            else:
                assert h not in regions, "a live handle was handed out twice"
                names[key], regions[h] = h, [addr, length]
        else:
            if op[0] == "unreg_name":
                h = names.get(op[1])
                rc = pool.unregister_memory_region(op[1])
                if h is not None and sum(1 for v in names.values() if v == h) > 1:
                    assert rc == 0  # other names remain: only this name goes, the region stays
                    del names[op[1]]
                    h = "kept"
            else:
                h = op[1] if op[1] in regions else None
                rc = pool.unregister_memory_region(op[1])
            assert (rc == 0) == (h is not None)
            if h is not None and h != "kept":
                del regions[h]
                names = {k: v for k, v in names.items() if v != h}
        info = pool.mr_info()
        assert pool.live_count() == len(regions) and set(info) == set(names)
        for k, h in names.items():
            assert (info[k]["handle"], info[k]["addr"], info[k]["length"]) == (h, regions[h][0], regions[h][1])
            assert pool.get_handle(k) == h


# ------------------------------------------------------------------------------------------------
# JSON through the whole control plane: client -> HTTP -> C++ parser -> store -> C++ writer -> HTTP -> client
# ------------------------------------------------------------------------------------------------
json_leaves = st.one_of(
    st.none(), st.booleans(), st.integers(-(2 ** 53), 2 ** 53),
    st.floats(allow_nan=False, allow_infinity=False, width=64),
    st.text(max_size=20),  # any unicode, including control characters, quotes, backslashes and astral code points
)
json_values = st.recursive(json_leaves, lambda inner: st.one_of(st.lists(inner, max_size=4), st.dictionaries(st.text(max_size=8), inner, max_size=4)),
                           max_leaves=12)


def test_json_survives_the_control_plane_round_trip():
    from hypothesis import HealthCheck

    from dlslime_b200.nanoctrl import NanoCtrlClient, start_local_nanoctrl

    ctrl = start_local_nanoctrl()
    try:
        client = NanoCtrlClient(ctrl.url, scope="json-fuzz")
        counter = [0]

        @settings(max_examples=150, deadline=None, suppress_health_check=[HealthCheck.too_slow])
        @given(st.dictionaries(st.text(max_size=8), json_values, max_size=4))
        def run(metadata):
            counter[0] += 1
            eid = f"fuzz:{counter[0]}"
            assert client.register(eid, "fuzz", endpoint={"host": "h", "port": 1}, metadata=metadata)["status"] == "ok"
            info = client.get_entity_info(eid)
            assert info is not None and info["metadata"] == metadata and info["endpoint"] == {"host": "h", "port": 1}
            client.unregister(eid)

        run()
    finally:
        ctrl.stop()


def test_resp_front_end_carries_any_text_and_reports_wrong_types():
    """Keys, fields and values with any characters (CR LF, quotes, empty, astral) survive the RESP2 front end, and a
    command against a key of another kind comes back as a WRONGTYPE error, as a Redis server answers."""
    import pytest
    from hypothesis import HealthCheck

    from dlslime_b200.nanoctrl import RespClient, RespError, start_local_nanoctrl

    ctrl = start_local_nanoctrl()
    try:
        r = RespClient("127.0.0.1", ctrl.resp_port, timeout=5.0)
        assert r.ping()
        texts = st.text(max_size=30)

        @settings(max_examples=120, deadline=None, suppress_health_check=[HealthCheck.too_slow])
        @given(texts.filter(lambda s: s != ""), texts, st.dictionaries(texts, texts, min_size=1, max_size=4), st.lists(texts, min_size=1, max_size=5))
        def run(key, value, mapping, items):
            r.flushall()
            assert r.set("s:" + key, value) and r.get("s:" + key) == value
            r.hset("h:" + key, mapping=mapping)
            assert r.hgetall("h:" + key) == mapping
            for f, v in mapping.items():
                assert r.hget("h:" + key, f) == v
            assert r.rpush("l:" + key, *items) == len(items)
            assert [r.lpop("l:" + key) for _ in items] == items and r.llen("l:" + key) == 0
            assert sorted(r.keys("*")) == sorted(["s:" + key, "h:" + key])
            with pytest.raises(RespError, match="WRONGTYPE"):
                r.hget("s:" + key, "f")
            with pytest.raises(RespError, match="WRONGTYPE"):
                r.lpush("h:" + key, "x")
            assert r.ping()  # the connection is still in step after the errors

        run()
        r.close()
    finally:
        ctrl.stop()


# ------------------------------------------------------------------------------------------------
# one-sided transfers over the TCP endpoint against two byte arrays
# ------------------------------------------------------------------------------------------------
REGION = 1 << 16
piece = st.tuples(st.integers(0, REGION), st.integers(0, REGION), st.sampled_from([0, 1, 7, 64, 1000, 4096, 30000, REGION]))
transfer_ops = st.lists(st.tuples(st.sampled_from(["read", "write"]), st.lists(piece, min_size=1, max_size=6)), min_size=1, max_size=8)


def test_tcp_transfers_match_a_model_and_bad_batches_change_nothing():
    """Random batches of (remote offset, local offset, length), zero lengths and whole-region pieces included: the two
    regions end up as the same sequence of copies applied to two byte arrays; a batch with a piece that leaves its
    region fails as a whole and moves nothing."""
    import ctypes
    import random

    import pytest
    from hypothesis import HealthCheck

    from dlslime_b200 import _slime_c as c

    a, b = c.TcpEndpoint(), c.TcpEndpoint()
    ba, bb = ctypes.create_string_buffer(REGION), ctypes.create_string_buffer(REGION)
    a.register_memory_region("buf", ctypes.addressof(ba), 0, REGION)
    b.register_memory_region("buf", ctypes.addressof(bb), 0, REGION)
    a.connect(b.endpoint_info())
    b.connect(a.endpoint_info())
    try:
        @settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
        @given(transfer_ops)
        def run(program):
            rnd = random.Random(3)  # the same bytes for every example, so that a failure replays
            local, remote = bytearray(rnd.randbytes(REGION)), bytearray(rnd.randbytes(REGION))
            ba.raw, bb.raw = bytes(local), bytes(remote)
            for op, pieces in program:
                ok = all(ro + n <= REGION and lo + n <= REGION for ro, lo, n in pieces)
                fut = getattr(a, op)([(0, 0, ro, lo, n) for ro, lo, n in pieces])
                if not ok:
                    with pytest.raises(RuntimeError):
                        fut.wait(10_000)
                    assert ba.raw == bytes(local) and bb.raw == bytes(remote), "a refused batch moved bytes"
                    continue
                assert fut.wait(10_000) == 0
                for ro, lo, n in pieces:  # pieces of one batch are applied in order
                    if op == "write":
                        remote[ro:ro + n] = local[lo:lo + n]
                    else:
                        local[lo:lo + n] = remote[ro:ro + n]
                assert ba.raw == bytes(local) and bb.raw == bytes(remote)

        run()
    finally:
        a.shutdown()
        b.shutdown()

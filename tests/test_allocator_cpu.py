"""Caching-allocator logic on the host-memory backend (no GPU): rounding, small/large pools,
split + merge, stream affinity, record_stream, private pools, memory fraction and OOM retry,
statistics and the event trace.  Mirrors the behaviours the reference checks in
tests/unittest/core/test_memory.py:28-398 and test_mempool.py:16-123."""
import pytest


@pytest.fixture
def h(bw):
    return bw._C._HostCacheHarness()


MiB = 1 << 20


def test_rounding_and_small_pool(h):
    p = h.alloc(1)
    s = h.stats()
    assert s["allocated_bytes"]["all"]["current"] == 512
    assert s["reserved_bytes"]["small_pool"]["current"] == 2 * MiB
    assert s["segment"]["all"]["current"] == 1
    q = h.alloc(1000)  # rounds to 1024, same 2 MiB segment
    s = h.stats()
    assert s["allocated_bytes"]["all"]["current"] == 512 + 1024
    assert s["segment"]["all"]["current"] == 1
    h.free(p); h.free(q)
    s = h.stats()
    assert s["allocated_bytes"]["all"]["current"] == 0
    assert s["reserved_bytes"]["all"]["current"] == 2 * MiB  # cached
    h.empty_cache()
    assert h.stats()["reserved_bytes"]["all"]["current"] == 0


def test_large_pool_segment_sizes(h):
    a = h.alloc(3 * MiB)          # < 10 MiB -> 20 MiB segment
    assert h.stats()["reserved_bytes"]["large_pool"]["current"] == 20 * MiB
    b = h.alloc(33 * MiB + 5)     # >= 10 MiB -> rounded to 2 MiB
    assert h.stats()["reserved_bytes"]["large_pool"]["current"] == 20 * MiB + 34 * MiB
    h.free(a); h.free(b)


def test_split_merge_and_reuse(h):
    a = h.alloc(4 * MiB)
    b = h.alloc(4 * MiB)
    c = h.alloc(4 * MiB)
    assert h.stats()["segment"]["all"]["current"] == 1  # all carved from one 20 MiB segment
    assert b == a + 4 * MiB and c == b + 4 * MiB
    h.free(b)
    d = h.alloc(4 * MiB)
    assert d == b  # best fit reuses the hole
    h.free(a); h.free(d); h.free(c)
    snap = h.snapshot()
    assert len(snap) == 1 and snap[0]["blocks"] == [(20 * MiB, False)]  # fully merged
    s = h.stats()
    assert s["inactive_split_bytes"]["all"]["current"] == 0


def test_stream_affinity(h):
    a = h.alloc(4 * MiB, stream=0x10)
    h.free(a)
    b = h.alloc(4 * MiB, stream=0x20)  # a block cached for another stream is not handed out
    assert h.stats()["segment"]["all"]["current"] == 2
    c = h.alloc(4 * MiB, stream=0x10)
    assert c == a
    h.free(b); h.free(c)


def test_private_pool_isolation(bw, h):
    pool = tuple(bw._C._new_mempool_id(True))
    h.begin_pool(pool, 0x30)
    a = h.alloc(4 * MiB, stream=0x30)   # goes to the private pool
    b = h.alloc(4 * MiB, stream=0x40)   # other stream: general pool
    h.end_pool(pool)
    snap = {s["address"]: s for s in h.snapshot()}
    pools = sorted(tuple(s["pool_id"]) for s in snap.values())
    assert (0, 0) in pools and pool in pools
    h.free(a)
    c = h.alloc(4 * MiB, stream=0x30)   # capture over: must not take the private block
    assert c != a
    h.free(b); h.free(c)
    h.release_pool(pool)
    assert all(tuple(s["pool_id"]) != pool for s in h.snapshot())


def test_memory_fraction_and_oom(h):
    h.set_memory_fraction(0.001)  # of the 16 GiB fake device: ~16 MiB
    a = h.alloc(1 * MiB)
    with pytest.raises(Exception, match="out of memory"):
        h.alloc(64 * MiB)
    assert h.stats()["num_ooms"] == 1
    h.free(a)


def test_oom_retry_frees_cache(h):
    h.set_memory_fraction(0.004)  # ~65 MiB allowed
    a = h.alloc(40 * MiB)
    h.free(a)                      # cached 40 MiB segment
    b = h.alloc(50 * MiB)          # does not fit beside the cache: allocator must release and retry
    s = h.stats()
    assert s["num_alloc_retries"] >= 1 and s["num_ooms"] == 0
    assert s["reserved_bytes"]["all"]["current"] == 50 * MiB
    h.free(b)


def test_trace_records_events(h):
    h.record_history(True, 100)
    a = h.alloc(1 * MiB)
    h.free(a)
    actions = [t[0] for t in h.trace()]
    assert 3 in actions and 0 in actions and 1 in actions and 2 in actions  # segment_alloc, alloc, free_req, free_done


def test_stats_peaks(h):
    a = h.alloc(8 * MiB)
    b = h.alloc(8 * MiB)
    h.free(a); h.free(b)
    s = h.stats()["allocated_bytes"]["all"]
    assert s["peak"] == 16 * MiB and s["current"] == 0 and s["allocated"] == 16 * MiB and s["freed"] == 16 * MiB


# ---------------------------------------------------------------- expandable segments
@pytest.fixture
def xh(bw):
    """Harness with expandable segments on (host backend: mmap/mprotect stand in for the driver's VMM)."""
    bw._C._set_allocator_settings("expandable_segments:True")
    try:
        yield bw._C._HostCacheHarness()
    finally:
        bw._C._set_allocator_settings("expandable_segments:False")


def test_expandable_segment_grows_in_place(xh):
    a = xh.alloc(30 * MiB)            # two 20 MiB units mapped at the start of the reserved range
    s = xh.stats()
    assert s["reserved_bytes"]["large_pool"]["current"] == 40 * MiB
    assert s["segment"]["all"]["current"] == 1
    b = xh.alloc(50 * MiB)            # 10 MiB free tail + 40 MiB newly mapped, contiguous with `a`
    assert b == a + 30 * MiB
    s = xh.stats()
    assert s["reserved_bytes"]["large_pool"]["current"] == 80 * MiB
    assert s["segment"]["all"]["current"] == 1   # still one segment: no second, differently sized one
    snap = xh.snapshot()
    assert len(snap) == 1 and snap[0]["is_expandable"] and snap[0]["total_size"] == 80 * MiB
    assert xh.write_read(b, 50 * MiB, 7) == 7    # the mapped range is real memory
    xh.free(a); xh.free(b)
    assert xh.stats()["reserved_bytes"]["all"]["current"] == 80 * MiB  # cached
    xh.empty_cache()
    s = xh.stats()
    assert s["reserved_bytes"]["all"]["current"] == 0 and s["segment"]["all"]["current"] == 0
    assert xh.snapshot() == []


def test_expandable_unmaps_only_whole_units_and_refills_holes(xh):
    a = xh.alloc(20 * MiB)
    b = xh.alloc(60 * MiB)
    c = xh.alloc(20 * MiB)
    assert b == a + 20 * MiB and c == b + 60 * MiB
    xh.free(b)
    xh.empty_cache()                  # the three units under `b` go back; `a` and `c` stay mapped
    s = xh.stats()
    assert s["reserved_bytes"]["all"]["current"] == 40 * MiB
    snap = xh.snapshot()
    assert [x["total_size"] for x in snap] == [20 * MiB, 20 * MiB]   # two mapped runs around the hole
    d = xh.alloc(40 * MiB)            # fits the hole: mapped again at the old address
    assert d == b
    assert xh.stats()["reserved_bytes"]["all"]["current"] == 80 * MiB
    e = xh.alloc(30 * MiB)            # hole has 20 MiB left: too small, grows past `c` instead
    assert e == c + 20 * MiB
    for p in (a, c, d, e):
        xh.free(p)
    xh.empty_cache()
    assert xh.stats()["reserved_bytes"]["all"]["current"] == 0


def test_expandable_small_pool_and_streams(xh):
    p = xh.alloc(1000)
    q = xh.alloc(1000, stream=0x20)   # another stream gets its own address range
    s = xh.stats()
    assert s["reserved_bytes"]["small_pool"]["current"] == 4 * MiB
    assert s["segment"]["small_pool"]["current"] == 2
    assert abs(p - q) >= 2 * MiB
    many = [xh.alloc(512 * 1024) for _ in range(7)]   # 3.5 MiB more on the default stream: grows by one unit
    assert xh.stats()["reserved_bytes"]["small_pool"]["current"] == 6 * MiB
    assert xh.stats()["segment"]["small_pool"]["current"] == 2
    for x in many + [p, q]:
        xh.free(x)
    xh.empty_cache()
    assert xh.stats()["reserved_bytes"]["all"]["current"] == 0


def test_expandable_respects_memory_fraction(xh):
    xh.set_memory_fraction(0.004)     # 16 GiB * 0.004 = ~65 MiB
    a = xh.alloc(30 * MiB)            # 40 MiB mapped
    with pytest.raises(RuntimeError, match="out of memory"):
        xh.alloc(60 * MiB)
    xh.free(a)
    b = xh.alloc(50 * MiB)            # 40 MiB cached + one more unit = 60 MiB: within the limit
    assert b == a
    xh.free(b)
    xh.empty_cache()


# ---------------------------------------------------------------- pool checkpoints
def test_pool_checkpoint_restore(h):
    pid = (0, 901)
    h.begin_pool(pid, 0x30)
    a = h.alloc(4 * MiB, stream=0x30)
    b = h.alloc(6 * MiB, stream=0x30)
    ck = h.checkpoint(pid)
    assert sorted(ck.live_pointers) == sorted([a, b])
    c = h.alloc(2 * MiB, stream=0x30)           # allocated after the checkpoint
    h.free(a)                                   # freed after the checkpoint
    h.end_pool(pid)
    freed, created = h.restore(ck)
    assert freed == [c]
    assert sorted(created) == sorted([a, b])
    snap = [s for s in h.snapshot() if tuple(s["pool_id"]) == pid]
    assert len(snap) == 1
    assert snap[0]["blocks"] == [(4 * MiB, True), (6 * MiB, True), (10 * MiB, False)]
    # the re-created blocks are ordinary live allocations again
    h.free(a); h.free(b)
    snap = [s for s in h.snapshot() if tuple(s["pool_id"]) == pid]
    assert snap[0]["blocks"] == [(20 * MiB, False)]
    h.release_pool(pid)
    assert h.stats()["reserved_bytes"]["all"]["current"] == 0


def test_canary_reports_a_write_past_the_end(bw):
    bw._C._set_allocator_settings("canary:True")
    try:
        h = bw._C._HostCacheHarness()
        a = h.alloc(1000)
        b = h.alloc(4096)
        h.write_read(a, 1000, 1)                      # stays inside: fine
        h.write_read(b, 4096 + 8, 2)                  # 8 bytes too many
        h.free(a)
        assert h.canary_violations() == 0
        h.free(b)                                     # logs a warning and counts the violation
        assert h.canary_violations() == 1
        assert "4096-byte allocation" in h.last_canary_report()
        # the guard bytes count towards the block size: 512 B requested no longer fits a 512 B block
        c = h.alloc(512)
        assert h.stats()["allocated_bytes"]["all"]["current"] == 1024
        h.free(c)
    finally:
        bw._C._set_allocator_settings("canary:False")


def test_snapshot_renderings(tmp_path):
    """Segment map, event trace and folded stacks from a snapshot dictionary (the layout `_snapshot()` returns)."""
    import pickle

    from torch_musa_b200.core import memory_viz as mv

    snap = {
        "segments": [
            {"device": 0, "address": 0x7000000, "total_size": 2 << 20, "allocated_size": 1 << 20, "segment_type": "small",
             "segment_pool_id": (0, 0), "is_expandable": False,
             "blocks": [{"address": 0x7000000, "size": 1 << 20, "requested_size": 1000000, "state": "active_allocated"},
                        {"address": 0x7100000, "size": 1 << 20, "requested_size": 0, "state": "inactive"}]},
            {"device": 0, "address": 0x9000000, "total_size": 20 << 20, "allocated_size": 0, "segment_type": "large",
             "segment_pool_id": (0, 3), "is_expandable": True, "blocks": []}],
        "device_traces": [[
            {"action": "segment_alloc", "addr": 0x7000000, "size": 2 << 20, "stream": 0, "device": 0, "time_us": 10},
            {"action": "alloc", "addr": 0x7000000, "size": 1 << 20, "stream": 0, "device": 0, "time_us": 11,
             "frames": "alloc_fn()\nat::empty()\nmodel_forward()\nmain"},
            {"action": "alloc", "addr": 0x7100000, "size": 1 << 20, "stream": 0, "device": 0, "time_us": 12,
             "frames": "alloc_fn()\nat::empty()\ntemp_buffer()\nmain"},
            {"action": "free_requested", "addr": 0x7100000, "size": 1 << 20, "stream": 0, "device": 0, "time_us": 13},
            {"action": "free_completed", "addr": 0x7100000, "size": 1 << 20, "stream": 0, "device": 0, "time_us": 14}]],
    }
    text = mv.segments_text(snap)
    assert "segment 0x7000000" in text and "expandable, pool (0, 3)" in text and "active_allocated (requested 976.6 KiB)" in text
    assert text.endswith("total: reserved 22.0 MiB, allocated 1.0 MiB, cached 21.0 MiB in 2 segments")
    assert mv.trace_text(snap).count("\n") == 4 and "free_completed" in mv.trace_text(snap, last=1)
    assert [e["addr"] for e in mv.live_allocations(snap)] == [0x7000000]
    assert mv.flamegraph_lines(snap) == ["main;model_forward();at::empty();alloc_fn() 1048576"]
    assert len(mv.flamegraph_lines(snap, live_only=False)) == 2
    p = tmp_path / "s.pickle"
    p.write_bytes(pickle.dumps(snap))
    assert mv.main([str(p), "--flamegraph", str(tmp_path / "o.folded")]) == 0
    assert (tmp_path / "o.folded").read_text().strip().endswith("1048576")
    assert mv.main([str(p)]) == 0 and mv.main([str(p), "--trace"]) == 0


@pytest.mark.parametrize("seed,expandable", [(0, False), (1, False), (2, True), (3, True)])
def test_randomised_alloc_free_keeps_invariants(bw, seed, expandable):
    """A few thousand random allocator operations (several streams, sizes from 1 byte to 40 MiB, frees in random order,
    cache flushes) on the host backend: live allocations never overlap, every one lies inside a segment of the
    snapshot, the statistics equal what the snapshot shows, and everything goes back to the system at the end."""
    import random

    prev = bw._C._allocator_config()["expandable_segments"]
    bw._C._set_allocator_settings(f"expandable_segments:{'True' if expandable else 'False'}")
    try:
        h = bw._C._HostCacheHarness()
        rng = random.Random(seed)
        live = {}                                  # ptr -> (nbytes, stream)
        sizes = [1, 17, 512, 4000, 70_000, 900_000, 3 * MiB, 11 * MiB, 40 * MiB]

        def check():
            spans = sorted((p, p + n) for p, (n, _) in live.items())
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 <= b0, "two live allocations overlap"
            snap = h.snapshot()
            segs = [(s["address"], s["address"] + s["total_size"]) for s in snap]
            for p, (n, _) in live.items():
                assert any(lo <= p and p + n <= hi for lo, hi in segs), "a live allocation lies outside every segment"
            st = h.stats()
            in_blocks = sum(size for s in snap for size, allocated in s["blocks"] if allocated)
            assert st["allocated_bytes"]["all"]["current"] == in_blocks
            assert st["allocated_bytes"]["all"]["current"] >= sum(n for n, _ in live.values())
            assert st["allocation"]["all"]["current"] == len(live)
            assert st["reserved_bytes"]["all"]["current"] >= st["allocated_bytes"]["all"]["current"]

        for step in range(1500):
            r = rng.random()
            if r < 0.55 or not live:
                n = max(1, int(rng.choice(sizes) * rng.uniform(0.5, 1.5)))
                stream = rng.choice([0, 0, 0x10, 0x20])
                p = h.alloc(n, stream=stream)
                assert p and p not in live
                live[p] = (n, stream)
            elif r < 0.95:
                p = rng.choice(list(live))
                if rng.random() < 0.2:
                    h.record_stream(p, rng.choice([0x10, 0x20, 0x30]))       # a use on another stream delays its reuse
                h.free(p)
                del live[p]
            else:
                h.empty_cache()
            if step % 100 == 0:
                check()
        check()
        for p in list(live):
            h.free(p)
        live.clear()
        h.empty_cache()
        st = h.stats()
        assert st["allocated_bytes"]["all"]["current"] == 0 and st["allocation"]["all"]["current"] == 0
        assert st["reserved_bytes"]["all"]["current"] == 0, "memory left cached after freeing everything and flushing"
    finally:
        bw._C._set_allocator_settings(f"expandable_segments:{'True' if prev else 'False'}")

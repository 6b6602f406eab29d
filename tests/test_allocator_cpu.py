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

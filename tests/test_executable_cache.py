"""Resident-executable cache policy, on the CPU through the C ABI.

The cases follow src/runtime/client_residency_tests.zig (:161-421): hit/miss accounting, lease counts, eviction under a
byte budget, victim order (largest first, then cheapest to compile, then least recently used), and memory-pressure
trims with their counters. Placeholder entries stand in for compiled executables, so no device is needed; the same
cache compiling real plans is covered by tests/test_gpu_ops.py.
"""
import pytest

from pjrtx_b200 import backend as be


@pytest.fixture()
def cache():
    c = be.ExecutableCache(be.Backend())
    yield c
    c.destroy()


def resident(cache, fingerprint, nbytes, bytes_in_use=0):
    hit = cache.record_compile(fingerprint)
    reused, trim = cache.install_placeholder(fingerprint, nbytes, bytes_in_use)
    return hit, reused, trim


def test_records_hits_and_misses(cache):
    assert cache.record_compile("same-program") is False
    assert cache.record_compile("same-program") is True
    s = cache.stats()
    assert (s["misses"], s["hits"]) == (1, 1)
    assert cache.entry("same-program") == {"resident": False, "resident_bytes": 0, "reference_count": 0,
                                           "compile_latency_us": 0}
    assert cache.entry("never-seen") is None


def test_reuses_resident_entry_and_counts_leases(cache):
    hit, reused, _ = resident(cache, "cached-add", 4)
    assert (hit, reused) == (False, False)
    assert cache.entry("cached-add")["reference_count"] == 1 and cache.entry("cached-add")["resident"]
    hit, reused, _ = resident(cache, "cached-add", 4)
    assert (hit, reused) == (True, True)
    s = cache.stats()
    assert (s["misses"], s["hits"], s["resident_entries"], s["resident_bytes"]) == (1, 1, 1, 4)
    assert cache.entry("cached-add")["reference_count"] == 2
    cache.release("cached-add")
    assert cache.entry("cached-add")["reference_count"] == 1
    cache.release("cached-add")
    e = cache.entry("cached-add")
    assert e["reference_count"] == 0 and e["resident"]          # idle entries stay resident without a budget
    cache.release("cached-add")                                 # an extra release does not underflow
    assert cache.entry("cached-add")["reference_count"] == 0


def test_unrecorded_fingerprint_is_refused(cache):
    with pytest.raises(be.BackendError, match="was not recorded"):
        cache.install_placeholder("unknown", 4)


def test_evicts_idle_entries_under_byte_limit(cache):
    cache.set_max_resident_bytes(0)
    resident(cache, "evict-idle-constant", 4)
    e = cache.entry("evict-idle-constant")
    assert e["resident"] and e["resident_bytes"] == 4 and e["reference_count"] == 1   # leased entries are never evicted
    assert cache.stats()["resident_entries"] == 1
    cache.release("evict-idle-constant")
    e = cache.entry("evict-idle-constant")
    assert not e["resident"] and e["reference_count"] == 0 and e["resident_bytes"] == 0
    s = cache.stats()
    assert (s["resident_entries"], s["resident_bytes"], s["evictions"], s["evicted_resident_bytes"]) == (0, 0, 1, 4)
    hit, reused, _ = resident(cache, "evict-idle-constant", 4)
    assert hit and not reused                                    # known fingerprint, but it has to compile again
    assert cache.entry("evict-idle-constant")["resident"]
    assert cache.stats()["hits"] == 1


def test_evicts_largest_idle_entry_before_older_smaller_ones(cache):
    resident(cache, "small-constant", 4)
    cache.release("small-constant")
    resident(cache, "large-constant", 8)
    cache.release("large-constant")
    cache.set_max_resident_bytes(4)
    assert cache.entry("small-constant")["resident"]
    assert not cache.entry("large-constant")["resident"]
    s = cache.stats()
    assert (s["resident_entries"], s["resident_bytes"], s["evictions"], s["evicted_resident_bytes"]) == (1, 4, 1, 8)
    assert s["peak_resident_bytes"] == 12 and s["largest_resident_bytes"] == 8


def test_keeps_the_more_expensive_of_equal_size_entries(cache):
    resident(cache, "cheap-constant", 4)
    cache.release("cheap-constant")
    cache.set_compile_latency("cheap-constant", 10)
    resident(cache, "expensive-constant", 4)
    cache.release("expensive-constant")
    cache.set_compile_latency("expensive-constant", 1000)
    cache.set_max_resident_bytes(4)
    assert not cache.entry("cheap-constant")["resident"]
    assert cache.entry("expensive-constant")["resident"]
    s = cache.stats()
    assert (s["resident_entries"], s["resident_bytes"], s["evictions"], s["evicted_resident_bytes"]) == (1, 4, 1, 4)


def test_least_recently_used_then_fingerprint_break_ties(cache):
    for name in ("b-entry", "a-entry", "c-entry"):
        resident(cache, name, 4)
    for name in ("b-entry", "a-entry", "c-entry"):
        cache.release(name)                                       # b is the least recently used
    cache.set_max_resident_bytes(8)
    assert [cache.entry(n)["resident"] for n in ("a-entry", "b-entry", "c-entry")] == [True, False, True]
    cache.set_max_resident_bytes(4)
    assert [cache.entry(n)["resident"] for n in ("a-entry", "b-entry", "c-entry")] == [False, False, True]


def test_trims_idle_entries_for_memory_pressure(cache):
    resident(cache, "pressure-small-constant", 4)
    cache.release("pressure-small-constant")
    resident(cache, "pressure-large-constant", 8)
    cache.release("pressure-large-constant")
    cache.set_capacity(4)
    trim = cache.trim_for_allocation(0, 0)
    assert trim == {"requested_bytes": 0, "target_resident_bytes": 4, "freed_bytes": 8, "evicted_entries": 1,
                    "remaining_resident_bytes": 4, "still_over_capacity": False}
    assert cache.entry("pressure-small-constant")["resident"]
    assert not cache.entry("pressure-large-constant")["resident"]
    s = cache.stats()
    assert (s["resident_bytes"], s["pressure_trim_requests"], s["pressure_trimmed_bytes"], s["pressure_trim_failures"]) == \
        (4, 1, 8, 0)
    # Within capacity: nothing is counted.
    trim = cache.trim_for_allocation(0, 0)
    assert trim["freed_bytes"] == 0 and trim["target_resident_bytes"] == 4
    assert cache.stats()["pressure_trim_requests"] == 1


def test_untracked_capacity_never_trims(cache):
    resident(cache, "idle", 8)
    cache.release("idle")
    trim = cache.trim_for_allocation(1 << 40, 1 << 40)
    assert trim == {"requested_bytes": 0, "target_resident_bytes": 0, "freed_bytes": 0, "evicted_entries": 0,
                    "remaining_resident_bytes": 0, "still_over_capacity": False}
    assert cache.entry("idle")["resident"]


def test_leased_entries_make_a_trim_fail(cache):
    resident(cache, "held", 8)
    cache.set_capacity(4)
    trim = cache.trim_for_allocation(0, 2)
    assert trim["still_over_capacity"] and trim["freed_bytes"] == 0 and trim["remaining_resident_bytes"] == 8
    assert trim["target_resident_bytes"] == 2 and trim["requested_bytes"] == 2
    assert cache.stats()["pressure_trim_failures"] == 1
    assert cache.entry("held")["resident"]


def test_compiling_trims_idle_entries_under_memory_pressure(cache):
    resident(cache, "compile-pressure-idle-constant", 8)
    cache.release("compile-pressure-idle-constant")
    cache.set_capacity(8)
    _, reused, trim = resident(cache, "compile-pressure-new-constant", 4)
    assert not reused
    assert cache.entry("compile-pressure-new-constant")["resident"]
    assert not cache.entry("compile-pressure-idle-constant")["resident"]
    assert trim == {"requested_bytes": 4, "target_resident_bytes": 4, "freed_bytes": 8, "evicted_entries": 1,
                    "remaining_resident_bytes": 0, "still_over_capacity": False}


def test_compile_needs_a_device(cache):
    """The compiling path goes to the device: without one it reports an error instead of installing anything."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from pjrtx_b200 import plan as plan_mod
    b = plan_mod.PlanBuilder()
    x = b.parameter(plan_mod.F32, [4])
    b.set_outputs([x + x])
    with pytest.raises(be.BackendError):
        cache.compile(b)
    s = cache.stats()
    assert s["misses"] == 1 and s["resident_entries"] == 0


def test_fingerprint_covers_the_target_devices():
    """src/runtime/executable_fingerprint.zig:38-56 hashes the resolved target devices: the same plan for another GPU
    (or another device list) is another cache entry, and the key is stable for equal lists."""
    from tests import cases

    backend = be.Backend()
    b, _ = cases.u8_chain()
    on0 = backend.plan_fingerprint(b, [0])
    assert on0 == backend.plan_fingerprint(b, [0])
    assert on0 != backend.plan_fingerprint(b, [1])
    assert len({on0, backend.plan_fingerprint(b, [1]), backend.plan_fingerprint(b, [0, 1]), backend.plan_fingerprint(b, [1, 0]),
                backend.plan_fingerprint(b)}) == 5

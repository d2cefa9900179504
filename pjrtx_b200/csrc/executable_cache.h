// Resident-executable cache keyed by plan fingerprint.
//
// Behaviour follows the reference's runtime cache (src/runtime/executable_cache.zig): a compile request is a hit when
// the fingerprint has been seen (:199-213); a compiled executable stays resident while leases hold it and afterwards
// until a byte budget or a memory-pressure trim asks for room (:246-330); the victim among idle resident entries is the
// one holding most bytes, then the cheapest to compile again, then the least recently used, then the smaller
// fingerprint (:284-313). A B200 executable's resident bytes are the device memory it owns (constants, arena,
// contraction scratch), so evicting one frees HBM for buffers.
//
// The cache stores opaque handles and a destroy callback, so the policy is exercised without a device.
#pragma once

#include <cstdint>
#include <functional>
#include <mutex>
#include <string>
#include <unordered_map>

namespace pjrtx {

struct CacheStats {
  uint64_t hits = 0;
  uint64_t misses = 0;
  uint64_t evictions = 0;
  uint64_t evicted_resident_bytes = 0;
  uint64_t resident_entries = 0;
  uint64_t resident_bytes = 0;
  uint64_t peak_resident_bytes = 0;
  uint64_t largest_resident_bytes = 0;
  uint64_t compile_latency_samples = 0;
  uint64_t compile_latency_us_total = 0;
  uint64_t compile_latency_us_peak = 0;
  uint64_t pressure_trim_requests = 0;
  uint64_t pressure_trimmed_bytes = 0;
  uint64_t pressure_trim_failures = 0;
};

struct CacheTrim {
  uint64_t requested_bytes = 0;
  uint64_t target_resident_bytes = 0;
  uint64_t freed_bytes = 0;
  uint64_t evicted_entries = 0;
  uint64_t remaining_resident_bytes = 0;
  bool still_over_capacity = false;
};

struct CacheEntrySnapshot {
  bool resident = false;
  uint64_t resident_bytes = 0;
  uint64_t reference_count = 0;
  uint64_t compile_latency_us = 0;
};

class ExecutableCache {
 public:
  using Destroy = std::function<void(void*)>;

  explicit ExecutableCache(Destroy destroy) : destroy_(std::move(destroy)) {}
  ~ExecutableCache();
  ExecutableCache(const ExecutableCache&) = delete;
  ExecutableCache& operator=(const ExecutableCache&) = delete;

  // Registers a compile request; true when the fingerprint was already known.
  bool record_compile(const std::string& fingerprint);

  // Takes a lease on the resident executable of `fingerprint`; nullptr when the fingerprint is unknown or not resident.
  void* retain_resident(const std::string& fingerprint);

  // Makes a freshly compiled handle resident with one lease. The fingerprint must have been recorded. `capacity_bytes`
  // (0 = untracked) and `bytes_in_use` describe the memory the executable's `resident_bytes` are placed in: idle entries
  // are trimmed first so that buffers, the cache and the new executable fit (`*compile_trim`). When another thread made
  // the fingerprint resident in the meantime, `handle` is destroyed and the winner is leased (`*reused` = true).
  // Returns nullptr for an unknown fingerprint (the handle is destroyed).
  void* install(const std::string& fingerprint, void* handle, uint64_t resident_bytes, uint64_t compile_latency_us,
                uint64_t capacity_bytes, uint64_t bytes_in_use, bool* reused, CacheTrim* compile_trim);

  // Returns a lease; idle entries beyond the byte budget are evicted.
  void release(const std::string& fingerprint);

  void set_max_resident_bytes(uint64_t max_resident_bytes);
  void set_compile_latency(const std::string& fingerprint, uint64_t latency_us);

  // Evicts idle entries until buffers (`bytes_in_use`), `allocation_bytes` and the cache fit into `capacity_bytes`.
  CacheTrim trim_for_allocation(uint64_t capacity_bytes, uint64_t bytes_in_use, uint64_t allocation_bytes);

  CacheStats stats() const;
  bool entry(const std::string& fingerprint, CacheEntrySnapshot* out) const;

 private:
  struct Entry {
    void* handle = nullptr;
    uint64_t resident_bytes = 0;
    uint64_t compile_latency_us = 0;
    uint64_t ref_count = 0;
    uint64_t last_use = 0;
  };
  using Map = std::unordered_map<std::string, Entry>;

  void touch(Entry& e) { e.last_use = ++next_use_; }
  Map::iterator victim();
  void evict(Entry& e);
  void evict_until_under_limit();
  CacheTrim trim_idle_to(uint64_t target_resident_bytes);
  CacheTrim trim_for_allocation_locked(uint64_t capacity_bytes, uint64_t bytes_in_use, uint64_t allocation_bytes);

  Destroy destroy_;
  mutable std::mutex mutex_;
  Map entries_;
  CacheStats stats_;
  uint64_t max_resident_bytes_ = UINT64_MAX;
  uint64_t next_use_ = 0;
};

}  // namespace pjrtx

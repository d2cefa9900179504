#include "executable_cache.h"

#include <algorithm>

namespace pjrtx {

namespace {
uint64_t sat_add(uint64_t a, uint64_t b) { return a > UINT64_MAX - b ? UINT64_MAX : a + b; }
}  // namespace

ExecutableCache::~ExecutableCache() {
  for (auto& kv : entries_)
    if (kv.second.handle) destroy_(kv.second.handle);
}

bool ExecutableCache::record_compile(const std::string& fingerprint) {
  std::lock_guard<std::mutex> lock(mutex_);
  if (entries_.count(fingerprint)) {
    stats_.hits++;
    return true;
  }
  entries_.emplace(fingerprint, Entry{});
  stats_.misses++;
  return false;
}

void* ExecutableCache::retain_resident(const std::string& fingerprint) {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = entries_.find(fingerprint);
  if (it == entries_.end() || !it->second.handle) return nullptr;
  it->second.ref_count++;
  touch(it->second);
  return it->second.handle;
}

void* ExecutableCache::install(const std::string& fingerprint, void* handle, uint64_t resident_bytes,
                               uint64_t compile_latency_us, uint64_t capacity_bytes, uint64_t bytes_in_use, bool* reused,
                               CacheTrim* compile_trim) {
  std::lock_guard<std::mutex> lock(mutex_);
  if (reused) *reused = false;
  if (compile_trim) *compile_trim = CacheTrim{};
  auto it = entries_.find(fingerprint);
  if (it == entries_.end()) {
    if (handle) destroy_(handle);
    return nullptr;
  }
  Entry& e = it->second;
  // Room for the new executable's device bytes comes out of idle entries before it is counted as resident
  // (src/runtime/executable_cache.zig:452-456).
  CacheTrim trim;
  if (resident_bytes != 0 && capacity_bytes != 0) trim = trim_for_allocation_locked(capacity_bytes, bytes_in_use, resident_bytes);
  if (compile_trim) *compile_trim = trim;
  if (e.handle) {  // lost a compile race: keep the resident one
    if (handle && handle != e.handle) destroy_(handle);
    e.ref_count++;
    touch(e);
    if (reused) *reused = true;
    return e.handle;
  }
  e.handle = handle;
  e.resident_bytes = resident_bytes;
  e.ref_count = 1;
  touch(e);
  stats_.resident_entries++;
  stats_.resident_bytes = sat_add(stats_.resident_bytes, resident_bytes);
  stats_.peak_resident_bytes = std::max(stats_.peak_resident_bytes, stats_.resident_bytes);
  stats_.largest_resident_bytes = std::max(stats_.largest_resident_bytes, resident_bytes);
  evict_until_under_limit();
  e.compile_latency_us = compile_latency_us;
  stats_.compile_latency_samples++;
  stats_.compile_latency_us_total = sat_add(stats_.compile_latency_us_total, compile_latency_us);
  stats_.compile_latency_us_peak = std::max(stats_.compile_latency_us_peak, compile_latency_us);
  return handle;
}

void ExecutableCache::release(const std::string& fingerprint) {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = entries_.find(fingerprint);
  if (it == entries_.end()) return;
  if (it->second.ref_count) it->second.ref_count--;
  touch(it->second);
  evict_until_under_limit();
}

void ExecutableCache::set_max_resident_bytes(uint64_t max_resident_bytes) {
  std::lock_guard<std::mutex> lock(mutex_);
  max_resident_bytes_ = max_resident_bytes;
  evict_until_under_limit();
}

void ExecutableCache::set_compile_latency(const std::string& fingerprint, uint64_t latency_us) {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = entries_.find(fingerprint);
  if (it != entries_.end()) it->second.compile_latency_us = latency_us;
}

CacheTrim ExecutableCache::trim_for_allocation(uint64_t capacity_bytes, uint64_t bytes_in_use, uint64_t allocation_bytes) {
  std::lock_guard<std::mutex> lock(mutex_);
  return trim_for_allocation_locked(capacity_bytes, bytes_in_use, allocation_bytes);
}

// src/runtime/executable_cache.zig:404-426: nothing to do while buffers + allocation + cache fit; otherwise the cache is
// asked to shrink to what the capacity leaves, and the request is counted (a failure when idle entries did not suffice).
CacheTrim ExecutableCache::trim_for_allocation_locked(uint64_t capacity_bytes, uint64_t bytes_in_use, uint64_t allocation_bytes) {
  CacheTrim trim;
  if (capacity_bytes == 0) return trim;
  const uint64_t without_cache = sat_add(bytes_in_use, allocation_bytes);
  const uint64_t resident = stats_.resident_bytes;
  if (sat_add(without_cache, resident) <= capacity_bytes) {
    trim.requested_bytes = allocation_bytes;
    trim.target_resident_bytes = resident;
    trim.remaining_resident_bytes = resident;
    return trim;
  }
  const uint64_t target = without_cache >= capacity_bytes ? 0 : capacity_bytes - without_cache;
  trim = trim_idle_to(target);
  trim.requested_bytes = allocation_bytes;
  trim.still_over_capacity = sat_add(without_cache, trim.remaining_resident_bytes) > capacity_bytes;
  stats_.pressure_trim_requests++;
  stats_.pressure_trimmed_bytes = sat_add(stats_.pressure_trimmed_bytes, trim.freed_bytes);
  if (trim.still_over_capacity) stats_.pressure_trim_failures++;
  return trim;
}

CacheStats ExecutableCache::stats() const {
  std::lock_guard<std::mutex> lock(mutex_);
  return stats_;
}

bool ExecutableCache::entry(const std::string& fingerprint, CacheEntrySnapshot* out) const {
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = entries_.find(fingerprint);
  if (it == entries_.end()) return false;
  if (out) {
    out->resident = it->second.handle != nullptr;
    out->resident_bytes = it->second.resident_bytes;
    out->reference_count = it->second.ref_count;
    out->compile_latency_us = it->second.compile_latency_us;
  }
  return true;
}

// Idle resident entry to give up first: most bytes; among equals the cheapest to compile again, then the least
// recently used, then the smaller fingerprint (src/runtime/executable_cache.zig:284-313).
ExecutableCache::Map::iterator ExecutableCache::victim() {
  auto best = entries_.end();
  for (auto it = entries_.begin(); it != entries_.end(); ++it) {
    const Entry& e = it->second;
    if (!e.handle || e.ref_count != 0) continue;
    if (best == entries_.end()) {
      best = it;
      continue;
    }
    const Entry& b = best->second;
    if (e.resident_bytes != b.resident_bytes) {
      if (e.resident_bytes > b.resident_bytes) best = it;
    } else if (e.compile_latency_us != b.compile_latency_us) {
      if (e.compile_latency_us < b.compile_latency_us) best = it;
    } else if (e.last_use != b.last_use) {
      if (e.last_use < b.last_use) best = it;
    } else if (it->first < best->first) {
      best = it;
    }
  }
  return best;
}

void ExecutableCache::evict(Entry& e) {
  if (!e.handle || e.ref_count != 0) return;
  destroy_(e.handle);
  e.handle = nullptr;
  stats_.evicted_resident_bytes = sat_add(stats_.evicted_resident_bytes, e.resident_bytes);
  stats_.resident_bytes = e.resident_bytes > stats_.resident_bytes ? 0 : stats_.resident_bytes - e.resident_bytes;
  e.resident_bytes = 0;
  if (stats_.resident_entries) stats_.resident_entries--;
  stats_.evictions++;
}

void ExecutableCache::evict_until_under_limit() {
  while (stats_.resident_bytes > max_resident_bytes_) {
    auto it = victim();
    if (it == entries_.end()) return;
    evict(it->second);
  }
}

CacheTrim ExecutableCache::trim_idle_to(uint64_t target_resident_bytes) {
  const uint64_t before_bytes = stats_.resident_bytes;
  const uint64_t before_evictions = stats_.evictions;
  while (stats_.resident_bytes > target_resident_bytes) {
    auto it = victim();
    if (it == entries_.end()) break;
    evict(it->second);
  }
  CacheTrim trim;
  trim.target_resident_bytes = target_resident_bytes;
  trim.freed_bytes = before_bytes - stats_.resident_bytes;
  trim.evicted_entries = stats_.evictions - before_evictions;
  trim.remaining_resident_bytes = stats_.resident_bytes;
  trim.still_over_capacity = stats_.resident_bytes > target_resident_bytes;
  return trim;
}

}  // namespace pjrtx

// CUDA device / stream / event / buffer model of the backend.
//
// The reference keeps one memory space per device and immutable device buffers
// with ready events (src/runtime/device_memory.zig:157-236, src/runtime/buffer.zig,
// src/backend/mlx_metal/api.cc:827-905 for host→device, :5685-5710 for
// device→host). Here each device owns one in-order compute stream, a
// cudaMallocAsync pool and (for tensor parallelism) one NCCL communicator.
#pragma once

#include <cuda_runtime.h>

#include <mutex>
#include <string>
#include <vector>

#include "common.h"

namespace pjrtx {

struct Device {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
  uint64_t memory_bytes = 0;
  char name[128] = {0};
  // Pinned staging for small host→device copies so the caller's memory is free
  // again when the call returns without a stream synchronize.
  uint8_t* staging = nullptr;
  size_t staging_size = 0, staging_head = 0;
  cudaEvent_t staging_wrap_event = nullptr;
  // Written by kernels whose bounded waits give up (host-mapped so the host reads it without a copy).
  int* error_flag_host = nullptr;
  int* error_flag_dev = nullptr;
  // Tensor-parallel communicator (void* = ncclComm_t), set by comm_init.
  void* comm = nullptr;
  int comm_rank = 0, comm_world = 1;
  // Peer-mapped regions for the one-shot all-reduce (kernels/peer_reduce.cu): peer_regions[r] is rank r's region as
  // mapped into this process, peer_regions[peer_rank] the local allocation.
  void* peer_regions[8] = {nullptr};
  uint64_t peer_slot_bytes = 0;
  int peer_rank = 0, peer_world = 0;
  bool peer_ready = false;
  std::mutex mu;
  // Transfer counters (src/runtime/device_memory.zig:258-304).
  uint64_t h2d_bytes = 0, d2h_bytes = 0, live_bytes = 0, peak_bytes = 0;
};

int device_count();                 // 0 when no CUDA device is usable
Device* get_device(int ordinal);    // nullptr + last_error on failure
bool check_cuda(cudaError_t e, const char* what);
// After a stream synchronize: false (with last_error set) when a kernel reported a timed-out device-side wait.
bool check_device_flag(Device* dev);

struct Buffer {
  int device = 0;
  int dtype = kInvalid;
  std::vector<int64_t> dims;
  void* ptr = nullptr;
  uint64_t bytes = 0;
  bool owns = true;
  bool donated = false;  // storage moved into an execution output
};

Buffer* buffer_alloc(Device* dev, int dtype, const std::vector<int64_t>& dims, bool zero);
Buffer* buffer_from_host(Device* dev, const void* data, uint64_t byte_size, int dtype,
                         const std::vector<int64_t>& dims);
bool buffer_to_host(Buffer* b, void* dst, uint64_t dst_size);
void buffer_free(Buffer* b);

void* device_malloc(Device* dev, uint64_t bytes);
void device_free(Device* dev, void* p, uint64_t bytes);

// Run-time compilation of generated kernels (NVRTC → cubin → cudaLibrary).
struct JitKernel {
  cudaLibrary_t library = nullptr;
  cudaKernel_t kernel = nullptr;
};
// Compiles for sm_100a and returns the cubin; needs no GPU.
bool jit_compile_cubin(const std::string& source, std::vector<char>* cubin, std::string* log);
// Compiles (cached by source text) and loads; needs a GPU.
JitKernel* jit_get_kernel(const std::string& source, const char* entry, std::string* log);

// NCCL, loaded with dlopen so the library also loads where NCCL is absent.
bool comm_unique_id(uint8_t out[128]);
bool comm_init(Device* dev, const uint8_t id[128], int rank, int world);
// Small sums go through the peer-memory kernel when the regions are set up (and PJRTX_B200_PEER_ALLREDUCE is not 0).
bool comm_all_reduce_sum(Device* dev, const void* src, void* dst, uint64_t count, int dtype, bool pdl = false);
// Peer regions: every rank exports a handle of its own region, the host ships all handles to all ranks, every rank
// imports them. All ranks must have exported before any rank executes.
bool comm_peer_export(Device* dev, uint8_t handle[64]);
bool comm_peer_import(Device* dev, const uint8_t* handles, int rank, int world);
void comm_peer_close(Device* dev);
bool comm_all_gather(Device* dev, const void* src, void* dst, uint64_t send_count, int dtype);
void comm_destroy(Device* dev);

}  // namespace pjrtx

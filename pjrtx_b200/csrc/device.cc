#include "device.h"

#include "kernels/kernels.h"

#include <dlfcn.h>
#include <nccl.h>
#include <nvrtc.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>

namespace pjrtx {

bool check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  set_last_error("%s: %s", what, cudaGetErrorString(e));
  return false;
}

int device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

static std::mutex g_devices_mu;
static std::map<int, std::unique_ptr<Device>> g_devices;

Device* get_device(int ordinal) {
  std::lock_guard<std::mutex> lock(g_devices_mu);
  auto it = g_devices.find(ordinal);
  if (it != g_devices.end()) return it->second.get();
  int n = device_count();
  if (ordinal < 0 || ordinal >= n) {
    set_last_error("device ordinal %d is not available (%d CUDA devices)", ordinal, n);
    return nullptr;
  }
  if (!check_cuda(cudaSetDevice(ordinal), "cudaSetDevice")) return nullptr;
  auto dev = std::make_unique<Device>();
  dev->ordinal = ordinal;
  cudaDeviceProp prop;
  if (!check_cuda(cudaGetDeviceProperties(&prop, ordinal), "cudaGetDeviceProperties")) return nullptr;
  if (prop.major != 10) {
    set_last_error("device %d is sm_%d%d; this backend only runs on sm_100a (B200)", ordinal, prop.major, prop.minor);
    return nullptr;
  }
  dev->sm_count = prop.multiProcessorCount;
  dev->memory_bytes = prop.totalGlobalMem;
  snprintf(dev->name, sizeof dev->name, "%.*s", (int)sizeof dev->name - 1, prop.name);
  if (!check_cuda(cudaStreamCreateWithFlags(&dev->stream, cudaStreamNonBlocking), "cudaStreamCreate")) return nullptr;
  cudaMemPool_t pool;
  if (check_cuda(cudaDeviceGetDefaultMemPool(&pool, ordinal), "cudaDeviceGetDefaultMemPool")) {
    uint64_t threshold = UINT64_MAX;  // keep freed blocks cached in the pool
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold);
  }
  dev->staging_size = 1 << 20;
  if (!check_cuda(cudaMallocHost((void**)&dev->staging, dev->staging_size), "cudaMallocHost")) return nullptr;
  cudaEventCreateWithFlags(&dev->staging_wrap_event, cudaEventDisableTiming);
  if (!check_cuda(cudaHostAlloc((void**)&dev->error_flag_host, sizeof(int), cudaHostAllocMapped), "cudaHostAlloc")) return nullptr;
  *dev->error_flag_host = 0;
  if (!check_cuda(cudaHostGetDevicePointer((void**)&dev->error_flag_dev, dev->error_flag_host, 0), "cudaHostGetDevicePointer")) return nullptr;
  Device* raw = dev.get();
  g_devices[ordinal] = std::move(dev);
  return raw;
}

bool check_device_flag(Device* dev) {
  if (!dev->error_flag_host) return true;
  int code = *(volatile int*)dev->error_flag_host;
  if (code == 0) return true;
  *(volatile int*)dev->error_flag_host = 0;
  set_last_error("a kernel on device %d gave up a bounded wait (code %d); results of this stream are invalid", dev->ordinal, code);
  return false;
}

void* device_malloc(Device* dev, uint64_t bytes) {
  void* p = nullptr;
  if (bytes == 0) bytes = 1;
  cudaSetDevice(dev->ordinal);
  if (!check_cuda(cudaMallocAsync(&p, bytes, dev->stream), "cudaMallocAsync")) return nullptr;
  std::lock_guard<std::mutex> lock(dev->mu);
  dev->live_bytes += bytes;
  if (dev->live_bytes > dev->peak_bytes) dev->peak_bytes = dev->live_bytes;
  return p;
}

void device_free(Device* dev, void* p, uint64_t bytes) {
  if (!p) return;
  cudaSetDevice(dev->ordinal);
  cudaFreeAsync(p, dev->stream);
  std::lock_guard<std::mutex> lock(dev->mu);
  if (bytes == 0) bytes = 1;
  dev->live_bytes -= bytes > dev->live_bytes ? dev->live_bytes : bytes;
}

Buffer* buffer_alloc(Device* dev, int dtype, const std::vector<int64_t>& dims, bool zero) {
  if (dtype_size(dtype) == 0) {
    set_last_error("unsupported element type %d", dtype);
    return nullptr;
  }
  for (int64_t d : dims)
    if (d < 0) {
      set_last_error("negative dimension");
      return nullptr;
    }
  uint64_t bytes = dense_byte_size(dtype, dims);
  void* p = device_malloc(dev, bytes);
  if (!p) return nullptr;
  if (zero && bytes && !check_cuda(cudaMemsetAsync(p, 0, bytes, dev->stream), "cudaMemsetAsync")) {
    device_free(dev, p, bytes);
    return nullptr;
  }
  Buffer* b = new Buffer();
  b->device = dev->ordinal;
  b->dtype = dtype;
  b->dims = dims;
  b->ptr = p;
  b->bytes = bytes;
  return b;
}

Buffer* buffer_from_host(Device* dev, const void* data, uint64_t byte_size, int dtype,
                         const std::vector<int64_t>& dims) {
  if (dense_byte_size(dtype, dims) != byte_size) {
    set_last_error("host buffer holds %llu bytes but the descriptor needs %llu", (unsigned long long)byte_size,
                   (unsigned long long)dense_byte_size(dtype, dims));
    return nullptr;
  }
  if (byte_size && !data) {
    set_last_error("null host pointer");
    return nullptr;
  }
  Buffer* b = buffer_alloc(dev, dtype, dims, false);
  if (!b) return nullptr;
  if (byte_size == 0) return b;
  bool ok;
  if (byte_size <= dev->staging_size / 64) {
    // Small transfer: bounce through the pinned ring, no host-side wait.
    std::lock_guard<std::mutex> lock(dev->mu);
    size_t need = (byte_size + 63) & ~(size_t)63;
    if (dev->staging_head + need > dev->staging_size) {
      // Wrapping: everything queued from the ring so far must have been consumed.
      cudaEventRecord(dev->staging_wrap_event, dev->stream);
      cudaEventSynchronize(dev->staging_wrap_event);
      dev->staging_head = 0;
    }
    uint8_t* slot = dev->staging + dev->staging_head;
    dev->staging_head += need;
    memcpy(slot, data, byte_size);
    ok = check_cuda(cudaMemcpyAsync(b->ptr, slot, byte_size, cudaMemcpyHostToDevice, dev->stream), "cudaMemcpyAsync h2d");
  } else {
    ok = check_cuda(cudaMemcpyAsync(b->ptr, data, byte_size, cudaMemcpyHostToDevice, dev->stream), "cudaMemcpyAsync h2d") &&
         check_cuda(cudaStreamSynchronize(dev->stream), "cudaStreamSynchronize");
  }
  if (!ok) {
    buffer_free(b);
    return nullptr;
  }
  dev->h2d_bytes += byte_size;
  return b;
}

bool buffer_to_host(Buffer* b, void* dst, uint64_t dst_size) {
  if (!b || b->donated || !b->ptr) {
    set_last_error("buffer is deleted or donated");
    return false;
  }
  if (dst_size < b->bytes) {
    set_last_error("destination holds %llu bytes, buffer needs %llu", (unsigned long long)dst_size,
                   (unsigned long long)b->bytes);
    return false;
  }
  Device* dev = get_device(b->device);
  if (!dev) return false;
  cudaSetDevice(dev->ordinal);
  if (b->bytes == 0) return true;
  if (!check_cuda(cudaMemcpyAsync(dst, b->ptr, b->bytes, cudaMemcpyDeviceToHost, dev->stream), "cudaMemcpyAsync d2h")) return false;
  if (!check_cuda(cudaStreamSynchronize(dev->stream), "cudaStreamSynchronize")) return false;
  if (!check_device_flag(dev)) return false;
  dev->d2h_bytes += b->bytes;
  return true;
}

void buffer_free(Buffer* b) {
  if (!b) return;
  if (b->owns && b->ptr && !b->donated) {
    Device* dev = get_device(b->device);
    if (dev) device_free(dev, b->ptr, b->bytes);
  }
  delete b;
}

// ---------------------------------------------------------------------------
// NVRTC, resolved at run time so that loading this library never needs it.

namespace {

struct Nvrtc {
  void* handle = nullptr;
  nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*);
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char*);
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char*);
  nvrtcResult (*DestroyProgram)(nvrtcProgram*);
  const char* (*GetErrorString)(nvrtcResult);
};

Nvrtc* nvrtc() {
  static Nvrtc api;
  static bool tried = false;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (tried) return api.handle ? &api : nullptr;
  tried = true;
  const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                         "/usr/local/cuda/lib64/libnvrtc.so"};
  for (const char* n : names) {
    api.handle = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    if (api.handle) break;
  }
  if (!api.handle) return nullptr;
#define LOAD(field, sym)                                             \
  *(void**)(&api.field) = dlsym(api.handle, sym);                    \
  if (!api.field) {                                                  \
    dlclose(api.handle);                                             \
    api.handle = nullptr;                                            \
    return nullptr;                                                  \
  }
  LOAD(CreateProgram, "nvrtcCreateProgram")
  LOAD(CompileProgram, "nvrtcCompileProgram")
  LOAD(GetProgramLogSize, "nvrtcGetProgramLogSize")
  LOAD(GetProgramLog, "nvrtcGetProgramLog")
  LOAD(GetCUBINSize, "nvrtcGetCUBINSize")
  LOAD(GetCUBIN, "nvrtcGetCUBIN")
  LOAD(DestroyProgram, "nvrtcDestroyProgram")
  LOAD(GetErrorString, "nvrtcGetErrorString")
#undef LOAD
  return &api;
}

std::string cuda_include_flag() {
  const char* home = getenv("CUDA_HOME");
  if (!home) home = getenv("CUDA_PATH");
  if (!home) home = "/usr/local/cuda";
  return std::string("-I") + home + "/include";
}

}  // namespace

bool jit_compile_cubin(const std::string& source, std::vector<char>* cubin, std::string* log) {
  Nvrtc* rt = nvrtc();
  if (!rt) {
    if (log) *log = "libnvrtc could not be loaded; generated fusion kernels cannot be compiled";
    return false;
  }
  nvrtcProgram prog;
  nvrtcResult r = rt->CreateProgram(&prog, source.c_str(), "pjrtx_fused.cu", 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) {
    if (log) *log = rt->GetErrorString(r);
    return false;
  }
  std::string inc = cuda_include_flag();
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", inc.c_str(), "-lineinfo"};
  r = rt->CompileProgram(prog, 4, opts);
  size_t log_size = 0;
  rt->GetProgramLogSize(prog, &log_size);
  if (log && log_size > 1) {
    log->resize(log_size);
    rt->GetProgramLog(prog, &(*log)[0]);
  }
  if (r != NVRTC_SUCCESS) {
    if (log && log->empty()) *log = rt->GetErrorString(r);
    rt->DestroyProgram(&prog);
    return false;
  }
  size_t size = 0;
  rt->GetCUBINSize(prog, &size);
  cubin->resize(size);
  rt->GetCUBIN(prog, cubin->data());
  rt->DestroyProgram(&prog);
  return true;
}

JitKernel* jit_get_kernel(const std::string& source, const char* entry, std::string* log) {
  static std::mutex mu;
  static std::map<std::string, std::unique_ptr<JitKernel>> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(source);
  if (it != cache.end()) return it->second.get();
  std::vector<char> cubin;
  if (!jit_compile_cubin(source, &cubin, log)) return nullptr;
  auto k = std::make_unique<JitKernel>();
  cudaError_t e = cudaLibraryLoadData(&k->library, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
  if (e != cudaSuccess) {
    if (log) *log = std::string("cudaLibraryLoadData: ") + cudaGetErrorString(e);
    return nullptr;
  }
  e = cudaLibraryGetKernel(&k->kernel, k->library, entry);
  if (e != cudaSuccess) {
    if (log) *log = std::string("cudaLibraryGetKernel: ") + cudaGetErrorString(e);
    return nullptr;
  }
  JitKernel* raw = k.get();
  cache[source] = std::move(k);
  return raw;
}

// ---------------------------------------------------------------------------
// NCCL through dlopen.

namespace {

struct Nccl {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  const char* (*GetErrorString)(ncclResult_t);
};

Nccl* nccl() {
  static Nccl api;
  static bool tried = false;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (tried) return api.handle ? &api : nullptr;
  tried = true;
  api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!api.handle) return nullptr;
  *(void**)(&api.GetUniqueId) = dlsym(api.handle, "ncclGetUniqueId");
  *(void**)(&api.CommInitRank) = dlsym(api.handle, "ncclCommInitRank");
  *(void**)(&api.AllReduce) = dlsym(api.handle, "ncclAllReduce");
  *(void**)(&api.AllGather) = dlsym(api.handle, "ncclAllGather");
  *(void**)(&api.CommDestroy) = dlsym(api.handle, "ncclCommDestroy");
  *(void**)(&api.GetErrorString) = dlsym(api.handle, "ncclGetErrorString");
  if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.AllGather || !api.CommDestroy) {
    api.handle = nullptr;
    return nullptr;
  }
  return &api;
}

bool nccl_type(int dtype, ncclDataType_t* out) {
  switch (dtype) {
    case kF32: *out = ncclFloat32; return true;
    case kF16: *out = ncclFloat16; return true;
    case kBF16: *out = ncclBfloat16; return true;
    case kS32: *out = ncclInt32; return true;
    case kU32: *out = ncclUint32; return true;
    case kS64: *out = ncclInt64; return true;
    case kU64: *out = ncclUint64; return true;
    case kS8: *out = ncclInt8; return true;
    case kU8: case kPred: *out = ncclUint8; return true;
    default: return false;
  }
}

bool check_nccl(Nccl* api, ncclResult_t r, const char* what) {
  if (r == ncclSuccess) return true;
  set_last_error("%s: %s", what, api->GetErrorString ? api->GetErrorString(r) : "nccl error");
  return false;
}

}  // namespace

bool comm_unique_id(uint8_t out[128]) {
  Nccl* api = nccl();
  if (!api) {
    set_last_error("libnccl could not be loaded");
    return false;
  }
  ncclUniqueId id;
  static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
  if (!check_nccl(api, api->GetUniqueId(&id), "ncclGetUniqueId")) return false;
  memcpy(out, &id, 128);
  return true;
}

bool comm_init(Device* dev, const uint8_t id_bytes[128], int rank, int world) {
  Nccl* api = nccl();
  if (!api) {
    set_last_error("libnccl could not be loaded");
    return false;
  }
  if (dev->comm) comm_destroy(dev);
  ncclUniqueId id;
  memcpy(&id, id_bytes, 128);
  cudaSetDevice(dev->ordinal);
  ncclComm_t comm;
  if (!check_nccl(api, api->CommInitRank(&comm, world, id, rank), "ncclCommInitRank")) return false;
  dev->comm = comm;
  dev->comm_rank = rank;
  dev->comm_world = world;
  return true;
}

namespace {
constexpr uint64_t kPeerSlotBytes = 1ull << 20;  // one part in wire format: sums of up to world x 512 KiB
bool peer_enabled() {
  const char* v = getenv("PJRTX_B200_PEER_ALLREDUCE");
  return !(v && *v == '0');
}
}  // namespace

bool comm_peer_export(Device* dev, uint8_t handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaSetDevice(dev->ordinal);
  if (!dev->peer_regions[0] || dev->peer_ready) {
    // (re)create the local region; it is parked in slot 0 until the import knows this rank's number
    comm_peer_close(dev);
    void* region = nullptr;
    const uint64_t bytes = peer_region_bytes(kPeerSlotBytes);
    if (!check_cuda(cudaMalloc(&region, bytes), "cudaMalloc(peer region)")) return false;
    if (!check_cuda(cudaMemset(region, 0, bytes), "cudaMemset(peer region)") ||
        !check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) {
      cudaFree(region);
      return false;
    }
    dev->peer_regions[0] = region;
    dev->peer_slot_bytes = kPeerSlotBytes;
    dev->peer_world = 0;
  }
  cudaIpcMemHandle_t h;
  if (!check_cuda(cudaIpcGetMemHandle(&h, dev->peer_regions[0]), "cudaIpcGetMemHandle")) return false;
  memcpy(handle, &h, 64);
  return true;
}

bool comm_peer_import(Device* dev, const uint8_t* handles, int rank, int world) {
  if (world < 2 || world > 8 || rank < 0 || rank >= world) {
    set_last_error("peer regions support 2..8 ranks (got rank %d of %d)", rank, world);
    return false;
  }
  if (!dev->peer_regions[0] || dev->peer_world != 0) {
    set_last_error("export this rank's peer region before importing the others");
    return false;
  }
  cudaSetDevice(dev->ordinal);
  void* local = dev->peer_regions[0];
  dev->peer_regions[0] = nullptr;
  for (int r = 0; r < world; r++) {
    if (r == rank) {
      dev->peer_regions[r] = local;
      continue;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * 64, 64);
    void* mapped = nullptr;
    if (!check_cuda(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) {
      dev->peer_rank = rank;
      dev->peer_world = world;
      comm_peer_close(dev);
      return false;
    }
    dev->peer_regions[r] = mapped;
  }
  dev->peer_rank = rank;
  dev->peer_world = world;
  dev->peer_ready = true;
  return true;
}

void comm_peer_close(Device* dev) {
  cudaSetDevice(dev->ordinal);
  if (dev->peer_world == 0) {  // exported only
    if (dev->peer_regions[0]) cudaFree(dev->peer_regions[0]);
  } else {
    for (int r = 0; r < dev->peer_world; r++) {
      if (!dev->peer_regions[r]) continue;
      if (r == dev->peer_rank) cudaFree(dev->peer_regions[r]);
      else cudaIpcCloseMemHandle(dev->peer_regions[r]);
    }
  }
  for (void*& p : dev->peer_regions) p = nullptr;
  dev->peer_ready = false;
  dev->peer_world = 0;
}

bool comm_all_reduce_sum(Device* dev, const void* src, void* dst, uint64_t count, int dtype, bool pdl) {
  if (dev->peer_ready && peer_enabled() && dev->peer_world == dev->comm_world &&
      peer_all_reduce_launch(dev->peer_regions, dev->peer_rank, dev->peer_world, dev->peer_slot_bytes, dtype, src, dst, count,
                             dev->error_flag_dev, pdl, dev->stream))
    return true;
  Nccl* api = nccl();
  ncclDataType_t t;
  if (!api || !dev->comm) {
    set_last_error("all_reduce needs an initialised communicator on device %d", dev->ordinal);
    return false;
  }
  if (!nccl_type(dtype, &t)) {
    set_last_error("all_reduce: unsupported element type");
    return false;
  }
  return check_nccl(api, api->AllReduce(src, dst, count, t, ncclSum, (ncclComm_t)dev->comm, dev->stream), "ncclAllReduce");
}

bool comm_all_gather(Device* dev, const void* src, void* dst, uint64_t send_count, int dtype) {
  Nccl* api = nccl();
  ncclDataType_t t;
  if (!api || !dev->comm) {
    set_last_error("all_gather needs an initialised communicator on device %d", dev->ordinal);
    return false;
  }
  if (!nccl_type(dtype, &t)) {
    set_last_error("all_gather: unsupported element type");
    return false;
  }
  return check_nccl(api, api->AllGather(src, dst, send_count, t, (ncclComm_t)dev->comm, dev->stream), "ncclAllGather");
}

void comm_destroy(Device* dev) {
  Nccl* api = nccl();
  if (api && dev->comm) api->CommDestroy((ncclComm_t)dev->comm);
  dev->comm = nullptr;
  dev->comm_world = 1;
  dev->comm_rank = 0;
}

}  // namespace pjrtx

// extern "C" surface declared in include/pjrtx_b200.h. Every body catches all
// exceptions: nothing is thrown across the ABI (the reference wraps every body
// the same way, e.g. src/backend/mlx_metal/api.cc:3391-3497).
#include "../../include/pjrtx_b200.h"

#include <cstring>
#include <new>

#include <chrono>

#include "device.h"
#include "executable_cache.h"
#include "executor.h"
#include "plan.h"
#include "program.h"
#include "sharding.h"
#include "stablehlo_text.h"

using namespace pjrtx;

struct PjrtxB200Buffer {
  Buffer* b;
};
struct PjrtxB200Plan {
  Plan plan;
};
struct PjrtxB200Executable {
  Executable* exe;
};
struct PjrtxB200ExecutableCache {
  ExecutableCache cache;
  uint64_t capacity_bytes;
  explicit PjrtxB200ExecutableCache(uint64_t capacity)
      : cache([](void* h) {
          // Placeholders carry no executable.
          PjrtxB200Executable* w = static_cast<PjrtxB200Executable*>(h);
          if (w->exe) destroy_executable(w->exe);
          delete w;
        }),
        capacity_bytes(capacity) {}
};
struct PjrtxB200ExecutionEvent {
  int device;
  cudaEvent_t event;
};
struct PjrtxB200DeviceEvent {
  int device;
  cudaEvent_t event;
};
struct PjrtxB200AsyncHostToDeviceTransfer {
  int device;
  int dtype;
  std::vector<int64_t> dims;
  std::vector<uint8_t> host;
};

namespace {

uint64_t write_text(const std::string& s, char* out, uint64_t capacity) {
  if (out && capacity) {
    uint64_t n = std::min<uint64_t>(s.size(), capacity - 1);
    memcpy(out, s.data(), n);
    out[n] = 0;
  }
  return s.size();
}

PjrtxB200Buffer* wrap(Buffer* b) {
  if (!b) return nullptr;
  return new PjrtxB200Buffer{b};
}

}  // namespace

#define GUARD_PTR(...)             \
  try {                            \
    __VA_ARGS__                    \
  } catch (const std::exception& e) { \
    set_last_error("%s", e.what()); \
    return nullptr;                \
  } catch (...) {                  \
    set_last_error("unknown error"); \
    return nullptr;                \
  }
#define GUARD_INT(...)             \
  try {                            \
    __VA_ARGS__                    \
  } catch (const std::exception& e) { \
    set_last_error("%s", e.what()); \
    return 0;                      \
  } catch (...) {                  \
    set_last_error("unknown error"); \
    return 0;                      \
  }

extern "C" {

int pjrtx_b200_version_major(void) { return 0; }
int pjrtx_b200_version_minor(void) { return 1; }
int pjrtx_b200_version_patch(void) { return 0; }
const char* pjrtx_b200_last_error(void) { return last_error(); }

int pjrtx_b200_capabilities(PjrtxB200Capabilities* out) {
  if (!out) return 0;
  out->name = "b200_cuda";
  out->supports_device_buffers = 1;
  out->supports_unified_memory = 0;
  out->supports_async_execution = 1;
  return 1;
}

int pjrtx_b200_device_count(void) { GUARD_INT(return device_count();) }

int pjrtx_b200_copy_devices(PjrtxB200DeviceInfo* out_devices, int max_devices) {
  GUARD_INT(
      int n = device_count(); int written = 0;
      for (int i = 0; i < n && written < max_devices && out_devices; i++) {
        Device* d = get_device(i);
        if (!d) continue;
        PjrtxB200DeviceInfo& info = out_devices[written++];
        memset(&info, 0, sizeof info);
        info.ordinal = i;
        info.registry_id = (uint64_t)i;
        info.memory_bytes = d->memory_bytes;
        info.has_unified_memory = 0;
        snprintf(info.name, sizeof info.name, "%s", d->name);
      } return written;)
}

int pjrtx_b200_device_memory_stats(int device_ordinal, PjrtxB200MemoryStats* out) {
  GUARD_INT(Device* d = get_device(device_ordinal); if (!d || !out) return 0; std::lock_guard<std::mutex> lock(d->mu);
            out->bytes_in_use = d->live_bytes; out->peak_bytes_in_use = d->peak_bytes; out->host_to_device_bytes = d->h2d_bytes;
            out->device_to_host_bytes = d->d2h_bytes; return 1;)
}

int pjrtx_b200_device_synchronize(int device_ordinal) {
  GUARD_INT(Device* d = get_device(device_ordinal); if (!d) return 0; cudaSetDevice(d->ordinal);
            if (!check_cuda(cudaStreamSynchronize(d->stream), "cudaStreamSynchronize")) return 0; return check_device_flag(d) ? 1 : 0;)
}

int pjrtx_b200_device_bounded_wait_probe(int device_ordinal, uint32_t timeout_ms) {
  GUARD_INT(Device* d = get_device(device_ordinal); if (!d) return 0; cudaSetDevice(d->ordinal);
            if (!bounded_wait_probe_launch(timeout_ms, d->error_flag_dev, d->stream)) {
              set_last_error("bounded-wait probe refused (timeout must be 1..1000 ms)");
              return 0;
            } return 1;)
}

PjrtxB200DeviceEvent* pjrtx_b200_device_event_record(int device_ordinal) {
  GUARD_PTR(Device* d = get_device(device_ordinal); if (!d) return nullptr; cudaSetDevice(d->ordinal);
            auto* ev = new PjrtxB200DeviceEvent{device_ordinal, nullptr};
            if (!check_cuda(cudaEventCreate(&ev->event), "cudaEventCreate") ||
                !check_cuda(cudaEventRecord(ev->event, d->stream), "cudaEventRecord")) {
              if (ev->event) cudaEventDestroy(ev->event);
              delete ev;
              return nullptr;
            } return ev;)
}

int pjrtx_b200_device_event_elapsed_ms(PjrtxB200DeviceEvent* start, PjrtxB200DeviceEvent* stop, double* out_ms) {
  GUARD_INT(if (!start || !stop || !out_ms) return 0; if (!check_cuda(cudaEventSynchronize(stop->event), "cudaEventSynchronize")) return 0;
            float ms = 0.f; if (!check_cuda(cudaEventElapsedTime(&ms, start->event, stop->event), "cudaEventElapsedTime")) return 0;
            *out_ms = ms; return 1;)
}

void pjrtx_b200_device_event_destroy(PjrtxB200DeviceEvent* event) {
  if (!event) return;
  if (event->event) cudaEventDestroy(event->event);
  delete event;
}

PjrtxB200Buffer* pjrtx_b200_buffer_from_host_typed(int device_ordinal, const void* data, uint64_t byte_size, int dtype,
                                                   const int64_t* dims, uint64_t rank) {
  GUARD_PTR(Device* d = get_device(device_ordinal); if (!d) return nullptr; if (rank && !dims) {
    set_last_error("null dims");
    return nullptr;
  } std::vector<int64_t> dv(dims, dims + rank);
            return wrap(buffer_from_host(d, data, byte_size, dtype, dv));)
}

PjrtxB200Buffer* pjrtx_b200_buffer_zeros(int device_ordinal, int dtype, const int64_t* dims, uint64_t rank) {
  GUARD_PTR(Device* d = get_device(device_ordinal); if (!d) return nullptr; if (rank && !dims) {
    set_last_error("null dims");
    return nullptr;
  } std::vector<int64_t> dv(dims, dims + rank);
            return wrap(buffer_alloc(d, dtype, dv, true));)
}

PjrtxB200Buffer* pjrtx_b200_buffer_clone(PjrtxB200Buffer* src) {
  GUARD_PTR(
      if (!src || !src->b || src->b->donated) {
        set_last_error("buffer is null, deleted or donated");
        return nullptr;
      } Device* d = get_device(src->b->device);
      if (!d) return nullptr; Buffer* b = buffer_alloc(d, src->b->dtype, src->b->dims, false); if (!b) return nullptr;
      if (b->bytes && !check_cuda(cudaMemcpyAsync(b->ptr, src->b->ptr, b->bytes, cudaMemcpyDeviceToDevice, d->stream), "clone")) {
        buffer_free(b);
        return nullptr;
      } return wrap(b);)
}

uint64_t pjrtx_b200_buffer_size(PjrtxB200Buffer* buffer) { return buffer && buffer->b ? buffer->b->bytes : 0; }
int pjrtx_b200_buffer_dtype(PjrtxB200Buffer* buffer) { return buffer && buffer->b ? buffer->b->dtype : 0; }
uint64_t pjrtx_b200_buffer_rank(PjrtxB200Buffer* buffer) { return buffer && buffer->b ? buffer->b->dims.size() : 0; }
int pjrtx_b200_buffer_dims(PjrtxB200Buffer* buffer, int64_t* out_dims, uint64_t max_rank) {
  if (!buffer || !buffer->b || (!out_dims && max_rank)) return 0;
  if (buffer->b->dims.size() > max_rank) return 0;
  for (size_t i = 0; i < buffer->b->dims.size(); i++) out_dims[i] = buffer->b->dims[i];
  return 1;
}
int pjrtx_b200_buffer_device(PjrtxB200Buffer* buffer) { return buffer && buffer->b ? buffer->b->device : -1; }
int pjrtx_b200_buffer_is_donated(PjrtxB200Buffer* buffer) { return buffer && buffer->b && buffer->b->donated ? 1 : 0; }

int pjrtx_b200_buffer_copy_to_host(PjrtxB200Buffer* buffer, void* dst, uint64_t dst_size) {
  GUARD_INT(
      if (!buffer || !buffer->b) {
        set_last_error("null buffer");
        return 0;
      } if (!dst && buffer->b->bytes) {
        set_last_error("null destination");
        return 0;
      } return buffer_to_host(buffer->b, dst, dst_size) ? 1 : 0;)
}

void pjrtx_b200_buffer_destroy(PjrtxB200Buffer* buffer) {
  try {
    if (!buffer) return;
    buffer_free(buffer->b);
    delete buffer;
  } catch (...) {
  }
}

PjrtxB200AsyncHostToDeviceTransfer* pjrtx_b200_async_h2d_create(int device_ordinal, int dtype, const int64_t* dims, uint64_t rank,
                                                                uint64_t byte_size) {
  GUARD_PTR(
      if (!get_device(device_ordinal)) return nullptr; std::vector<int64_t> dv(dims, dims + rank);
      if (dense_byte_size(dtype, dv) != byte_size || dtype_size(dtype) == 0) {
        set_last_error("transfer size does not match its descriptor");
        return nullptr;
      } auto* t = new PjrtxB200AsyncHostToDeviceTransfer{device_ordinal, dtype, dv, std::vector<uint8_t>(byte_size)};
      return t;)
}

int pjrtx_b200_async_h2d_write(PjrtxB200AsyncHostToDeviceTransfer* transfer, uint64_t offset, const void* data, uint64_t byte_size) {
  GUARD_INT(
      if (!transfer || (!data && byte_size) || offset > transfer->host.size() || byte_size > transfer->host.size() - offset) {
        set_last_error("write is outside the transfer");
        return 0;
      } if (byte_size) memcpy(transfer->host.data() + offset, data, byte_size);
      return 1;)
}

PjrtxB200Buffer* pjrtx_b200_async_h2d_finish(PjrtxB200AsyncHostToDeviceTransfer* transfer) {
  GUARD_PTR(if (!transfer) return nullptr; Device* d = get_device(transfer->device); if (!d) return nullptr;
            return wrap(buffer_from_host(d, transfer->host.data(), transfer->host.size(), transfer->dtype, transfer->dims));)
}

void pjrtx_b200_async_h2d_destroy(PjrtxB200AsyncHostToDeviceTransfer* transfer) { delete transfer; }

// ---- plan -------------------------------------------------------------------

PjrtxB200Plan* pjrtx_b200_plan_create(int32_t num_replicas, int32_t num_partitions, const int32_t* device_assignment,
                                      uint64_t device_assignment_count) {
  GUARD_PTR(auto* p = new PjrtxB200Plan(); p->plan.num_replicas = num_replicas; p->plan.num_partitions = num_partitions;
            if (device_assignment) p->plan.device_assignment.assign(device_assignment, device_assignment + device_assignment_count);
            return p;)
}

void pjrtx_b200_plan_destroy(PjrtxB200Plan* plan) { delete plan; }

PjrtxB200Plan* pjrtx_b200_plan_from_stablehlo_text(const char* text, uint64_t length) {
  GUARD_PTR(if (!text) return nullptr; auto p = std::make_unique<PjrtxB200Plan>(); std::string error;
            if (!import_stablehlo_text(std::string(text, length), &p->plan, &error)) {
              set_last_error("%s", error.c_str());
              return nullptr;
            } return p.release();)
}

uint32_t pjrtx_b200_plan_add_value(PjrtxB200Plan* plan, int role, int dtype, const int64_t* dims, uint64_t rank) {
  try {
    if (!plan || (rank && !dims) || role < 0 || role > 3) return UINT32_MAX;
    Value v;
    v.id = (uint32_t)plan->plan.values.size();
    v.role = (ValueRole)role;
    v.dtype = dtype;
    v.dims.assign(dims, dims + rank);
    plan->plan.values.push_back(v);
    if (v.role == ValueRole::parameter) plan->plan.parameter_shardings.push_back(Sharding{});
    return v.id;
  } catch (...) {
    return UINT32_MAX;
  }
}

int pjrtx_b200_plan_add_instruction(PjrtxB200Plan* plan, const char* kind, const uint32_t* inputs, uint64_t input_count,
                                    const uint32_t* outputs, uint64_t output_count, const PjrtxB200Attribute* attributes,
                                    uint64_t attribute_count, const void* literal, uint64_t literal_size,
                                    const char* custom_call_target) {
  GUARD_INT(
      if (!plan || !kind) return 0; Instruction ins; ins.kind = kind_from_name(kind); if (ins.kind == Kind::unsupported) {
        set_last_error("unsupported op: op=%s feature=stablehlo-op", kind);
        return 0;
      } if (inputs) ins.inputs.assign(inputs, inputs + input_count);
      if (outputs) ins.outputs.assign(outputs, outputs + output_count);
      for (uint64_t a = 0; a < attribute_count; a++) {
        if (!attributes[a].name) return 0;
        std::vector<int64_t> vals;
        if (attributes[a].values) vals.assign(attributes[a].values, attributes[a].values + attributes[a].count);
        ins.attrs[attributes[a].name] = vals;
      } if (literal && literal_size) ins.literal.assign((const uint8_t*)literal, (const uint8_t*)literal + literal_size);
      if (custom_call_target) ins.custom_call_target = custom_call_target; plan->plan.instructions.push_back(std::move(ins));
      return 1;)
}

int pjrtx_b200_plan_set_outputs(PjrtxB200Plan* plan, const uint32_t* value_ids, uint64_t count) {
  GUARD_INT(if (!plan || (count && !value_ids)) return 0; plan->plan.output_ids.assign(value_ids, value_ids + count);
            plan->plan.output_shardings.assign(count, Sharding{}); return 1;)
}

static int set_sharding(std::vector<Sharding>& list, uint64_t index, int kind, const char* mesh_name, int64_t split_dim) {
  if (index >= list.size() || kind < 0 || kind > 2) {
    set_last_error("sharding index or kind is out of range");
    return 0;
  }
  list[index].kind = (ShardingKind)kind;
  list[index].mesh_name = mesh_name ? mesh_name : "";
  list[index].split_dim = split_dim;
  return 1;
}

int pjrtx_b200_plan_set_parameter_sharding(PjrtxB200Plan* plan, uint64_t index, int kind, const char* mesh_name, int64_t split_dim) {
  GUARD_INT(if (!plan) return 0; return set_sharding(plan->plan.parameter_shardings, index, kind, mesh_name, split_dim);)
}

int pjrtx_b200_plan_set_output_sharding(PjrtxB200Plan* plan, uint64_t index, int kind, const char* mesh_name, int64_t split_dim) {
  GUARD_INT(if (!plan) return 0; return set_sharding(plan->plan.output_shardings, index, kind, mesh_name, split_dim);)
}

int pjrtx_b200_plan_set_donation(PjrtxB200Plan* plan, const uint32_t* donated, uint64_t donated_count, const uint32_t* alias_outputs,
                                 const uint32_t* alias_parameters, uint64_t alias_count) {
  GUARD_INT(
      if (!plan || (donated_count && !donated) || (alias_count && (!alias_outputs || !alias_parameters))) return 0;
      plan->plan.donated_parameter_indices.assign(donated, donated + donated_count); plan->plan.output_aliases.clear();
      for (uint64_t a = 0; a < alias_count; a++) plan->plan.output_aliases.push_back(OutputAlias{alias_outputs[a], alias_parameters[a], 1});
      return 1;)
}

int pjrtx_b200_plan_verify(PjrtxB200Plan* plan, char* out, uint64_t capacity) {
  GUARD_INT(if (!plan) return 0; std::string msg = verify_plan(plan->plan); if (msg.empty()) {
    write_text("", out, capacity);
    return 1;
  } write_text(msg, out, capacity);
            set_last_error("%s", msg.c_str()); return 0;)
}

uint64_t pjrtx_b200_plan_describe(PjrtxB200Plan* plan, char* out, uint64_t capacity) {
  GUARD_INT(if (!plan) return 0; return write_text(describe_plan(plan->plan), out, capacity);)
}

uint64_t pjrtx_b200_plan_fingerprint(PjrtxB200Plan* plan, char* out, uint64_t capacity) {
  GUARD_INT(if (!plan) return 0; return write_text(plan_fingerprint(plan->plan, "b200_cuda", custom_call_registry_version()), out, capacity);)
}

uint64_t pjrtx_b200_plan_fingerprint_for_devices(PjrtxB200Plan* plan, const int32_t* device_ordinals, uint64_t device_count,
                                                 char* out, uint64_t capacity) {
  GUARD_INT(if (!plan || (device_count && !device_ordinals)) return 0;
            std::vector<int32_t> devs(device_ordinals, device_ordinals + device_count);
            return write_text(plan_fingerprint(plan->plan, "b200_cuda", custom_call_registry_version(), devs), out, capacity);)
}

uint64_t pjrtx_b200_plan_describe_program(PjrtxB200Plan* plan, char* out, uint64_t capacity) {
  GUARD_INT(if (!plan) return 0; std::string msg = verify_plan(plan->plan); if (!msg.empty()) {
    set_last_error("%s", msg.c_str());
    return 0;
  } Program p; std::string err;
            if (!build_program(plan->plan, &p, &err)) {
              set_last_error("%s", err.c_str());
              return 0;
            } return write_text(describe_program(p), out, capacity);)
}

uint64_t pjrtx_b200_plan_describe_kernels(PjrtxB200Plan* plan, char* out, uint64_t capacity) {
  GUARD_INT(if (!plan) return 0; std::string err; std::string text = describe_kernel_plan(plan->plan, &err); if (text.empty()) {
    set_last_error("%s", err.c_str());
    return 0;
  } return write_text(text, out, capacity);)
}

PjrtxB200Plan* pjrtx_b200_plan_partition(PjrtxB200Plan* plan, int32_t partition, int32_t num_partitions) {
  GUARD_PTR(if (!plan) return nullptr; auto* out = new PjrtxB200Plan(); std::string err;
            if (!partition_plan(plan->plan, partition, num_partitions, &out->plan, &err)) {
              set_last_error("%s", err.c_str());
              delete out;
              return nullptr;
            } return out;)
}

// ---- compile / execute --------------------------------------------------------

PjrtxB200Executable* pjrtx_b200_compile_executable(PjrtxB200Plan* plan, const int32_t* device_ordinals, uint64_t device_count) {
  GUARD_PTR(
      if (!plan || (device_count && !device_ordinals)) {
        set_last_error("null plan or device list");
        return nullptr;
      } std::vector<int> devs(device_ordinals, device_ordinals + device_count);
      std::string err; Executable* exe = compile_executable(plan->plan, devs, &err); if (!exe) {
        set_last_error("%s", err.c_str());
        return nullptr;
      } return new PjrtxB200Executable{exe};)
}

uint64_t pjrtx_b200_write_executable_lowering_diagnostic(PjrtxB200Plan* plan, uint64_t device_count, char* out, uint64_t capacity) {
  GUARD_INT(if (!plan) return 0; std::string msg = verify_plan(plan->plan); if (msg.empty()) msg = lowering_diagnostic(plan->plan, device_count);
            return write_text(msg, out, capacity);)
}

int pjrtx_b200_execute_executable(PjrtxB200Executable* executable, uint64_t device_index, PjrtxB200Buffer* const* arguments,
                                  uint64_t argument_count, PjrtxB200Buffer*** out_outputs, uint64_t* out_output_count,
                                  PjrtxB200ExecutionEvent** out_event) {
  GUARD_INT(
      if (out_outputs) *out_outputs = nullptr; if (out_output_count) *out_output_count = 0; if (out_event) *out_event = nullptr;
      if (!executable || !executable->exe || !out_outputs || !out_output_count || (argument_count && !arguments)) {
        set_last_error("null executable, argument list or output slot");
        return 0;
      } std::vector<Buffer*> args(argument_count);
      for (uint64_t i = 0; i < argument_count; i++) {
        if (!arguments[i] || !arguments[i]->b) {
          set_last_error("argument %llu is null", (unsigned long long)i);
          return 0;
        }
        args[i] = arguments[i]->b;
      } std::vector<Buffer*> outs;
      std::string err; if (!execute_executable(executable->exe, device_index, args.data(), args.size(), &outs, &err)) {
        set_last_error("%s", err.c_str());
        return 0;
      } PjrtxB200Buffer** arr = new PjrtxB200Buffer*[outs.size() + 1];
      for (size_t i = 0; i < outs.size(); i++) arr[i] = wrap(outs[i]); arr[outs.size()] = nullptr; *out_outputs = arr;
      *out_output_count = outs.size(); if (out_event) {
        int ordinal = outs.empty() ? (args.empty() ? 0 : args[0]->device) : outs[0]->device;
        Device* d = get_device(ordinal);
        auto* ev = new PjrtxB200ExecutionEvent{ordinal, nullptr};
        if (d && cudaEventCreateWithFlags(&ev->event, cudaEventDisableTiming) == cudaSuccess) cudaEventRecord(ev->event, d->stream);
        *out_event = ev;
      } return 1;)
}

void pjrtx_b200_output_array_destroy(PjrtxB200Buffer** outputs) { delete[] outputs; }

int pjrtx_b200_execution_event_status(PjrtxB200ExecutionEvent* event) {
  if (!event || !event->event) return -1;
  cudaError_t e = cudaEventQuery(event->event);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) return 0;
  set_last_error("execution failed: %s", cudaGetErrorString(e));
  return -1;
}

int pjrtx_b200_execution_event_await(PjrtxB200ExecutionEvent* event) {
  if (!event || !event->event) return 0;
  return check_cuda(cudaEventSynchronize(event->event), "cudaEventSynchronize") ? 1 : 0;
}

void pjrtx_b200_execution_event_destroy(PjrtxB200ExecutionEvent* event) {
  if (!event) return;
  if (event->event) cudaEventDestroy(event->event);
  delete event;
}

int pjrtx_b200_executable_stats(PjrtxB200Executable* executable, PjrtxB200ExecutableStats* out) {
  GUARD_INT(
      if (!executable || !executable->exe || !out) return 0; ExecutableStats s = executable_stats(executable->exe);
      PjrtxB200ExecutableStats r; memset(&r, 0, sizeof r); r.struct_size = sizeof r;
      r.resident_constant_count = s.resident_constant_count; r.resident_constant_bytes = s.resident_constant_bytes;
      r.program_value_count = s.program_value_count; r.program_node_count = s.program_node_count;
      r.program_edge_count = s.program_edge_count; r.program_schedule_item_count = s.program_schedule_item_count;
      r.program_subprogram_count = s.program_subprogram_count; r.program_control_flow_count = s.program_control_flow_count;
      r.program_fusion_group_count = s.program_fusion_group_count;
      r.program_materialization_boundary_count = s.program_materialization_boundary_count;
      r.program_planned_release_count = s.program_planned_release_count; r.program_planned_release_bytes = s.program_planned_release_bytes;
      r.program_peak_live_value_count = s.program_peak_live_value_count; r.program_peak_live_bytes = s.program_peak_live_bytes;
      r.program_device_count = s.program_device_count; r.last_execute_device_index = s.last_execute_device_index;
      r.last_execute_local_hardware_id = s.last_execute_local_hardware_id; r.execute_count = s.execute_count;
      r.compiled_program_execute_count = s.compiled_program_execute_count; r.compiled_program_output_count = s.compiled_program_output_count;
      r.captured_program_execute_count = s.captured_program_execute_count;
      r.captured_program_dynamic_input_count = s.captured_program_dynamic_input_count;
      r.captured_program_captured_input_count = s.captured_program_captured_input_count;
      r.donation_alias_output_count = s.donation_alias_output_count; r.donation_alias_output_bytes = s.donation_alias_output_bytes;
      r.fusion_group_execute_count = s.fusion_group_execute_count; r.execute_wall_us_total = s.execute_wall_us_total;
      r.execute_wall_us_peak = s.execute_wall_us_peak; r.kernel_step_count = s.kernel_step_count;
      r.generated_kernel_count = s.generated_kernel_count; r.arena_bytes = s.arena_bytes; r.scratch_bytes = s.scratch_bytes;
      r.graph_capture_count = s.graph_capture_count; r.graph_launch_count = s.graph_launch_count;
      r.kernel_launch_total = s.kernel_launch_total;
      r.profile_event_gap_ns = s.profile_event_gap_ns;
      uint64_t n = out->struct_size ? std::min<uint64_t>(out->struct_size, sizeof r) : sizeof r; memcpy(out, &r, n); return 1;)
}

int pjrtx_b200_executable_set_profiling(PjrtxB200Executable* executable, int enabled) {
  GUARD_INT(if (!executable || !executable->exe) return 0; executable_set_profiling(executable->exe, enabled != 0); return 1;)
}

uint64_t pjrtx_b200_executable_step_times(PjrtxB200Executable* executable, float* out_ms, uint64_t capacity) {
  GUARD_INT(if (!executable || !executable->exe) return 0; std::vector<float> t = executable_step_times(executable->exe);
            for (uint64_t k = 0; k < t.size() && k < capacity && out_ms; k++) out_ms[k] = t[k]; return t.size();)
}

uint64_t pjrtx_b200_executable_describe(PjrtxB200Executable* executable, char* out, uint64_t capacity) {
  GUARD_INT(if (!executable || !executable->exe) return 0; return write_text(executable_describe(executable->exe), out, capacity);)
}

void pjrtx_b200_executable_destroy(PjrtxB200Executable* executable) {
  try {
    if (!executable) return;
    destroy_executable(executable->exe);
    delete executable;
  } catch (...) {
  }
}

// ---- resident-executable cache -------------------------------------------------

namespace {

void fill_trim(const CacheTrim& t, PjrtxB200ExecutableCacheTrim* out) {
  if (!out) return;
  out->requested_bytes = t.requested_bytes;
  out->target_resident_bytes = t.target_resident_bytes;
  out->freed_bytes = t.freed_bytes;
  out->evicted_entries = t.evicted_entries;
  out->remaining_resident_bytes = t.remaining_resident_bytes;
  out->still_over_capacity = t.still_over_capacity ? 1 : 0;
}

}  // namespace

PjrtxB200ExecutableCache* pjrtx_b200_executable_cache_create(uint64_t capacity_bytes) {
  GUARD_PTR(return new PjrtxB200ExecutableCache(capacity_bytes);)
}

void pjrtx_b200_executable_cache_destroy(PjrtxB200ExecutableCache* cache) {
  try {
    delete cache;
  } catch (...) {
  }
}

int pjrtx_b200_executable_cache_record_compile(PjrtxB200ExecutableCache* cache, const char* fingerprint) {
  try {
    if (!cache || !fingerprint) {
      set_last_error("null cache or fingerprint");
      return -1;
    }
    return cache->cache.record_compile(fingerprint) ? 1 : 0;
  } catch (const std::exception& e) {
    set_last_error("%s", e.what());
    return -1;
  } catch (...) {
    set_last_error("unknown error");
    return -1;
  }
}

PjrtxB200Executable* pjrtx_b200_executable_cache_acquire(PjrtxB200ExecutableCache* cache, const char* fingerprint,
                                                         PjrtxB200Plan* plan, const int32_t* device_ordinals,
                                                         uint64_t device_count, int* out_reused,
                                                         PjrtxB200ExecutableCacheTrim* out_compile_trim) {
  GUARD_PTR(
      if (out_reused) *out_reused = 0; fill_trim(CacheTrim{}, out_compile_trim);
      if (!cache || !fingerprint || !plan || (device_count && !device_ordinals)) {
        set_last_error("null cache, fingerprint, plan or device list");
        return nullptr;
      } CacheEntrySnapshot snap;
      if (!cache->cache.entry(fingerprint, &snap)) {
        set_last_error("fingerprint %s was not recorded", fingerprint);
        return nullptr;
      } std::vector<int> devs(device_ordinals, device_ordinals + device_count);
      if (void* h = cache->cache.retain_resident(fingerprint)) {
        // A key that does not cover the target devices would hand out an executable of another GPU: refuse it.
        PjrtxB200Executable* held = static_cast<PjrtxB200Executable*>(h);
        if (held->exe && executable_device_ordinals(held->exe) != devs) {
          cache->cache.release(fingerprint);
          set_last_error("fingerprint %s is resident for other devices; key the request with pjrtx_b200_plan_fingerprint_for_devices",
                         fingerprint);
          return nullptr;
        }
        if (out_reused) *out_reused = 1;
        return held;
      }
      std::string err; auto t0 = std::chrono::steady_clock::now(); Executable* exe = compile_executable(plan->plan, devs, &err);
      if (!exe) {
        set_last_error("%s", err.c_str());
        return nullptr;
      } const uint64_t latency_us =
          (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
      ExecutableStats st = executable_stats(exe);
      const uint64_t resident = st.resident_constant_bytes + st.arena_bytes + st.scratch_bytes;
      // Buffer bytes outside the cache: the device counts every allocation, the executables' included.
      uint64_t in_use = 0; if (Device* d = devs.empty() ? nullptr : get_device(devs[0])) {
        std::lock_guard<std::mutex> lock(d->mu);
        const uint64_t held = cache->cache.stats().resident_bytes + resident;
        in_use = d->live_bytes > held ? d->live_bytes - held : 0;
      } bool reused = false;
      CacheTrim trim; void* h = cache->cache.install(fingerprint, new PjrtxB200Executable{exe}, resident, latency_us,
                                                     cache->capacity_bytes, in_use, &reused, &trim);
      if (out_reused) *out_reused = reused ? 1 : 0; fill_trim(trim, out_compile_trim);
      return static_cast<PjrtxB200Executable*>(h);)
}

void pjrtx_b200_executable_cache_release(PjrtxB200ExecutableCache* cache, const char* fingerprint) {
  try {
    if (cache && fingerprint) cache->cache.release(fingerprint);
  } catch (...) {
  }
}

void pjrtx_b200_executable_cache_set_max_resident_bytes(PjrtxB200ExecutableCache* cache, uint64_t max_resident_bytes) {
  try {
    if (cache) cache->cache.set_max_resident_bytes(max_resident_bytes);
  } catch (...) {
  }
}

void pjrtx_b200_executable_cache_set_capacity(PjrtxB200ExecutableCache* cache, uint64_t capacity_bytes) {
  if (cache) cache->capacity_bytes = capacity_bytes;
}

int pjrtx_b200_executable_cache_trim_for_allocation(PjrtxB200ExecutableCache* cache, uint64_t bytes_in_use,
                                                    uint64_t allocation_bytes, PjrtxB200ExecutableCacheTrim* out) {
  GUARD_INT(if (!cache) return 0;
            fill_trim(cache->cache.trim_for_allocation(cache->capacity_bytes, bytes_in_use, allocation_bytes), out); return 1;)
}

int pjrtx_b200_executable_cache_stats(PjrtxB200ExecutableCache* cache, PjrtxB200ExecutableCacheStats* out) {
  GUARD_INT(if (!cache || !out) return 0; CacheStats s = cache->cache.stats(); out->hits = s.hits; out->misses = s.misses;
            out->evictions = s.evictions; out->evicted_resident_bytes = s.evicted_resident_bytes;
            out->resident_entries = s.resident_entries; out->resident_bytes = s.resident_bytes;
            out->peak_resident_bytes = s.peak_resident_bytes; out->largest_resident_bytes = s.largest_resident_bytes;
            out->compile_latency_samples = s.compile_latency_samples; out->compile_latency_us_total = s.compile_latency_us_total;
            out->compile_latency_us_peak = s.compile_latency_us_peak; out->pressure_trim_requests = s.pressure_trim_requests;
            out->pressure_trimmed_bytes = s.pressure_trimmed_bytes; out->pressure_trim_failures = s.pressure_trim_failures;
            return 1;)
}

int pjrtx_b200_executable_cache_entry(PjrtxB200ExecutableCache* cache, const char* fingerprint,
                                      PjrtxB200ExecutableCacheEntry* out) {
  GUARD_INT(if (!cache || !fingerprint) return 0; CacheEntrySnapshot s; if (!cache->cache.entry(fingerprint, &s)) return 0;
            if (out) {
              out->resident = s.resident ? 1 : 0;
              out->resident_bytes = s.resident_bytes;
              out->reference_count = s.reference_count;
              out->compile_latency_us = s.compile_latency_us;
            } return 1;)
}

int pjrtx_b200_executable_cache_install_placeholder(PjrtxB200ExecutableCache* cache, const char* fingerprint,
                                                    uint64_t resident_bytes, uint64_t bytes_in_use,
                                                    PjrtxB200ExecutableCacheTrim* out_compile_trim) {
  GUARD_INT(fill_trim(CacheTrim{}, out_compile_trim); if (!cache || !fingerprint) return 0;
            if (cache->cache.retain_resident(fingerprint)) return 2;
            bool reused = false; CacheTrim trim;
            void* h = cache->cache.install(fingerprint, new PjrtxB200Executable{nullptr}, resident_bytes, 0,
                                           cache->capacity_bytes, bytes_in_use, &reused, &trim);
            fill_trim(trim, out_compile_trim); if (!h) {
              set_last_error("fingerprint %s was not recorded", fingerprint);
              return 0;
            } return reused ? 2 : 1;)
}

void pjrtx_b200_executable_cache_set_compile_latency(PjrtxB200ExecutableCache* cache, const char* fingerprint,
                                                     uint64_t latency_us) {
  try {
    if (cache && fingerprint) cache->cache.set_compile_latency(fingerprint, latency_us);
  } catch (...) {
  }
}

int pjrtx_b200_register_custom_call(const char* target, const char* op_name, int arity) {
  GUARD_INT(if (!target || !op_name) return 0; if (!register_custom_call(target, op_name, arity)) {
    set_last_error("custom call %s cannot lower to %s", target, op_name);
    return 0;
  } return 1;)
}

void pjrtx_b200_unregister_custom_call(const char* target) {
  try {
    if (target) unregister_custom_call(target);
  } catch (...) {
  }
}

uint64_t pjrtx_b200_custom_call_registry_version(void) { return custom_call_registry_version(); }

int pjrtx_b200_comm_unique_id(uint8_t out_id[128]) { GUARD_INT(if (!out_id) return 0; return comm_unique_id(out_id) ? 1 : 0;) }

int pjrtx_b200_comm_init(int device_ordinal, const uint8_t id[128], int rank, int world_size) {
  GUARD_INT(Device* d = get_device(device_ordinal); if (!d || !id) return 0; return comm_init(d, id, rank, world_size) ? 1 : 0;)
}

int pjrtx_b200_comm_peer_export(int device_ordinal, uint8_t out_handle[64]) {
  GUARD_INT(Device* d = get_device(device_ordinal); if (!d || !out_handle) return 0; return comm_peer_export(d, out_handle) ? 1 : 0;)
}

int pjrtx_b200_comm_peer_import(int device_ordinal, const uint8_t* handles, int rank, int world_size) {
  GUARD_INT(Device* d = get_device(device_ordinal); if (!d || !handles) return 0; return comm_peer_import(d, handles, rank, world_size) ? 1 : 0;)
}

void pjrtx_b200_comm_destroy(int device_ordinal) {
  try {
    Device* d = get_device(device_ordinal);
    if (d) {
      comm_peer_close(d);
      comm_destroy(d);
    }
  } catch (...) {
  }
}

int pjrtx_b200_dot_static_scratch(int device_ordinal, int dtype, const void* lhs, const void* rhs, void* out, int64_t m, int64_t k,
                                  int64_t n, void* stream) {
  GUARD_INT(return stream_dot_static_scratch(device_ordinal, dtype, lhs, rhs, out, m, k, n, (cudaStream_t)stream);)
}

int pjrtx_b200_dot_static_scratch_status(int device_ordinal, void* stream) {
  GUARD_INT(return stream_dot_static_scratch_status(device_ordinal, (cudaStream_t)stream);)
}

int pjrtx_b200_compile_check(const char* source, char* out, uint64_t capacity) {
  GUARD_INT(if (!source) return 0; std::vector<char> cubin; std::string log; bool ok = jit_compile_cubin(source, &cubin, &log);
            write_text(log, out, capacity); if (!ok) set_last_error("%s", log.c_str()); return ok ? 1 : 0;)
}

}  // extern "C"

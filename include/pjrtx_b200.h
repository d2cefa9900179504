/* C ABI of the B200 execution backend for PjRTx.
 *
 * This is the boundary a PjRTx runtime binds instead of the Zig `Backend`
 * facade of the Metal backend (src/backend/mlx_metal/backend.zig:91-180) and
 * the private C shim under it (src/backend/mlx_metal/api.h:198-477). Every
 * entry point below names the reference interface it replaces.
 *
 * Conventions (the same as src/backend/mlx_metal/api.cc): functions that return
 * a pointer return NULL on any failure and never throw across the ABI;
 * functions that return int return 1 on success and 0 on failure; after a
 * failure pjrtx_b200_last_error() holds a one-line reason for the calling
 * thread. Arrays returned through `out_outputs` are owned by the caller and
 * released with pjrtx_b200_output_array_destroy (the array) and
 * pjrtx_b200_buffer_destroy (each element). Element-type codes equal the
 * reference's (api.h:107-120); 12..14 are additions.
 */
#ifndef PJRTX_B200_H_
#define PJRTX_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PJRTX_B200_DEVICE_NAME_BYTES 128

enum {
  PJRTX_B200_DTYPE_INVALID = 0,
  PJRTX_B200_DTYPE_U8 = 1,
  PJRTX_B200_DTYPE_F32 = 2,
  PJRTX_B200_DTYPE_PRED = 3,
  PJRTX_B200_DTYPE_S32 = 4,
  PJRTX_B200_DTYPE_U32 = 5,
  PJRTX_B200_DTYPE_S8 = 6,
  PJRTX_B200_DTYPE_F16 = 7,
  PJRTX_B200_DTYPE_BF16 = 8,
  PJRTX_B200_DTYPE_C64 = 9,
  PJRTX_B200_DTYPE_U16 = 10,
  PJRTX_B200_DTYPE_U64 = 11,
  PJRTX_B200_DTYPE_S64 = 12,
  PJRTX_B200_DTYPE_S16 = 13,
  PJRTX_B200_DTYPE_F64 = 14,
};

/* Value roles (src/compiler/executable_plan.zig:17-22). */
enum {
  PJRTX_B200_ROLE_PARAMETER = 0,
  PJRTX_B200_ROLE_CONSTANT = 1,
  PJRTX_B200_ROLE_INSTRUCTION_RESULT = 2,
  PJRTX_B200_ROLE_OUTPUT = 3,
};

/* Sharding kinds (src/compiler/topology.zig:69-73). */
enum {
  PJRTX_B200_SHARDING_REPLICATED = 0,
  PJRTX_B200_SHARDING_PARTITIONED = 1,
  PJRTX_B200_SHARDING_MANUAL = 2,
};

/* Compare directions (src/compiler/operation.zig:46-53, api.h:181-188). */
enum {
  PJRTX_B200_COMPARE_EQ = 0,
  PJRTX_B200_COMPARE_NE = 1,
  PJRTX_B200_COMPARE_GE = 2,
  PJRTX_B200_COMPARE_GT = 3,
  PJRTX_B200_COMPARE_LE = 4,
  PJRTX_B200_COMPARE_LT = 5,
};

typedef struct PjrtxB200Buffer PjrtxB200Buffer;
typedef struct PjrtxB200Plan PjrtxB200Plan;
typedef struct PjrtxB200Executable PjrtxB200Executable;
typedef struct PjrtxB200ExecutionEvent PjrtxB200ExecutionEvent;
typedef struct PjrtxB200AsyncHostToDeviceTransfer PjrtxB200AsyncHostToDeviceTransfer;
typedef struct PjrtxB200DeviceEvent PjrtxB200DeviceEvent;

/* Replaces PjrtxMlxMetalDeviceInfo (api.h:12-18). */
typedef struct PjrtxB200DeviceInfo {
  int32_t ordinal;
  uint64_t registry_id;
  uint64_t memory_bytes;
  uint8_t has_unified_memory;
  char name[PJRTX_B200_DEVICE_NAME_BYTES];
} PjrtxB200DeviceInfo;

/* Replaces device.Capabilities (src/backend/mlx_metal/device.zig:7-25). */
typedef struct PjrtxB200Capabilities {
  const char *name; /* "b200_cuda" */
  uint8_t supports_device_buffers;
  uint8_t supports_unified_memory;
  uint8_t supports_async_execution;
} PjrtxB200Capabilities;

/* One integer-list attribute of an instruction, named as the field of
 * ir.PlanInstruction it stands for (src/compiler/executable_plan.zig:56-128):
 * "dims", "permutation", "broadcast_dimensions", "start_indices",
 * "limit_indices", "strides", "slice_sizes", "dimension", "dimensions",
 * "iota_dimension", "reduce_dimensions", "lhs_batch_dimensions",
 * "rhs_batch_dimensions", "lhs_contracting_dimensions",
 * "rhs_contracting_dimensions", "compare_direction", "index_vector_dim",
 * "offset_dims", "collapsed_slice_dims", "start_index_map",
 * "operand_batching_dims", "start_indices_batching_dims". */
typedef struct PjrtxB200Attribute {
  const char *name;
  const int64_t *values;
  uint64_t count;
} PjrtxB200Attribute;

/* Replaces executable_mod.Stats (src/backend/mlx_metal/executable_stats.zig:6-56);
 * fields that only describe MLX/Metal strategies are dropped, kernel-plan
 * counters are added at the end. */
typedef struct PjrtxB200ExecutableStats {
  uint64_t struct_size;
  uint64_t resident_constant_count;
  uint64_t resident_constant_bytes;
  uint64_t program_value_count;
  uint64_t program_node_count;
  uint64_t program_edge_count;
  uint64_t program_schedule_item_count;
  uint64_t program_subprogram_count;
  uint64_t program_control_flow_count;
  uint64_t program_fusion_group_count;
  uint64_t program_materialization_boundary_count;
  uint64_t program_planned_release_count;
  uint64_t program_planned_release_bytes;
  uint64_t program_peak_live_value_count;
  uint64_t program_peak_live_bytes;
  uint64_t program_device_count;
  uint64_t last_execute_device_index; /* UINT64_MAX before the first execute */
  int32_t last_execute_local_hardware_id; /* -1 before the first execute */
  uint64_t execute_count;
  uint64_t compiled_program_execute_count;
  uint64_t compiled_program_output_count;
  uint64_t captured_program_execute_count;
  uint64_t captured_program_dynamic_input_count;
  uint64_t captured_program_captured_input_count;
  uint64_t donation_alias_output_count;
  uint64_t donation_alias_output_bytes;
  uint64_t fusion_group_execute_count;
  uint64_t execute_wall_us_total;
  uint64_t execute_wall_us_peak;
  uint64_t kernel_step_count;
  uint64_t generated_kernel_count;
  uint64_t arena_bytes;
  uint64_t scratch_bytes;
  uint64_t graph_capture_count;
  uint64_t graph_launch_count;
  uint64_t kernel_launch_total;
  uint64_t profile_event_gap_ns; /* profiled executions: what two event records with nothing between them read */
} PjrtxB200ExecutableStats;

/* Replaces MemoryStats (src/runtime/device_memory.zig:258-304). */
typedef struct PjrtxB200MemoryStats {
  uint64_t bytes_in_use;
  uint64_t peak_bytes_in_use;
  uint64_t host_to_device_bytes;
  uint64_t device_to_host_bytes;
} PjrtxB200MemoryStats;

/* ---- library ----------------------------------------------------------- */
/* api.h:198-201 pjrtx_mlx_metal_version_{major,minor,patch}. */
int pjrtx_b200_version_major(void);
int pjrtx_b200_version_minor(void);
int pjrtx_b200_version_patch(void);
/* pjrtx_metalcpp_last_error (api.h:283). */
const char *pjrtx_b200_last_error(void);
/* Backend.capabilities (backend.zig:92). */
int pjrtx_b200_capabilities(PjrtxB200Capabilities *out);

/* ---- devices ----------------------------------------------------------- */
/* pjrtx_mlx_metal_device_count / copy_devices (api.h:202-204); Backend.enumerateDevices (backend.zig:94-98). */
int pjrtx_b200_device_count(void);
int pjrtx_b200_copy_devices(PjrtxB200DeviceInfo *out_devices, int max_devices);
/* PJRT_Device_MemoryStats source (src/plugin/device_memory.zig:273-309). */
int pjrtx_b200_device_memory_stats(int device_ordinal, PjrtxB200MemoryStats *out);
/* Blocks until everything queued on the device's stream is done (mlx synchronize, api.cc:1512-1520). */
int pjrtx_b200_device_synchronize(int device_ordinal);
/* No counterpart in the reference (its failure tests overwrite buffer readiness on the host,
 * src/runtime/execution_call.zig:355-360). Exercises the path by which a device-side wait that cannot complete is
 * reported: enqueues one CTA that waits, with the bounded wait of the streaming kernels, for a barrier nothing ever
 * completes; after `timeout_ms` (1..1000) it gives up, raises the device's error word (code 31) and returns. The next
 * pjrtx_b200_device_synchronize then returns 0 with "gave up a bounded wait (code 31)" and clears the word; the
 * context stays usable. 1 when enqueued. */
int pjrtx_b200_device_bounded_wait_probe(int device_ordinal, uint32_t timeout_ms);

/* Device-side timing on the stream every buffer and executable of the device uses. The reference measures the same
 * interval on the host around a forced device sync (PJRTX_PROFILE_DEVICE_SYNC, src/backend/mlx_metal/api.cc:65-75,
 * PjrtxMlxMetalProgramExecuteProfile.device_sync_wait_us, api.h:25-32). `record` enqueues an event; `elapsed_ms`
 * waits for `stop` and returns the device time between the two. */
PjrtxB200DeviceEvent *pjrtx_b200_device_event_record(int device_ordinal);
int pjrtx_b200_device_event_elapsed_ms(PjrtxB200DeviceEvent *start, PjrtxB200DeviceEvent *stop, double *out_ms);
void pjrtx_b200_device_event_destroy(PjrtxB200DeviceEvent *event);

/* ---- buffers ----------------------------------------------------------- */
/* pjrtx_mlx_metal_buffer_from_host_typed (api.h:208-211); Backend.bufferFromHost (backend.zig:104-106).
 * The host memory may be reused as soon as the call returns. */
PjrtxB200Buffer *pjrtx_b200_buffer_from_host_typed(int device_ordinal, const void *data, uint64_t byte_size, int dtype,
                                                   const int64_t *dims, uint64_t rank);
/* pjrtx_mlx_metal_buffer_zeros (api.h:223-225); Backend.allocateBuffer (backend.zig:124-126). */
PjrtxB200Buffer *pjrtx_b200_buffer_zeros(int device_ordinal, int dtype, const int64_t *dims, uint64_t rank);
/* pjrtx_mlx_metal_buffer_clone (api.h:233); Backend.cloneBuffer (backend.zig:128). */
PjrtxB200Buffer *pjrtx_b200_buffer_clone(PjrtxB200Buffer *src);
/* pjrtx_mlx_metal_buffer_size (api.h:447). */
uint64_t pjrtx_b200_buffer_size(PjrtxB200Buffer *buffer);
int pjrtx_b200_buffer_dtype(PjrtxB200Buffer *buffer);
uint64_t pjrtx_b200_buffer_rank(PjrtxB200Buffer *buffer);
int pjrtx_b200_buffer_dims(PjrtxB200Buffer *buffer, int64_t *out_dims, uint64_t max_rank);
int pjrtx_b200_buffer_device(PjrtxB200Buffer *buffer);
/* 1 when the buffer's storage was moved into an execution output (donation). */
int pjrtx_b200_buffer_is_donated(PjrtxB200Buffer *buffer);
/* pjrtx_mlx_metal_buffer_copy_to_host (api.h:452-453); Backend.copyToHost (backend.zig:177). Synchronous. */
int pjrtx_b200_buffer_copy_to_host(PjrtxB200Buffer *buffer, void *dst, uint64_t dst_size);
/* pjrtx_mlx_metal_buffer_destroy (api.h:454); Backend.destroyBuffer (backend.zig:179). */
void pjrtx_b200_buffer_destroy(PjrtxB200Buffer *buffer);

/* pjrtx_mlx_metal_async_h2d_{create,write,finish,destroy} (api.h:212-222);
 * Backend.{begin,write,finish,destroy}AsyncHostToDeviceTransfer (backend.zig:108-122). */
PjrtxB200AsyncHostToDeviceTransfer *pjrtx_b200_async_h2d_create(int device_ordinal, int dtype, const int64_t *dims,
                                                                uint64_t rank, uint64_t byte_size);
int pjrtx_b200_async_h2d_write(PjrtxB200AsyncHostToDeviceTransfer *transfer, uint64_t offset, const void *data,
                               uint64_t byte_size);
PjrtxB200Buffer *pjrtx_b200_async_h2d_finish(PjrtxB200AsyncHostToDeviceTransfer *transfer);
void pjrtx_b200_async_h2d_destroy(PjrtxB200AsyncHostToDeviceTransfer *transfer);

/* ---- executable plan ---------------------------------------------------- */
/* The plan is the reference's ir.ExecutablePlan (src/compiler/executable_plan.zig:131-147)
 * built field by field, the way the reference's own backend tests build one
 * (src/backend/mlx_metal/execution_call.zig:147-211). */
PjrtxB200Plan *pjrtx_b200_plan_create(int32_t num_replicas, int32_t num_partitions, const int32_t *device_assignment,
                                      uint64_t device_assignment_count);
void pjrtx_b200_plan_destroy(PjrtxB200Plan *plan);
/* Appends a value; returns its id (== table index) or UINT32_MAX. */
uint32_t pjrtx_b200_plan_add_value(PjrtxB200Plan *plan, int role, int dtype, const int64_t *dims, uint64_t rank);
/* Appends an instruction. `kind` is the reference's PlanInstructionKind tag name
 * (src/compiler/operation.zig:84-168), e.g. "add", "dot_general", "reduce_sum";
 * "all_reduce" / "all_gather" are the collective kinds the tensor-parallel planner adds. */
int pjrtx_b200_plan_add_instruction(PjrtxB200Plan *plan, const char *kind, const uint32_t *inputs, uint64_t input_count,
                                    const uint32_t *outputs, uint64_t output_count, const PjrtxB200Attribute *attributes,
                                    uint64_t attribute_count, const void *literal, uint64_t literal_size,
                                    const char *custom_call_target);
int pjrtx_b200_plan_set_outputs(PjrtxB200Plan *plan, const uint32_t *value_ids, uint64_t count);
/* Sharding of parameter `index` (in parameter order) / output `index`; split_dim = -1 when replicated. */
int pjrtx_b200_plan_set_parameter_sharding(PjrtxB200Plan *plan, uint64_t index, int kind, const char *mesh_name,
                                           int64_t split_dim);
int pjrtx_b200_plan_set_output_sharding(PjrtxB200Plan *plan, uint64_t index, int kind, const char *mesh_name,
                                        int64_t split_dim);
/* donated_parameter_indices and output_aliases (executable_plan.zig:143-144). */
int pjrtx_b200_plan_set_donation(PjrtxB200Plan *plan, const uint32_t *donated_parameter_indices, uint64_t donated_count,
                                 const uint32_t *alias_output_indices, const uint32_t *alias_parameter_indices,
                                 uint64_t alias_count);
/* verifyExecutablePlan (src/compiler/executable_plan_verify.zig:328-449): 1 when valid; otherwise writes the
 * diagnostic line into `out` (truncated to capacity, always NUL terminated) and returns 0. */
int pjrtx_b200_plan_verify(PjrtxB200Plan *plan, char *out, uint64_t capacity);
/* The plan itself as JSON (values, instructions, attributes, constant payloads in hex, shardings, outputs): the
 * inverse of the builder calls above, used to inspect what pjrtx_b200_plan_partition produced. Returns the full length. */
uint64_t pjrtx_b200_plan_describe(PjrtxB200Plan *plan, char *out, uint64_t capacity);
/* Stable cache key of the plan under the current backend state ("pjrtx-<16 hex digits>"): the fields the reference's
 * executable cache hashes (src/runtime/executable_fingerprint.zig:9-140: capabilities name, custom-call registry
 * version, compile options, shardings, donation, values, instructions with attributes, constants, call targets). A host
 * keeps compiled executables under this key. Same text-out convention as plan_describe. */
uint64_t pjrtx_b200_plan_fingerprint(PjrtxB200Plan *plan, char *out, uint64_t capacity);
/* The same key with the target devices mixed in, as the reference hashes the resolved device ids and local hardware ids
 * of the executable's devices (src/runtime/executable_fingerprint.zig:38-56): the key to use with the executable cache,
 * whose acquire refuses a resident executable that was compiled for other devices. */
uint64_t pjrtx_b200_plan_fingerprint_for_devices(PjrtxB200Plan *plan, const int32_t *device_ordinals, uint64_t device_count,
                                                 char *out, uint64_t capacity);
/* Backend program graph (nodes, edges, fusion groups, schedule, liveness) as JSON; needs no device.
 * Returns the full length; writes at most capacity-1 bytes. program_build.build (program_build.zig:10-207). */
uint64_t pjrtx_b200_plan_describe_program(PjrtxB200Plan *plan, char *out, uint64_t capacity);
/* Kernel plan (steps, generated sources, arena size) as JSON; needs no device. 0 on failure. */
uint64_t pjrtx_b200_plan_describe_kernels(PjrtxB200Plan *plan, char *out, uint64_t capacity);
/* Tensor-parallel planner: rewrites a full-size plan whose parameter shardings carry split dimensions into the
 * per-partition plan of `partition` (column/row-parallel contractions, all_reduce after row-parallel ones).
 * New capability on top of the reference's sharding metadata (src/compiler/stablehlo_sharding.zig:40-93). */
PjrtxB200Plan *pjrtx_b200_plan_partition(PjrtxB200Plan *plan, int32_t partition, int32_t num_partitions);

/* ---- compile / execute --------------------------------------------------- */
/* Backend.compileExecutable (backend.zig:130-132). */
PjrtxB200Executable *pjrtx_b200_compile_executable(PjrtxB200Plan *plan, const int32_t *device_ordinals,
                                                   uint64_t device_count);
/* Backend.writeExecutableLoweringDiagnostic (backend.zig:134-136). Returns the full length (0 = no issue). */
uint64_t pjrtx_b200_write_executable_lowering_diagnostic(PjrtxB200Plan *plan, uint64_t device_count, char *out,
                                                         uint64_t capacity);
/* Backend.executeExecutable (backend.zig:138-140); output ownership as pjrtx_mlx_metal_program_execute (api.h:464-476).
 * `out_event` may be NULL. */
int pjrtx_b200_execute_executable(PjrtxB200Executable *executable, uint64_t device_index, PjrtxB200Buffer *const *arguments,
                                  uint64_t argument_count, PjrtxB200Buffer ***out_outputs, uint64_t *out_output_count,
                                  PjrtxB200ExecutionEvent **out_event);
/* pjrtx_mlx_metal_program_output_array_destroy (api.h:477). Frees the array, not the buffers. */
void pjrtx_b200_output_array_destroy(PjrtxB200Buffer **outputs);
/* Backend.executionEventStatus / destroyExecutionEvent (backend.zig:142-144): 0 pending, 1 complete, -1 failed. */
int pjrtx_b200_execution_event_status(PjrtxB200ExecutionEvent *event);
int pjrtx_b200_execution_event_await(PjrtxB200ExecutionEvent *event);
void pjrtx_b200_execution_event_destroy(PjrtxB200ExecutionEvent *event);
/* Backend.executableStats (backend.zig:146). Set out->struct_size before the call. */
int pjrtx_b200_executable_stats(PjrtxB200Executable *executable, PjrtxB200ExecutableStats *out);
uint64_t pjrtx_b200_executable_describe(PjrtxB200Executable *executable, char *out, uint64_t capacity);
/* Per-step device times (the reference's `backend_schedule_item` profile events, src/backend/mlx_metal/
 * profiling_writer.zig:160). While enabled, executions run the step list without graph replay and time every step
 * with a CUDA event pair; step_times copies the latest execution's durations (ms, step order) and returns the
 * step count. */
int pjrtx_b200_executable_set_profiling(PjrtxB200Executable *executable, int enabled);
uint64_t pjrtx_b200_executable_step_times(PjrtxB200Executable *executable, float *out_ms, uint64_t capacity);
/* Backend.destroyExecutable (backend.zig:148). */
void pjrtx_b200_executable_destroy(PjrtxB200Executable *executable);

/* ---- resident-executable cache ----------------------------------------------- */
/* Replaces the runtime's executable residency (src/runtime/executable_cache.zig): compile requests are keyed by
 * fingerprint (pjrtx_b200_plan_fingerprint), a compiled executable stays resident while leased and afterwards until
 * the byte budget or a memory-pressure trim needs its device memory. Victim order among idle entries: most resident
 * bytes, then cheapest to compile, then least recently used, then smaller fingerprint (:284-313). An executable's
 * resident bytes are the device memory it owns (resident constants + arena + contraction scratch). */
typedef struct PjrtxB200ExecutableCache PjrtxB200ExecutableCache;

/* executable_cache.Stats (src/runtime/executable_cache.zig:10-25). */
typedef struct PjrtxB200ExecutableCacheStats {
  uint64_t hits;
  uint64_t misses;
  uint64_t evictions;
  uint64_t evicted_resident_bytes;
  uint64_t resident_entries;
  uint64_t resident_bytes;
  uint64_t peak_resident_bytes;
  uint64_t largest_resident_bytes;
  uint64_t compile_latency_samples;
  uint64_t compile_latency_us_total;
  uint64_t compile_latency_us_peak;
  uint64_t pressure_trim_requests;
  uint64_t pressure_trimmed_bytes;
  uint64_t pressure_trim_failures;
} PjrtxB200ExecutableCacheStats;

/* executable_cache.Trim (:66-73). */
typedef struct PjrtxB200ExecutableCacheTrim {
  uint64_t requested_bytes;
  uint64_t target_resident_bytes;
  uint64_t freed_bytes;
  uint64_t evicted_entries;
  uint64_t remaining_resident_bytes;
  int32_t still_over_capacity;
} PjrtxB200ExecutableCacheTrim;

/* executable_cache.EntrySnapshot (:58-63). */
typedef struct PjrtxB200ExecutableCacheEntry {
  int32_t resident;
  uint64_t resident_bytes;
  uint64_t reference_count;
  uint64_t compile_latency_us;
} PjrtxB200ExecutableCacheEntry;

/* Residency.init / deinit (:333-343). `capacity_bytes` is the device memory that buffers and resident executables
 * share (0 = untracked: no pressure trims). Destroying the cache destroys every resident executable. */
PjrtxB200ExecutableCache *pjrtx_b200_executable_cache_create(uint64_t capacity_bytes);
void pjrtx_b200_executable_cache_destroy(PjrtxB200ExecutableCache *cache);
/* Residency.recordCompile (:346-352): 1 = seen before (hit), 0 = new (miss), -1 = error. */
int pjrtx_b200_executable_cache_record_compile(PjrtxB200ExecutableCache *cache, const char *fingerprint);
/* Residency.acquireBackendExecutable (:379-391, 429-470): leases the resident executable of a recorded fingerprint, or
 * compiles `plan` for the devices, trims idle entries to make room for its device bytes (`out_compile_trim`), and makes
 * it resident with one lease. `*out_reused` = 1 when no compile ran. The executable belongs to the cache: give the lease
 * back with pjrtx_b200_executable_cache_release, never pjrtx_b200_executable_destroy. NULL on failure or for a
 * fingerprint that was never recorded. */
PjrtxB200Executable *pjrtx_b200_executable_cache_acquire(PjrtxB200ExecutableCache *cache, const char *fingerprint,
                                                         PjrtxB200Plan *plan, const int32_t *device_ordinals,
                                                         uint64_t device_count, int *out_reused,
                                                         PjrtxB200ExecutableCacheTrim *out_compile_trim);
/* Residency.release (:394-399): returns one lease; idle entries beyond the byte budget are evicted. */
void pjrtx_b200_executable_cache_release(PjrtxB200ExecutableCache *cache, const char *fingerprint);
/* Residency.setMaxResidentBytes (:366-371). */
void pjrtx_b200_executable_cache_set_max_resident_bytes(PjrtxB200ExecutableCache *cache, uint64_t max_resident_bytes);
/* Residency.trimForAllocation (:374-376, 404-426): `bytes_in_use` = buffer bytes outside the cache. */
int pjrtx_b200_executable_cache_trim_for_allocation(PjrtxB200ExecutableCache *cache, uint64_t bytes_in_use,
                                                    uint64_t allocation_bytes, PjrtxB200ExecutableCacheTrim *out);
/* The capacity that pressure trims work against (the reference's tests set memory.stats.capacity_bytes directly). */
void pjrtx_b200_executable_cache_set_capacity(PjrtxB200ExecutableCache *cache, uint64_t capacity_bytes);
/* Residency.statsSnapshot / entrySnapshot (:355-362). entry returns 0 for an unknown fingerprint. */
int pjrtx_b200_executable_cache_stats(PjrtxB200ExecutableCache *cache, PjrtxB200ExecutableCacheStats *out);
int pjrtx_b200_executable_cache_entry(PjrtxB200ExecutableCache *cache, const char *fingerprint,
                                      PjrtxB200ExecutableCacheEntry *out);
/* Policy-test hooks (the reference's Testing namespaces: setCompileLatencyForTest :167-170, initBorrowedResident):
 * install_placeholder makes a recorded fingerprint resident with one lease and `resident_bytes` of accounted memory
 * but no executable behind it, so the eviction policy runs without a device; it returns 1 when the placeholder became
 * resident, 2 when the fingerprint was resident already (the lease is taken on that entry), 0 on error. */
int pjrtx_b200_executable_cache_install_placeholder(PjrtxB200ExecutableCache *cache, const char *fingerprint,
                                                    uint64_t resident_bytes, uint64_t bytes_in_use,
                                                    PjrtxB200ExecutableCacheTrim *out_compile_trim);
void pjrtx_b200_executable_cache_set_compile_latency(PjrtxB200ExecutableCache *cache, const char *fingerprint,
                                                     uint64_t latency_us);

/* ---- StableHLO text ------------------------------------------------------- */
/* Reads `func.func @main` of a textual StableHLO module into a plan (the subset of operations the backend executes;
 * static shapes; pretty or generic operation syntax). Replaces, for text, the MLIR-based importer
 * (src/compiler/stablehlo_module_import.zig:241-264, stablehlo_operation_import.zig:22-456). NULL on failure with
 * last_error holding one line in the reference's format (src/compiler/stablehlo_decode.zig:117-140):
 *   unsupported op: op=<name> loc=L:C dtype=<t> rank=<r|unknown> sharding=<...> feature=stablehlo-op
 * or, for malformed text, `invalid module: loc=L:C detail="..." feature=stablehlo-text`. */
PjrtxB200Plan *pjrtx_b200_plan_from_stablehlo_text(const char *text, uint64_t length);

/* ---- custom calls -------------------------------------------------------- */
/* Backend.register{Identity,Unary,Binary}CustomCall / unregisterCustomCall / customCallRegistryVersion
 * (backend.zig:150-175). `op_name` is "identity" or an elementwise kind name; arity 1 or 2. */
int pjrtx_b200_register_custom_call(const char *target, const char *op_name, int arity);
void pjrtx_b200_unregister_custom_call(const char *target);
uint64_t pjrtx_b200_custom_call_registry_version(void);

/* ---- tensor-parallel communicator (no counterpart: the reference has no collectives) ---- */
int pjrtx_b200_comm_unique_id(uint8_t out_id[128]);
int pjrtx_b200_comm_init(int device_ordinal, const uint8_t id[128], int rank, int world_size);
void pjrtx_b200_comm_destroy(int device_ordinal);
/* Peer-memory all-reduce (no counterpart in the reference). Optional, after comm_init: every rank calls
 * comm_peer_export (allocates this rank's region and returns its 64-byte CUDA IPC handle), the host ships all handles
 * to all ranks in rank order, every rank calls comm_peer_import with the world_size x 64 bytes; from then on sums of up
 * to world_size x 512 KiB inside executables run as one kernel per rank (reduce-scatter and all-gather through the
 * peers' regions over NVLink) instead of a library collective. All ranks must have exported before any of them executes (the exchange of the handles is that
 * barrier). Ranks are processes on one node, one GPU each, 2..8 of them. 1 on success, 0 with last_error set. */
int pjrtx_b200_comm_peer_export(int device_ordinal, uint8_t out_handle[64]);
int pjrtx_b200_comm_peer_import(int device_ordinal, const uint8_t *handles, int rank, int world_size);

/* ---- contraction without allocation ---------------------------------------- */
/* No counterpart in the reference. out[m, n] = lhs[m, k] . rhs[k, n] for dense row-major device pointers, 1 <= m <= 8,
 * element type f32 / f16 / bf16, n a multiple of 16 bytes' worth of elements, rhs and out 16-byte aligned.
 *
 * For callers that cannot allocate device memory where they need the product: a runtime whose arena already owns all
 * of HBM, code running under another allocator's lock, a serving loop that forbids allocator calls after start-up.
 * The split-K scratch of the streaming kernel (f32 partial sums, per-tile counters) comes from a fixed 8 MiB + 64 KiB
 * array inside the library image, so the call makes no cudaMalloc / cudaFree / pool call. Consequences:
 *  - problems whose scratch does not fit are refused with a message that names the sizes (m <= 8 against rhs up to
 *    4096 x 128256 fits);
 *  - every GPU that loads the library holds the array until the process exits;
 *  - all calls share the array, and it keeps the previous call's contents (the counters and the error word are
 *    cleared on the stream before each launch): two calls that overlap on the GPU race, so keep them on one stream
 *    or order them with events;
 *  - the first call on a device resolves the array's address and raises the kernel's shared-memory limit; make that
 *    first call before any stream capture begins.
 * The caller's current CUDA device is left as it was. `stream` is a cudaStream_t (NULL = the default stream).
 * Returns 1 when the work was enqueued, 0 with pjrtx_b200_last_error() set. */
int pjrtx_b200_dot_static_scratch(int device_ordinal, int dtype, const void *lhs, const void *rhs, void *out, int64_t m,
                                  int64_t k, int64_t n, void *stream);
/* No counterpart in the reference. Completion status of the most recent pjrtx_b200_dot_static_scratch call on the
 * device: waits for `stream`, reads the kernel's error word out of the static array (a 4-byte copy into a stack
 * variable; nothing is allocated) and returns 1 when the kernel ran to completion, 0 with last_error set when one of
 * its bounded device-side waits gave up (the output of that call is then not valid). Ask before the next call on the
 * device: every call clears the word. */
int pjrtx_b200_dot_static_scratch_status(int device_ordinal, void *stream);

/* ---- generated-kernel check (no device needed) ---------------------------- */
/* Compiles CUDA source for sm_100a with the run-time compiler; 1 when it compiles. The log goes to `out`. */
int pjrtx_b200_compile_check(const char *source, char *out, uint64_t capacity);

#ifdef __cplusplus
}
#endif

#endif /* PJRTX_B200_H_ */

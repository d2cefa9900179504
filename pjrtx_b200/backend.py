"""ctypes binding of `libpjrtx_b200.so` and a Python mirror of the reference's `Backend` facade.

`Backend` has the method set of src/backend/mlx_metal/backend.zig:91-180
(capabilities, enumerate_devices, buffer_from_host, allocate_buffer,
clone_buffer, compile_executable, write_executable_lowering_diagnostic,
execute_executable, executable_stats, copy_to_host, destroy_*), with the same
error classes (backend.zig:21-31 → `BackendError.kind`). Nothing here computes:
every call goes through the C ABI declared in include/pjrtx_b200.h, and a
missing or unloadable library is an error, never a fallback.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import List, Optional, Sequence

import numpy as np

from . import plan as plan_mod

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libpjrtx_b200.so")


class BackendError(RuntimeError):
    """Mirrors the reference's backend error set; `kind` is the Zig error name."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind
        self.message = message


class Attribute(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("values", ctypes.POINTER(ctypes.c_int64)), ("count", ctypes.c_uint64)]


class DeviceInfo(ctypes.Structure):
    _fields_ = [("ordinal", ctypes.c_int32), ("registry_id", ctypes.c_uint64), ("memory_bytes", ctypes.c_uint64),
                ("has_unified_memory", ctypes.c_uint8), ("name", ctypes.c_char * 128)]


class Capabilities(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("supports_device_buffers", ctypes.c_uint8),
                ("supports_unified_memory", ctypes.c_uint8), ("supports_async_execution", ctypes.c_uint8)]


_STATS_FIELDS = [
    "struct_size", "resident_constant_count", "resident_constant_bytes", "program_value_count", "program_node_count",
    "program_edge_count", "program_schedule_item_count", "program_subprogram_count", "program_control_flow_count",
    "program_fusion_group_count", "program_materialization_boundary_count", "program_planned_release_count",
    "program_planned_release_bytes", "program_peak_live_value_count", "program_peak_live_bytes", "program_device_count",
    "last_execute_device_index", "last_execute_local_hardware_id", "execute_count", "compiled_program_execute_count",
    "compiled_program_output_count", "captured_program_execute_count", "captured_program_dynamic_input_count",
    "captured_program_captured_input_count", "donation_alias_output_count", "donation_alias_output_bytes",
    "fusion_group_execute_count", "execute_wall_us_total", "execute_wall_us_peak", "kernel_step_count",
    "generated_kernel_count", "arena_bytes", "scratch_bytes", "graph_capture_count", "graph_launch_count",
    "kernel_launch_total", "profile_event_gap_ns",
]


class ExecutableStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32 if n == "last_execute_local_hardware_id" else ctypes.c_uint64) for n in _STATS_FIELDS]


class MemoryStats(ctypes.Structure):
    _fields_ = [("bytes_in_use", ctypes.c_uint64), ("peak_bytes_in_use", ctypes.c_uint64),
                ("host_to_device_bytes", ctypes.c_uint64), ("device_to_host_bytes", ctypes.c_uint64)]


_CACHE_STATS_FIELDS = ["hits", "misses", "evictions", "evicted_resident_bytes", "resident_entries", "resident_bytes",
                       "peak_resident_bytes", "largest_resident_bytes", "compile_latency_samples",
                       "compile_latency_us_total", "compile_latency_us_peak", "pressure_trim_requests",
                       "pressure_trimmed_bytes", "pressure_trim_failures"]


class ExecutableCacheStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in _CACHE_STATS_FIELDS]


class ExecutableCacheTrim(ctypes.Structure):
    _fields_ = [("requested_bytes", ctypes.c_uint64), ("target_resident_bytes", ctypes.c_uint64),
                ("freed_bytes", ctypes.c_uint64), ("evicted_entries", ctypes.c_uint64),
                ("remaining_resident_bytes", ctypes.c_uint64), ("still_over_capacity", ctypes.c_int32)]

    def as_dict(self) -> dict:
        d = {n: getattr(self, n) for n, _ in self._fields_}
        d["still_over_capacity"] = bool(d["still_over_capacity"])
        return d


class ExecutableCacheEntry(ctypes.Structure):
    _fields_ = [("resident", ctypes.c_int32), ("resident_bytes", ctypes.c_uint64), ("reference_count", ctypes.c_uint64),
                ("compile_latency_us", ctypes.c_uint64)]


# Every symbol include/pjrtx_b200.h declares: name -> (restype, argtypes).
_P = ctypes.c_void_p
_I64P = ctypes.POINTER(ctypes.c_int64)
_U32P = ctypes.POINTER(ctypes.c_uint32)
SYMBOLS = {
    "pjrtx_b200_version_major": (ctypes.c_int, []),
    "pjrtx_b200_version_minor": (ctypes.c_int, []),
    "pjrtx_b200_version_patch": (ctypes.c_int, []),
    "pjrtx_b200_last_error": (ctypes.c_char_p, []),
    "pjrtx_b200_capabilities": (ctypes.c_int, [ctypes.POINTER(Capabilities)]),
    "pjrtx_b200_device_count": (ctypes.c_int, []),
    "pjrtx_b200_copy_devices": (ctypes.c_int, [ctypes.POINTER(DeviceInfo), ctypes.c_int]),
    "pjrtx_b200_device_memory_stats": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(MemoryStats)]),
    "pjrtx_b200_device_synchronize": (ctypes.c_int, [ctypes.c_int]),
    "pjrtx_b200_device_event_record": (_P, [ctypes.c_int]),
    "pjrtx_b200_device_event_elapsed_ms": (ctypes.c_int, [_P, _P, ctypes.POINTER(ctypes.c_double)]),
    "pjrtx_b200_device_event_destroy": (None, [_P]),
    "pjrtx_b200_buffer_from_host_typed": (_P, [ctypes.c_int, _P, ctypes.c_uint64, ctypes.c_int, _I64P, ctypes.c_uint64]),
    "pjrtx_b200_buffer_zeros": (_P, [ctypes.c_int, ctypes.c_int, _I64P, ctypes.c_uint64]),
    "pjrtx_b200_buffer_clone": (_P, [_P]),
    "pjrtx_b200_buffer_size": (ctypes.c_uint64, [_P]),
    "pjrtx_b200_buffer_dtype": (ctypes.c_int, [_P]),
    "pjrtx_b200_buffer_rank": (ctypes.c_uint64, [_P]),
    "pjrtx_b200_buffer_dims": (ctypes.c_int, [_P, _I64P, ctypes.c_uint64]),
    "pjrtx_b200_buffer_device": (ctypes.c_int, [_P]),
    "pjrtx_b200_buffer_is_donated": (ctypes.c_int, [_P]),
    "pjrtx_b200_buffer_copy_to_host": (ctypes.c_int, [_P, _P, ctypes.c_uint64]),
    "pjrtx_b200_buffer_destroy": (None, [_P]),
    "pjrtx_b200_async_h2d_create": (_P, [ctypes.c_int, ctypes.c_int, _I64P, ctypes.c_uint64, ctypes.c_uint64]),
    "pjrtx_b200_async_h2d_write": (ctypes.c_int, [_P, ctypes.c_uint64, _P, ctypes.c_uint64]),
    "pjrtx_b200_async_h2d_finish": (_P, [_P]),
    "pjrtx_b200_async_h2d_destroy": (None, [_P]),
    "pjrtx_b200_plan_create": (_P, [ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(ctypes.c_int32), ctypes.c_uint64]),
    "pjrtx_b200_plan_destroy": (None, [_P]),
    "pjrtx_b200_plan_add_value": (ctypes.c_uint32, [_P, ctypes.c_int, ctypes.c_int, _I64P, ctypes.c_uint64]),
    "pjrtx_b200_plan_add_instruction": (ctypes.c_int, [_P, ctypes.c_char_p, _U32P, ctypes.c_uint64, _U32P, ctypes.c_uint64,
                                                       ctypes.POINTER(Attribute), ctypes.c_uint64, ctypes.c_char_p,
                                                       ctypes.c_uint64, ctypes.c_char_p]),
    "pjrtx_b200_plan_set_outputs": (ctypes.c_int, [_P, _U32P, ctypes.c_uint64]),
    "pjrtx_b200_plan_set_parameter_sharding": (ctypes.c_int, [_P, ctypes.c_uint64, ctypes.c_int, ctypes.c_char_p, ctypes.c_int64]),
    "pjrtx_b200_plan_set_output_sharding": (ctypes.c_int, [_P, ctypes.c_uint64, ctypes.c_int, ctypes.c_char_p, ctypes.c_int64]),
    "pjrtx_b200_plan_set_donation": (ctypes.c_int, [_P, _U32P, ctypes.c_uint64, _U32P, _U32P, ctypes.c_uint64]),
    "pjrtx_b200_plan_from_stablehlo_text": (_P, [ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_plan_verify": (ctypes.c_int, [_P, ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_plan_describe": (ctypes.c_uint64, [_P, ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_plan_fingerprint": (ctypes.c_uint64, [_P, ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_plan_fingerprint_for_devices": (ctypes.c_uint64, [_P, ctypes.POINTER(ctypes.c_int32), ctypes.c_uint64,
                                                                  ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_plan_describe_program": (ctypes.c_uint64, [_P, ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_plan_describe_kernels": (ctypes.c_uint64, [_P, ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_plan_partition": (_P, [_P, ctypes.c_int32, ctypes.c_int32]),
    "pjrtx_b200_compile_executable": (_P, [_P, ctypes.POINTER(ctypes.c_int32), ctypes.c_uint64]),
    "pjrtx_b200_write_executable_lowering_diagnostic": (ctypes.c_uint64, [_P, ctypes.c_uint64, ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_execute_executable": (ctypes.c_int, [_P, ctypes.c_uint64, ctypes.POINTER(_P), ctypes.c_uint64,
                                                     ctypes.POINTER(ctypes.POINTER(_P)), ctypes.POINTER(ctypes.c_uint64),
                                                     ctypes.POINTER(_P)]),
    "pjrtx_b200_output_array_destroy": (None, [ctypes.POINTER(_P)]),
    "pjrtx_b200_execution_event_status": (ctypes.c_int, [_P]),
    "pjrtx_b200_execution_event_await": (ctypes.c_int, [_P]),
    "pjrtx_b200_execution_event_destroy": (None, [_P]),
    "pjrtx_b200_executable_stats": (ctypes.c_int, [_P, ctypes.POINTER(ExecutableStats)]),
    "pjrtx_b200_executable_describe": (ctypes.c_uint64, [_P, ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_executable_set_profiling": (ctypes.c_int, [_P, ctypes.c_int]),
    "pjrtx_b200_executable_step_times": (ctypes.c_uint64, [_P, ctypes.POINTER(ctypes.c_float), ctypes.c_uint64]),
    "pjrtx_b200_executable_destroy": (None, [_P]),
    "pjrtx_b200_register_custom_call": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]),
    "pjrtx_b200_unregister_custom_call": (None, [ctypes.c_char_p]),
    "pjrtx_b200_custom_call_registry_version": (ctypes.c_uint64, []),
    "pjrtx_b200_comm_unique_id": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint8)]),
    "pjrtx_b200_comm_init": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(ctypes.c_uint8), ctypes.c_int, ctypes.c_int]),
    "pjrtx_b200_comm_destroy": (None, [ctypes.c_int]),
    "pjrtx_b200_comm_peer_export": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(ctypes.c_uint8)]),
    "pjrtx_b200_comm_peer_import": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(ctypes.c_uint8), ctypes.c_int, ctypes.c_int]),
    "pjrtx_b200_dot_static_scratch": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _P, _P, _P, ctypes.c_int64, ctypes.c_int64,
                                                      ctypes.c_int64, _P]),
    "pjrtx_b200_device_bounded_wait_probe": (ctypes.c_int, [ctypes.c_int, ctypes.c_uint32]),
    "pjrtx_b200_dot_static_scratch_status": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p]),
    "pjrtx_b200_compile_check": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint64]),
    "pjrtx_b200_executable_cache_create": (_P, [ctypes.c_uint64]),
    "pjrtx_b200_executable_cache_destroy": (None, [_P]),
    "pjrtx_b200_executable_cache_record_compile": (ctypes.c_int, [_P, ctypes.c_char_p]),
    "pjrtx_b200_executable_cache_acquire": (_P, [_P, ctypes.c_char_p, _P, ctypes.POINTER(ctypes.c_int32), ctypes.c_uint64,
                                                 ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ExecutableCacheTrim)]),
    "pjrtx_b200_executable_cache_release": (None, [_P, ctypes.c_char_p]),
    "pjrtx_b200_executable_cache_set_max_resident_bytes": (None, [_P, ctypes.c_uint64]),
    "pjrtx_b200_executable_cache_set_capacity": (None, [_P, ctypes.c_uint64]),
    "pjrtx_b200_executable_cache_trim_for_allocation": (ctypes.c_int, [_P, ctypes.c_uint64, ctypes.c_uint64,
                                                                       ctypes.POINTER(ExecutableCacheTrim)]),
    "pjrtx_b200_executable_cache_stats": (ctypes.c_int, [_P, ctypes.POINTER(ExecutableCacheStats)]),
    "pjrtx_b200_executable_cache_entry": (ctypes.c_int, [_P, ctypes.c_char_p, ctypes.POINTER(ExecutableCacheEntry)]),
    "pjrtx_b200_executable_cache_install_placeholder": (ctypes.c_int, [_P, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint64,
                                                                        ctypes.POINTER(ExecutableCacheTrim)]),
    "pjrtx_b200_executable_cache_set_compile_latency": (None, [_P, ctypes.c_char_p, ctypes.c_uint64]),
}

_lib = None


def load_library(path: Optional[str] = None):
    """Loads the shared library once and types every entry point. Fails loudly when it is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or os.environ.get("PJRTX_B200_LIBRARY", LIB_PATH)
    if not os.path.exists(p):
        raise BackendError("InvalidProgram", f"{p} is not built; run `python -c 'import __graft_entry__ as g; g.build()'`")
    lib = ctypes.CDLL(p)
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError = header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    if path is None:
        _lib = lib
    return lib


def _text(lib, fn, handle, *extra) -> str:
    """Calls a `(handle, ..., char* out, capacity) -> length` entry point, growing the buffer as needed."""
    cap = 1 << 16
    while True:
        buf = ctypes.create_string_buffer(cap)
        n = fn(handle, *extra, buf, cap)
        if n < cap:
            return buf.value.decode() if n else ""
        cap = int(n) + 1


class DeviceBuffer:
    """Owning handle of one device buffer (BufferHandle in the reference)."""

    def __init__(self, lib, handle):
        self._lib = lib
        self.handle = handle

    @property
    def dtype(self) -> int:
        return self._lib.pjrtx_b200_buffer_dtype(self.handle)

    @property
    def dims(self):
        rank = self._lib.pjrtx_b200_buffer_rank(self.handle)
        out = (ctypes.c_int64 * max(rank, 1))()
        self._lib.pjrtx_b200_buffer_dims(self.handle, out, rank)
        return tuple(out[i] for i in range(rank))

    @property
    def nbytes(self) -> int:
        return self._lib.pjrtx_b200_buffer_size(self.handle)

    @property
    def is_donated(self) -> bool:
        return bool(self._lib.pjrtx_b200_buffer_is_donated(self.handle))

    def to_numpy(self) -> np.ndarray:
        out = np.empty(self.dims, dtype=plan_mod.np_dtype(self.dtype))
        if not self._lib.pjrtx_b200_buffer_copy_to_host(self.handle, out.ctypes.data_as(ctypes.c_void_p), out.nbytes):
            raise BackendError("BufferCopyFailed", self._lib.pjrtx_b200_last_error().decode())
        return out

    def destroy(self):
        if self.handle:
            self._lib.pjrtx_b200_buffer_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class Executable:
    def __init__(self, lib, handle, builder: plan_mod.PlanBuilder):
        self._lib = lib
        self.handle = handle
        self.builder = builder

    def stats(self) -> dict:
        s = ExecutableStats()
        s.struct_size = ctypes.sizeof(ExecutableStats)
        if not self._lib.pjrtx_b200_executable_stats(self.handle, ctypes.byref(s)):
            raise BackendError("InvalidProgram", "executable_stats failed")
        return {n: getattr(s, n) for n in _STATS_FIELDS}

    def describe(self) -> dict:
        return json.loads(_text(self._lib, self._lib.pjrtx_b200_executable_describe, self.handle))

    def set_profiling(self, enabled: bool) -> None:
        self._lib.pjrtx_b200_executable_set_profiling(self.handle, 1 if enabled else 0)

    def step_times_ms(self) -> List[float]:
        n = self._lib.pjrtx_b200_executable_step_times(self.handle, None, 0)
        buf = (ctypes.c_float * max(int(n), 1))()
        self._lib.pjrtx_b200_executable_step_times(self.handle, buf, n)
        return [buf[i] for i in range(int(n))]

    def destroy(self):
        if self.handle:
            self._lib.pjrtx_b200_executable_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class CachedExecutable(Executable):
    """A lease on a resident executable: `destroy` gives the lease back to the cache instead of freeing the executable."""

    def __init__(self, lib, handle, builder, cache: "ExecutableCache", fingerprint: str, reused: bool, compile_trim: dict):
        super().__init__(lib, handle, builder)
        self.cache = cache
        self.fingerprint = fingerprint
        self.reused = reused
        self.compile_trim = compile_trim

    def destroy(self):
        if self.handle:
            self.handle = None
            self.cache.release(self.fingerprint)


class ExecutableCache:
    """Resident executables keyed by plan fingerprint (the reference's `Residency`, src/runtime/executable_cache.zig:
    333-400, driven the way src/runtime/client_residency_tests.zig drives it)."""

    def __init__(self, backend: "Backend", capacity_bytes: int = 0):
        self.backend = backend
        self.lib = backend.lib
        self.handle = self.lib.pjrtx_b200_executable_cache_create(capacity_bytes)
        if not self.handle:
            raise BackendError("OutOfMemory", backend._err())

    def record_compile(self, fingerprint: str) -> bool:
        r = self.lib.pjrtx_b200_executable_cache_record_compile(self.handle, fingerprint.encode())
        if r < 0:
            raise BackendError("InvalidProgram", self.backend._err())
        return r == 1

    def compile(self, builder: plan_mod.PlanBuilder, devices: Sequence[int] = (0,),
                fingerprint: Optional[str] = None) -> CachedExecutable:
        """`recordCompile` + `acquireBackendExecutable`: a resident executable is leased again, otherwise the plan compiles."""
        plan = builder.build(self.lib)
        try:
            devs = (ctypes.c_int32 * len(devices))(*devices)
            fp = fingerprint or _text(self.lib, self.lib.pjrtx_b200_plan_fingerprint_for_devices, plan, devs, len(devices))
            self.record_compile(fp)
            reused = ctypes.c_int(0)
            trim = ExecutableCacheTrim()
            h = self.lib.pjrtx_b200_executable_cache_acquire(self.handle, fp.encode(), plan, devs, len(devices),
                                                             ctypes.byref(reused), ctypes.byref(trim))
            if not h:
                raise BackendError("InvalidProgram", self.backend._err())
            return CachedExecutable(self.lib, h, builder, self, fp, bool(reused.value), trim.as_dict())
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    def install_placeholder(self, fingerprint: str, resident_bytes: int, bytes_in_use: int = 0):
        """Policy-test hook: a resident entry with accounted bytes and no executable. Returns (reused, compile trim)."""
        trim = ExecutableCacheTrim()
        r = self.lib.pjrtx_b200_executable_cache_install_placeholder(self.handle, fingerprint.encode(), resident_bytes,
                                                                     bytes_in_use, ctypes.byref(trim))
        if r == 0:
            raise BackendError("InvalidProgram", self.backend._err())
        return r == 2, trim.as_dict()

    def release(self, fingerprint: str) -> None:
        if self.handle:
            self.lib.pjrtx_b200_executable_cache_release(self.handle, fingerprint.encode())

    def set_max_resident_bytes(self, max_resident_bytes: int) -> None:
        self.lib.pjrtx_b200_executable_cache_set_max_resident_bytes(self.handle, max_resident_bytes)

    def set_capacity(self, capacity_bytes: int) -> None:
        self.lib.pjrtx_b200_executable_cache_set_capacity(self.handle, capacity_bytes)

    def set_compile_latency(self, fingerprint: str, latency_us: int) -> None:
        self.lib.pjrtx_b200_executable_cache_set_compile_latency(self.handle, fingerprint.encode(), latency_us)

    def trim_for_allocation(self, bytes_in_use: int, allocation_bytes: int) -> dict:
        trim = ExecutableCacheTrim()
        if not self.lib.pjrtx_b200_executable_cache_trim_for_allocation(self.handle, bytes_in_use, allocation_bytes,
                                                                        ctypes.byref(trim)):
            raise BackendError("InvalidProgram", self.backend._err())
        return trim.as_dict()

    def stats(self) -> dict:
        s = ExecutableCacheStats()
        if not self.lib.pjrtx_b200_executable_cache_stats(self.handle, ctypes.byref(s)):
            raise BackendError("InvalidProgram", self.backend._err())
        return {n: getattr(s, n) for n in _CACHE_STATS_FIELDS}

    def entry(self, fingerprint: str) -> Optional[dict]:
        e = ExecutableCacheEntry()
        if not self.lib.pjrtx_b200_executable_cache_entry(self.handle, fingerprint.encode(), ctypes.byref(e)):
            return None
        return {"resident": bool(e.resident), "resident_bytes": e.resident_bytes, "reference_count": e.reference_count,
                "compile_latency_us": e.compile_latency_us}

    def destroy(self) -> None:
        if self.handle:
            self.lib.pjrtx_b200_executable_cache_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class Backend:
    """The B200 backend behind the reference's facade (src/backend/mlx_metal/backend.zig:91-180)."""

    def __init__(self, library_path: Optional[str] = None):
        self.lib = load_library(library_path)

    def _err(self) -> str:
        return self.lib.pjrtx_b200_last_error().decode()

    # -- devices --
    def capabilities(self) -> dict:
        c = Capabilities()
        self.lib.pjrtx_b200_capabilities(ctypes.byref(c))
        return {"name": c.name.decode(), "supports_device_buffers": bool(c.supports_device_buffers),
                "supports_unified_memory": bool(c.supports_unified_memory),
                "supports_async_execution": bool(c.supports_async_execution)}

    def enumerate_devices(self) -> List[dict]:
        n = self.lib.pjrtx_b200_device_count()
        arr = (DeviceInfo * max(n, 1))()
        got = self.lib.pjrtx_b200_copy_devices(arr, n)
        if got < 1:
            raise BackendError("InvalidDeviceCount", self._err() or "no B200 device is visible")
        return [{"ordinal": arr[i].ordinal, "registry_id": arr[i].registry_id, "memory_bytes": arr[i].memory_bytes,
                 "has_unified_memory": bool(arr[i].has_unified_memory), "name": arr[i].name.decode()} for i in range(got)]

    def memory_stats(self, device: int = 0) -> dict:
        m = MemoryStats()
        if not self.lib.pjrtx_b200_device_memory_stats(device, ctypes.byref(m)):
            raise BackendError("InvalidDeviceCount", self._err())
        return {n: getattr(m, n) for n, _ in MemoryStats._fields_}

    def bounded_wait_probe(self, device: int = 0, timeout_ms: int = 50) -> None:
        """Enqueues a kernel whose bounded wait cannot complete; the next `synchronize` reports it (code 31)."""
        if not self.lib.pjrtx_b200_device_bounded_wait_probe(device, timeout_ms):
            raise BackendError("CommandSubmissionFailed", self._err())

    def record_event(self, device: int = 0):
        """Enqueues a timing event on the device's stream; pair two of them with `elapsed_ms`."""
        h = self.lib.pjrtx_b200_device_event_record(device)
        if not h:
            raise BackendError("CommandSubmissionFailed", self._err())
        return h

    def elapsed_ms(self, start, stop, destroy: bool = True) -> float:
        out = ctypes.c_double(0.0)
        if not self.lib.pjrtx_b200_device_event_elapsed_ms(start, stop, ctypes.byref(out)):
            raise BackendError("CommandSubmissionFailed", self._err())
        if destroy:
            self.lib.pjrtx_b200_device_event_destroy(start)
            self.lib.pjrtx_b200_device_event_destroy(stop)
        return out.value

    def synchronize(self, device: int = 0) -> None:
        if not self.lib.pjrtx_b200_device_synchronize(device):
            raise BackendError("CommandSubmissionFailed", self._err())

    # -- buffers --
    def buffer_from_host(self, array: np.ndarray, device: int = 0, dtype: Optional[int] = None) -> DeviceBuffer:
        shape = np.shape(array)  # ascontiguousarray promotes rank 0 to rank 1
        arr = np.ascontiguousarray(array)
        code = dtype if dtype is not None else plan_mod.dtype_code(arr.dtype)
        dims = (ctypes.c_int64 * len(shape))(*shape)
        h = self.lib.pjrtx_b200_buffer_from_host_typed(device, arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes, code, dims, len(shape))
        if not h:
            raise BackendError("BufferAllocationFailed", self._err())
        return DeviceBuffer(self.lib, h)

    def buffer_from_pointer(self, pointer: int, nbytes: int, dtype: int, dims: Sequence[int], device: int = 0) -> DeviceBuffer:
        """Uploads from raw host memory (e.g. a pinned torch tensor's data_ptr)."""
        d = (ctypes.c_int64 * len(dims))(*dims)
        h = self.lib.pjrtx_b200_buffer_from_host_typed(device, ctypes.c_void_p(pointer), nbytes, dtype, d, len(dims))
        if not h:
            raise BackendError("BufferAllocationFailed", self._err())
        return DeviceBuffer(self.lib, h)

    def allocate_buffer(self, dtype: int, dims: Sequence[int], device: int = 0) -> DeviceBuffer:
        d = (ctypes.c_int64 * len(dims))(*dims)
        h = self.lib.pjrtx_b200_buffer_zeros(device, dtype, d, len(dims))
        if not h:
            raise BackendError("BufferAllocationFailed", self._err())
        return DeviceBuffer(self.lib, h)

    def clone_buffer(self, src: DeviceBuffer) -> DeviceBuffer:
        h = self.lib.pjrtx_b200_buffer_clone(src.handle)
        if not h:
            raise BackendError("BufferAllocationFailed", self._err())
        return DeviceBuffer(self.lib, h)

    def copy_to_host(self, src: DeviceBuffer) -> np.ndarray:
        return src.to_numpy()

    def copy_to_pointer(self, src: DeviceBuffer, pointer: int, nbytes: int) -> None:
        if not self.lib.pjrtx_b200_buffer_copy_to_host(src.handle, ctypes.c_void_p(pointer), nbytes):
            raise BackendError("BufferCopyFailed", self._err())

    # -- plans --
    def verify_plan(self, builder: plan_mod.PlanBuilder) -> str:
        plan = builder.build(self.lib)
        try:
            buf = ctypes.create_string_buffer(4096)
            ok = self.lib.pjrtx_b200_plan_verify(plan, buf, 4096)
            return "" if ok else buf.value.decode()
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    def import_stablehlo_text(self, text: str) -> plan_mod.PlanBuilder:
        """`func.func @main` of a textual StableHLO module as a PlanBuilder (compile it like any other plan).

        Raises BackendError("Unimplemented") with the reference-format diagnostic for operations outside the subset and
        BackendError("InvalidProgram") for malformed text."""
        raw = text.encode()
        plan = self.lib.pjrtx_b200_plan_from_stablehlo_text(raw, len(raw))
        if not plan:
            err = self._err()
            raise BackendError("Unimplemented" if err.startswith("unsupported op") else "InvalidProgram", err)
        try:
            return plan_mod.PlanBuilder.from_description(json.loads(_text(self.lib, self.lib.pjrtx_b200_plan_describe, plan)))
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    def partition_plan(self, builder: plan_mod.PlanBuilder, partition: int) -> plan_mod.PlanBuilder:
        """The tensor-parallel plan of one partition, read back as a PlanBuilder (for inspection and the CPU oracle)."""
        plan = builder.build(self.lib)
        try:
            part = self.lib.pjrtx_b200_plan_partition(plan, partition, builder.num_partitions)
            if not part:
                raise BackendError("InvalidProgram", self._err())
            try:
                return plan_mod.PlanBuilder.from_description(json.loads(_text(self.lib, self.lib.pjrtx_b200_plan_describe, part)))
            finally:
                self.lib.pjrtx_b200_plan_destroy(part)
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    def plan_fingerprint(self, builder: plan_mod.PlanBuilder, devices: Optional[Sequence[int]] = None) -> str:
        """Cache key of the plan under the current backend state (custom-call registry version included); with
        `devices` the target device ordinals are part of the key (the form the executable cache uses)."""
        plan = builder.build(self.lib)
        try:
            if devices is not None:
                devs = (ctypes.c_int32 * len(devices))(*devices)
                return _text(self.lib, self.lib.pjrtx_b200_plan_fingerprint_for_devices, plan, devs, len(devices))
            return _text(self.lib, self.lib.pjrtx_b200_plan_fingerprint, plan)
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    def describe_program(self, builder: plan_mod.PlanBuilder) -> dict:
        plan = builder.build(self.lib)
        try:
            text = _text(self.lib, self.lib.pjrtx_b200_plan_describe_program, plan)
            if not text:
                raise BackendError("InvalidProgram", self._err())
            return json.loads(text)
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    def describe_kernels(self, builder: plan_mod.PlanBuilder, partition: Optional[int] = None) -> dict:
        plan = builder.build(self.lib)
        try:
            target = plan
            if partition is not None:
                target = self.lib.pjrtx_b200_plan_partition(plan, partition, builder.num_partitions)
                if not target:
                    raise BackendError("InvalidProgram", self._err())
            try:
                text = _text(self.lib, self.lib.pjrtx_b200_plan_describe_kernels, target)
                if not text:
                    raise BackendError("InvalidProgram", self._err())
                return json.loads(text)
            finally:
                if target != plan:
                    self.lib.pjrtx_b200_plan_destroy(target)
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    def write_executable_lowering_diagnostic(self, builder: plan_mod.PlanBuilder, device_count: int = 1) -> str:
        plan = builder.build(self.lib)
        try:
            return _text(self.lib, self.lib.pjrtx_b200_write_executable_lowering_diagnostic, plan, device_count)
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    # -- compile / execute --
    def compile_executable(self, builder: plan_mod.PlanBuilder, devices: Sequence[int] = (0,),
                           partition: Optional[int] = None) -> Executable:
        """Compiles the plan; with `partition` set, first derives that partition's tensor-parallel plan."""
        plan = builder.build(self.lib)
        try:
            target = plan
            if partition is not None:
                target = self.lib.pjrtx_b200_plan_partition(plan, partition, builder.num_partitions)
                if not target:
                    raise BackendError("InvalidProgram", self._err())
            try:
                devs = (ctypes.c_int32 * len(devices))(*devices)
                h = self.lib.pjrtx_b200_compile_executable(target, devs, len(devices))
                if not h:
                    raise BackendError("InvalidProgram", self._err())
                return Executable(self.lib, h, builder)
            finally:
                if target != plan:
                    self.lib.pjrtx_b200_plan_destroy(target)
        finally:
            self.lib.pjrtx_b200_plan_destroy(plan)

    def execute_executable(self, exe: Executable, arguments: Sequence[DeviceBuffer], device_index: int = 0) -> List[DeviceBuffer]:
        args = (ctypes.c_void_p * len(arguments))(*[a.handle for a in arguments])
        outs = ctypes.POINTER(ctypes.c_void_p)()
        count = ctypes.c_uint64(0)
        ok = self.lib.pjrtx_b200_execute_executable(exe.handle, device_index, args, len(arguments), ctypes.byref(outs),
                                                    ctypes.byref(count), None)
        if not ok:
            raise BackendError("CommandSubmissionFailed", self._err())
        result = [DeviceBuffer(self.lib, outs[i]) for i in range(count.value)]
        self.lib.pjrtx_b200_output_array_destroy(outs)
        return result

    # -- custom calls --
    def register_custom_call(self, target: str, op_name: str, arity: int) -> None:
        if not self.lib.pjrtx_b200_register_custom_call(target.encode(), op_name.encode(), arity):
            raise BackendError("InvalidCustomCall", self._err())

    def unregister_custom_call(self, target: str) -> None:
        self.lib.pjrtx_b200_unregister_custom_call(target.encode())

    def custom_call_registry_version(self) -> int:
        return self.lib.pjrtx_b200_custom_call_registry_version()

    # -- tensor-parallel communicator --
    def comm_unique_id(self) -> bytes:
        buf = (ctypes.c_uint8 * 128)()
        if not self.lib.pjrtx_b200_comm_unique_id(buf):
            raise BackendError("CommandSubmissionFailed", self._err())
        return bytes(buf)

    def comm_init(self, device: int, unique_id: bytes, rank: int, world: int) -> None:
        buf = (ctypes.c_uint8 * 128)(*unique_id)
        if not self.lib.pjrtx_b200_comm_init(device, buf, rank, world):
            raise BackendError("CommandSubmissionFailed", self._err())

    def comm_peer_export(self, device: int) -> bytes:
        """Allocates this rank's peer region and returns its 64-byte IPC handle (ship it to every other rank)."""
        buf = (ctypes.c_uint8 * 64)()
        if not self.lib.pjrtx_b200_comm_peer_export(device, buf):
            raise BackendError("CommandSubmissionFailed", self._err())
        return bytes(buf)

    def comm_peer_import(self, device: int, handles: Sequence[bytes], rank: int, world: int) -> None:
        """Maps every rank's region (handles in rank order); small all-reduces then run over peer memory."""
        flat = b"".join(handles)
        buf = (ctypes.c_uint8 * len(flat))(*flat)
        if not self.lib.pjrtx_b200_comm_peer_import(device, buf, rank, world):
            raise BackendError("CommandSubmissionFailed", self._err())

    def enable_peer_all_reduce(self, device: int, rank: int, world: int, all_gather_object) -> None:
        """Export, exchange through `all_gather_object(list_out, obj)` (torch.distributed's signature), import."""
        mine = self.comm_peer_export(device)
        handles = [None] * world
        all_gather_object(handles, mine)
        self.comm_peer_import(device, handles, rank, world)

    def dot_static_scratch(self, dtype: int, lhs_ptr: int, rhs_ptr: int, out_ptr: int, m: int, k: int, n: int, device: int = 0,
                           stream: int = 0) -> None:
        """out[m, n] = lhs[m, k] . rhs[k, n] on raw device pointers without any device allocation.

        For callers that may not allocate where they need the product (all of HBM already owned by their own arena,
        code under another allocator's lock, allocation-free serving loops): the kernel's split-K scratch is a fixed
        8 MiB array inside the library, shared by all calls; calls that overlap on the GPU race. Oversized problems
        raise with the sizes in the message. Make the first call on a device outside stream capture.
        """
        ok = self.lib.pjrtx_b200_dot_static_scratch(device, dtype, ctypes.c_void_p(lhs_ptr), ctypes.c_void_p(rhs_ptr),
                                                    ctypes.c_void_p(out_ptr), m, k, n, ctypes.c_void_p(stream))
        if not ok:
            raise BackendError("CommandSubmissionFailed", self._err())

    def dot_static_scratch_status(self, device: int = 0, stream: int = 0) -> None:
        """Waits for `stream` and raises if the most recent `dot_static_scratch` call on the device gave up one of its
        bounded device-side waits (its output is then not valid). Allocates nothing; ask before the next call."""
        if not self.lib.pjrtx_b200_dot_static_scratch_status(device, ctypes.c_void_p(stream)):
            raise BackendError("CommandSubmissionFailed", self._err())

    def compile_check(self, source: str) -> str:
        """Compiles generated CUDA source for sm_100a (no GPU needed); returns "" or the compiler log."""
        buf = ctypes.create_string_buffer(1 << 16)
        ok = self.lib.pjrtx_b200_compile_check(source.encode(), buf, 1 << 16)
        return "" if ok else (buf.value.decode() or "compile failed")

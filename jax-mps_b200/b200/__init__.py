"""Python face of the B200 PJRT core: a ctypes binding over the C ABI in
include/b200_core.h, shaped like the client objects jaxlib hands a user of the
reference plugin (`client.compile_and_load(text)`, `jax.device_put`,
`exe.execute([buf])`, `numpy.asarray(buf)` — compare the reference's raw-MLIR
test, tests/test_ops.py:245-281).

There is no CPU fallback: importing works anywhere (so host-side tooling can
run), but creating a `Client` raises `B200Error` unless the CUDA extension is
built and a GPU is present.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

_LIB_NAME = "libb200core.so"


class B200Error(RuntimeError):
    def __init__(self, message: str, code: int = 2):
        super().__init__(message)
        self.code = code


OK, CANCELLED, UNKNOWN, INVALID_ARGUMENT, NOT_FOUND = 0, 1, 2, 3, 5
RESOURCE_EXHAUSTED, FAILED_PRECONDITION, UNIMPLEMENTED, INTERNAL = 8, 9, 12, 13

# element types (b200_dtype)
PRED, S8, S16, S32, S64, U8, U16, U32, U64, F16, F32, F64, BF16 = range(1, 14)
_NP_TO_DT = {np.dtype(np.bool_): PRED, np.dtype(np.int8): S8, np.dtype(np.int16): S16, np.dtype(np.int32): S32,
             np.dtype(np.int64): S64, np.dtype(np.uint8): U8, np.dtype(np.uint16): U16, np.dtype(np.uint32): U32,
             np.dtype(np.uint64): U64, np.dtype(np.float16): F16, np.dtype(np.float32): F32,
             np.dtype(np.float64): F64}
_DT_TO_NP = {v: k for k, v in _NP_TO_DT.items()}
_DT_TO_NP[BF16] = np.dtype(np.uint16)          # raw bf16 bit patterns
_DT_NAMES = {PRED: "i1", S8: "i8", S16: "i16", S32: "i32", S64: "i64", U8: "ui8", U16: "ui16", U32: "ui32",
             U64: "ui64", F16: "f16", F32: "f32", F64: "f64", BF16: "bf16"}
_NAME_TO_DT = {v: k for k, v in _DT_NAMES.items()}
NCCL_ID_BYTES = 128


class _ClientOptions(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("device_ordinal", C.c_int), ("process_index", C.c_int),
                ("num_processes", C.c_int), ("nccl_unique_id", C.c_char_p), ("pool_release_threshold", C.c_size_t)]


class _CompileOptions(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("num_partitions", C.c_int), ("disable_fusion", C.c_int)]


class _ExecuteOptions(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("donate_arguments", C.c_int)]


class MemoryStats(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("bytes_in_use", C.c_int64),
                ("peak_bytes_in_use", C.c_int64), ("peak_bytes_in_use_is_set", C.c_int),
                ("bytes_limit", C.c_int64), ("bytes_limit_is_set", C.c_int),
                ("pool_bytes", C.c_int64), ("pool_bytes_is_set", C.c_int),
                ("peak_pool_bytes", C.c_int64), ("peak_pool_bytes_is_set", C.c_int),
                ("num_allocs", C.c_int64), ("num_allocs_is_set", C.c_int),
                ("largest_alloc_size", C.c_int64), ("largest_alloc_size_is_set", C.c_int)]


EVENT_CALLBACK = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)

# name -> (restype, argtypes); every symbol include/b200_core.h declares
_P = C.c_void_p
SIGNATURES = {
    "b200_error_destroy": (None, [_P]),
    "b200_error_message": (C.c_char_p, [_P]),
    "b200_error_get_code": (C.c_int, [_P]),
    "b200_client_create": (_P, [C.POINTER(_ClientOptions), C.POINTER(_P)]),
    "b200_client_destroy": (_P, [_P]),
    "b200_client_platform_name": (C.c_char_p, [_P]),
    "b200_client_platform_version": (C.c_char_p, [_P]),
    "b200_client_process_index": (C.c_int, [_P]),
    "b200_client_device_count": (C.c_int, [_P]),
    "b200_client_addressable_device_count": (C.c_int, [_P]),
    "b200_nccl_unique_id": (_P, [C.c_char_p]),
    "b200_device_id": (C.c_int, [_P]),
    "b200_device_local_hardware_id": (C.c_int, [_P]),
    "b200_device_kind": (C.c_char_p, [_P]),
    "b200_device_debug_string": (C.c_char_p, [_P]),
    "b200_device_memory_stats": (_P, [_P, C.POINTER(MemoryStats)]),
    "b200_client_compile": (_P, [_P, C.c_char_p, C.c_size_t, C.c_char_p, C.POINTER(_CompileOptions), C.POINTER(_P)]),
    "b200_executable_destroy": (_P, [_P]),
    "b200_executable_name": (C.c_char_p, [_P]),
    "b200_executable_fingerprint": (C.c_char_p, [_P]),
    "b200_executable_num_replicas": (C.c_int, [_P]),
    "b200_executable_num_partitions": (C.c_int, [_P]),
    "b200_executable_num_args": (C.c_size_t, [_P]),
    "b200_executable_num_outputs": (C.c_size_t, [_P]),
    "b200_executable_output_info": (_P, [_P, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int64)), C.POINTER(C.c_size_t)]),
    "b200_executable_arg_info": (_P, [_P, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.POINTER(C.c_int64)), C.POINTER(C.c_size_t)]),
    "b200_executable_launches_per_execute": (C.c_int64, [_P]),
    "b200_executable_num_kernels": (C.c_int64, [_P]),
    "b200_executable_temp_bytes": (C.c_int64, [_P]),
    "b200_executable_plan_text": (C.c_char_p, [_P]),
    "b200_compile_to_plan": (_P, [C.c_char_p, C.c_size_t, C.POINTER(_CompileOptions), C.c_int, C.c_int, C.c_int,
                                  C.POINTER(_P), C.POINTER(_P)]),
    "b200_string_free": (None, [_P]),
    "b200_buffer_from_host": (_P, [_P, _P, C.c_int, C.POINTER(C.c_int64), C.c_size_t, C.POINTER(C.c_int64), C.POINTER(_P), C.POINTER(_P)]),
    "b200_buffer_to_host": (_P, [_P, _P, C.POINTER(C.c_size_t), C.POINTER(_P)]),
    "b200_buffer_dtype": (C.c_int, [_P]),
    "b200_buffer_num_dims": (C.c_size_t, [_P]),
    "b200_buffer_dims": (C.POINTER(C.c_int64), [_P]),
    "b200_buffer_on_device_size": (C.c_size_t, [_P]),
    "b200_buffer_device": (C.c_int, [_P]),
    "b200_buffer_ready_event": (_P, [_P, C.POINTER(_P)]),
    "b200_buffer_copy": (_P, [_P, C.POINTER(_P)]),
    "b200_buffer_delete": (_P, [_P]),
    "b200_buffer_is_deleted": (C.c_int, [_P]),
    "b200_buffer_destroy": (_P, [_P]),
    "b200_buffer_device_pointer": (_P, [_P]),
    "b200_executable_execute": (_P, [_P, C.POINTER(_P), C.c_size_t, C.POINTER(_P), C.POINTER(_P), C.POINTER(_ExecuteOptions)]),
    "b200_event_is_ready": (C.c_int, [_P]),
    "b200_event_await": (_P, [_P]),
    "b200_event_error": (_P, [_P]),
    "b200_event_on_ready": (_P, [_P, EVENT_CALLBACK, _P]),
    "b200_event_destroy": (_P, [_P]),
    "b200_client_synchronize": (_P, [_P]),
    "b200_client_compute_stream": (_P, [_P]),
    "b200_client_launch_count": (C.c_int64, [_P]),
    "b200_client_probe_tf32_mma_rate": (_P, [_P, C.POINTER(C.c_double)]),
    "b200_client_debug_arm_wait_expiry": (_P, [_P, C.c_int]),
    "b200_client_host_syncs": (C.c_longlong, [_P]),
    "b200_device_num_memories": (C.c_int, [_P]),
    "b200_memory_id": (C.c_int, [_P, C.c_int]),
    "b200_memory_kind": (C.c_char_p, [_P, C.c_int]),
    "b200_memory_kind_id": (C.c_int, [_P, C.c_int]),
    "b200_memory_debug_string": (C.c_char_p, [_P, C.c_int]),
    "b200_memory_to_string": (C.c_char_p, [_P, C.c_int]),
    "b200_memory_addressable_by_devices": (_P, [_P, C.c_int, C.POINTER(C.c_int), C.c_size_t, C.POINTER(C.c_size_t)]),
    "b200_buffer_memory": (C.c_int, [_P]),
    "b200_topology_platform_name": (C.c_char_p, [_P]),
    "b200_topology_platform_version": (C.c_char_p, [_P]),
    "b200_topology_num_devices": (C.c_int, [_P]),
    "b200_topology_device_description": (_P, [_P, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_char_p),
                                              C.POINTER(C.c_char_p)]),
    "b200_topology_fingerprint": (C.c_uint64, [_P]),
    "b200_topology_serialize": (_P, [_P, C.POINTER(_P), C.POINTER(C.c_size_t)]),
    "b200_client_default_device_assignment": (_P, [_P, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_size_t]),
    "b200_executable_device_assignment": (_P, [_P, C.POINTER(_P), C.POINTER(C.c_size_t)]),
    "b200_encode_device_assignment": (_P, [C.c_int, C.c_int, C.POINTER(C.c_int64), C.POINTER(_P), C.POINTER(C.c_size_t)]),
    "b200_executable_output_memory_kinds": (_P, [_P, C.POINTER(C.POINTER(C.c_char_p)), C.POINTER(C.POINTER(C.c_size_t)),
                                                 C.POINTER(C.c_size_t)]),
    "b200_device_group_create": (_P, [C.POINTER(C.c_int), C.c_int, C.POINTER(_P)]),
    "b200_device_group_size": (C.c_int, [_P]),
    "b200_device_group_client": (_P, [_P, C.c_int]),
    "b200_device_group_destroy": (_P, [_P]),
    "b200_device_group_compile": (_P, [_P, C.c_char_p, C.c_size_t, C.c_char_p, C.POINTER(_CompileOptions), C.POINTER(_P)]),
    "b200_device_group_execute": (_P, [_P, C.POINTER(_P), C.POINTER(C.POINTER(_P)), C.c_size_t, C.POINTER(C.POINTER(_P)),
                                       C.POINTER(_P), C.POINTER(_ExecuteOptions)]),
    "b200_profiler_create": (_P, [C.c_char_p, C.c_size_t, C.POINTER(_P)]),
    "b200_profiler_start": (_P, [_P]),
    "b200_profiler_stop": (_P, [_P]),
    "b200_profiler_collect_data": (_P, [_P, _P, C.POINTER(C.c_size_t)]),
    "b200_profiler_destroy": (_P, [_P]),
    "b200_client_set_profiling": (_P, [_P, C.c_int]),
    "b200_client_profile_report": (_P, [_P, C.POINTER(_P)]),
    "b200_matmul_f32_static_scratch": (_P, [_P, _P, _P, C.c_int64, C.c_int64, C.c_int64, _P]),
}

_lib = None


def library_path() -> Path:
    """B200_LIBRARY_PATH wins, else the in-tree build next to this file (the
    reference resolves its dylib the same way: src/jax_plugins/mps/__init__.py:37-61)."""
    env = os.environ.get("B200_LIBRARY_PATH")
    if env:
        if not Path(env).exists():
            raise B200Error(f"B200_LIBRARY_PATH is set to '{env}', but the file does not exist.", FAILED_PRECONDITION)
        return Path(env)
    return Path(__file__).resolve().parent / _LIB_NAME


def load_library():
    """dlopen the core and bind every declared symbol. Raises B200Error when
    the extension has not been built — nothing here falls back to the CPU."""
    global _lib
    if _lib is not None:
        return _lib
    p = library_path()
    if not p.exists():
        raise B200Error(f"{p} not found: build it with `python jax-mps_b200/build.py` (there is no CPU fallback)",
                        FAILED_PRECONDITION)
    lib = C.CDLL(str(p))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(err):
    if err:
        lib = load_library()
        msg = lib.b200_error_message(err).decode("utf-8", "replace")
        code = lib.b200_error_get_code(err)
        lib.b200_error_destroy(err)
        raise B200Error(msg, code)


def compile_to_plan(text: str | bytes, num_processes: int = 1, process_index: int = 0, validate: bool = False,
                    disable_fusion: bool = False, slots: bool = False):
    """Host-only compile: returns (plan text, generated CUDA source). Needs no GPU. With `slots` the plan text ends
    with a table of the memory its steps name (arguments, results, temporaries, constants with their bytes)."""
    lib = load_library()
    code = text.encode() if isinstance(text, str) else text
    opts = _CompileOptions(C.sizeof(_CompileOptions), 0, 1 if disable_fusion else 0)
    plan, src = _P(), _P()
    _check(lib.b200_compile_to_plan(code, len(code), C.byref(opts), num_processes, process_index,
                                    (1 if validate else 0) | (2 if slots else 0), C.byref(plan), C.byref(src)))
    out = (C.string_at(plan.value).decode(), C.string_at(src.value).decode())
    lib.b200_string_free(plan)
    lib.b200_string_free(src)
    return out


def encode_device_assignment(device_ids) -> bytes:
    """Serialized xla.DeviceAssignmentProto for device_ids[computation][replica] (needs no device)."""
    comps = [list(row) for row in device_ids]
    reps = len(comps[0]) if comps else 0
    flat = [int(v) for row in comps for v in row]
    arr = (C.c_int64 * max(len(flat), 1))(*flat)
    out, size = _P(), C.c_size_t(0)
    lib = load_library()
    _check(lib.b200_encode_device_assignment(reps, len(comps), arr, C.byref(out), C.byref(size)))
    data = C.string_at(out.value, size.value)
    lib.b200_string_free(out)
    return data


def decode_device_assignment(data: bytes):
    """Reads a serialized xla.DeviceAssignmentProto back: (replica_count, computation_count, device_ids[computation][replica])."""
    def varint(buf, i):
        v, shift = 0, 0
        while True:
            b = buf[i]; i += 1
            v |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                return v, i
    reps = comps = 0
    rows = []
    i = 0
    while i < len(data):
        tag, i = varint(data, i)
        field, wire = tag >> 3, tag & 7
        if wire == 0:
            v, i = varint(data, i)
            if field == 1: reps = v
            elif field == 2: comps = v
        elif wire == 2:
            n, i = varint(data, i)
            sub, i = data[i:i + n], i + n
            if field == 3:
                row, j = [], 0
                while j < len(sub):
                    t, j = varint(sub, j)
                    if t == 0x0A:
                        m, j = varint(sub, j)
                        end = j + m
                        while j < end:
                            v, j = varint(sub, j)
                            row.append(v)
                    elif t == 0x08:
                        v, j = varint(sub, j)
                        row.append(v)
                    else:
                        raise ValueError("unexpected field in ComputationDevice")
                rows.append(row)
        else:
            raise ValueError("unexpected wire type")
    return reps, comps, rows


class Profiler:
    """The profiler-extension stub (PJRT_Profiler_Extension): start / stop are accepted, the trace is empty."""

    def __init__(self, options: bytes = b""):
        h = _P()
        _check(load_library().b200_profiler_create(options, len(options), C.byref(h)))
        self._h = h.value

    def start(self): _check(load_library().b200_profiler_start(self._h))
    def stop(self): _check(load_library().b200_profiler_stop(self._h))

    def collect(self) -> bytes:
        size = C.c_size_t(0)
        _check(load_library().b200_profiler_collect_data(self._h, None, C.byref(size)))
        return b"" if size.value == 0 else bytes(size.value)

    def __del__(self):
        if getattr(self, "_h", None):
            load_library().b200_profiler_destroy(self._h)
            self._h = None


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(NCCL_ID_BYTES)
    _check(load_library().b200_nccl_unique_id(buf))
    return buf.raw


class Event:
    def __init__(self, handle):
        self._h = handle

    def is_ready(self) -> bool:
        return bool(load_library().b200_event_is_ready(self._h))

    def wait(self):
        _check(load_library().b200_event_await(self._h))

    def error(self):
        """None, or the B200Error the event completed with (PJRT_Event_Error)."""
        try:
            _check(load_library().b200_event_error(self._h))
        except B200Error as e:
            return e
        return None

    def on_ready(self, fn):
        """Calls fn(error_or_None) on the completion thread once the event is ready (PJRT_Event_OnReady). The event
        must stay alive until the callback has run."""
        lib = load_library()

        def tramp(err, _arg):
            exc = None
            if err:
                exc = B200Error(lib.b200_error_message(err).decode(), lib.b200_error_get_code(err))
                lib.b200_error_destroy(err)
            fn(exc)
        self._cb = EVENT_CALLBACK(tramp)              # keep the trampoline alive with the event
        _check(lib.b200_event_on_ready(self._h, self._cb, None))

    def __del__(self):
        if getattr(self, "_h", None):
            load_library().b200_event_destroy(self._h)
            self._h = None


class Buffer:
    """A device array (PJRT_Buffer)."""

    def __init__(self, client: "Client", handle):
        self.client, self._h = client, handle

    @property
    def dtype_code(self) -> int:
        return load_library().b200_buffer_dtype(self._h)

    @property
    def dtype(self) -> str:
        return _DT_NAMES[self.dtype_code]

    @property
    def shape(self) -> tuple:
        lib = load_library()
        n = lib.b200_buffer_num_dims(self._h)
        d = lib.b200_buffer_dims(self._h)
        return tuple(int(d[i]) for i in range(n))

    @property
    def nbytes(self) -> int:
        return load_library().b200_buffer_on_device_size(self._h)

    def device_pointer(self) -> int:
        return load_library().b200_buffer_device_pointer(self._h) or 0

    def is_deleted(self) -> bool:
        return bool(load_library().b200_buffer_is_deleted(self._h))

    def delete(self):
        _check(load_library().b200_buffer_delete(self._h))

    def copy(self) -> "Buffer":
        out = _P()
        _check(load_library().b200_buffer_copy(self._h, C.byref(out)))
        return Buffer(self.client, out.value)

    def block_until_ready(self) -> "Buffer":
        ev = _P()
        _check(load_library().b200_buffer_ready_event(self._h, C.byref(ev)))
        Event(ev.value).wait()
        return self

    def to_host_async(self, out: np.ndarray) -> Event:
        """Start a device-to-host copy into `out` (same shape/dtype; pinned memory makes it truly asynchronous)."""
        size = C.c_size_t(out.nbytes)
        ev = _P()
        _check(load_library().b200_buffer_to_host(self._h, out.ctypes.data_as(_P), C.byref(size), C.byref(ev)))
        return Event(ev.value)

    def to_numpy(self) -> np.ndarray:
        """bf16 buffers come back as float32 (exactly representable)."""
        code = self.dtype_code
        out = np.empty(self.shape, dtype=_DT_TO_NP[code])
        size = C.c_size_t(out.nbytes)
        _check(load_library().b200_buffer_to_host(self._h, out.ctypes.data_as(_P), C.byref(size), None))
        if code == BF16:
            return (out.astype(np.uint32) << 16).view(np.float32)
        return out

    def __array__(self, dtype=None, copy=None):
        a = self.to_numpy()
        return a.astype(dtype) if dtype is not None else a

    def __del__(self):
        if getattr(self, "_h", None) and load_library is not None:
            try:
                load_library().b200_buffer_destroy(self._h)
            except Exception:
                pass
            self._h = None


class Executable:
    """A compiled and loaded program (PJRT_LoadedExecutable)."""

    def __init__(self, client: "Client", handle):
        self.client, self._h = client, handle
        lib = load_library()
        self.num_args = lib.b200_executable_num_args(handle)
        self.num_outputs = lib.b200_executable_num_outputs(handle)

    @property
    def name(self) -> str:
        return load_library().b200_executable_name(self._h).decode()

    @property
    def fingerprint(self) -> str:
        return load_library().b200_executable_fingerprint(self._h).decode()

    @property
    def launches_per_execute(self) -> int:
        return load_library().b200_executable_launches_per_execute(self._h)

    @property
    def num_kernels(self) -> int:
        return load_library().b200_executable_num_kernels(self._h)

    @property
    def temp_bytes(self) -> int:
        return load_library().b200_executable_temp_bytes(self._h)

    def plan_text(self) -> str:
        return load_library().b200_executable_plan_text(self._h).decode()

    def device_assignment(self):
        """(replica_count, computation_count, device_ids[computation][replica]) decoded from the serialized proto."""
        out, size = _P(), C.c_size_t(0)
        lib = load_library()
        _check(lib.b200_executable_device_assignment(self._h, C.byref(out), C.byref(size)))
        data = C.string_at(out.value, size.value)
        lib.b200_string_free(out)
        return decode_device_assignment(data)

    def output_memory_kinds(self) -> list:
        kinds, sizes, n = C.POINTER(C.c_char_p)(), C.POINTER(C.c_size_t)(), C.c_size_t(0)
        _check(load_library().b200_executable_output_memory_kinds(self._h, C.byref(kinds), C.byref(sizes), C.byref(n)))
        return [kinds[k][:sizes[k]].decode() for k in range(n.value)]

    def output_info(self, i: int):
        dt, dims, nd = C.c_int(), C.POINTER(C.c_int64)(), C.c_size_t()
        _check(load_library().b200_executable_output_info(self._h, i, C.byref(dt), C.byref(dims), C.byref(nd)))
        return _DT_NAMES[dt.value], tuple(int(dims[k]) for k in range(nd.value))

    def execute(self, args, donate: bool = False, with_event: bool = False):
        """Enqueue one execution; returns the output buffers without waiting (with `with_event`: the buffers and the
        completion event of the execution)."""
        lib = load_library()
        n = len(args)
        arr = (_P * max(n, 1))(*[a._h for a in args])
        outs = (_P * max(self.num_outputs, 1))()
        opts = _ExecuteOptions(C.sizeof(_ExecuteOptions), 1 if donate else 0)
        done = _P()
        _check(lib.b200_executable_execute(self._h, arr, n, outs, C.byref(done) if with_event else None, C.byref(opts)))
        bufs = [Buffer(self.client, outs[k]) for k in range(self.num_outputs)]
        return (bufs, Event(done.value)) if with_event else bufs

    def __call__(self, *arrays):
        bufs = [a if isinstance(a, Buffer) else self.client.buffer_from_host(a) for a in arrays]
        return [b.to_numpy() for b in self.execute(bufs)]

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                load_library().b200_executable_destroy(self._h)
            except Exception:
                pass
            self._h = None


class Client:
    """One process, one B200 (PJRT_Client). For data-parallel jobs every
    process passes its rank, the world size and the shared NCCL id."""

    _owned = True

    @classmethod
    def _wrap(cls, handle) -> "Client":
        """A client owned by somebody else (a device of a DeviceGroup)."""
        c = cls.__new__(cls)
        c._h, c._id, c._owned = handle, None, False
        return c

    def __init__(self, device_ordinal: int = -1, process_index: int = 0, num_processes: int = 1,
                 nccl_id: bytes | None = None):
        lib = load_library()
        self._id = nccl_id
        opts = _ClientOptions(C.sizeof(_ClientOptions), device_ordinal, process_index, num_processes, nccl_id, 0)
        h = _P()
        _check(lib.b200_client_create(C.byref(opts), C.byref(h)))
        self._h = h.value

    @property
    def platform(self) -> str:
        return load_library().b200_client_platform_name(self._h).decode()

    @property
    def platform_version(self) -> str:
        return load_library().b200_client_platform_version(self._h).decode()

    @property
    def process_index(self) -> int:
        return load_library().b200_client_process_index(self._h)

    def device_count(self) -> int:
        return load_library().b200_client_device_count(self._h)

    def device_kind(self) -> str:
        return load_library().b200_device_kind(self._h).decode()

    def device_debug_string(self) -> str:
        return load_library().b200_device_debug_string(self._h).decode()

    def memory_stats(self) -> MemoryStats:
        st = MemoryStats(C.sizeof(MemoryStats))
        _check(load_library().b200_device_memory_stats(self._h, C.byref(st)))
        return st

    def compile(self, text: str | bytes, disable_fusion: bool = False) -> Executable:
        """StableHLO module text -> loaded executable (compile_and_load)."""
        code = text.encode() if isinstance(text, str) else text
        opts = _CompileOptions(C.sizeof(_CompileOptions), 0, 1 if disable_fusion else 0)
        h = _P()
        _check(load_library().b200_client_compile(self._h, code, len(code), b"mlir", C.byref(opts), C.byref(h)))
        return Executable(self, h.value)

    compile_and_load = compile

    def buffer_from_host(self, array, dtype: str | None = None) -> Buffer:
        """Host array -> device buffer. `dtype='bf16'` converts float32 input to bfloat16 on the host (a uint16 array
        is taken as bfloat16 bit patterns as it is)."""
        a = np.asarray(array)
        if dtype == "bf16":
            if a.dtype != np.uint16:                      # uint16 input is taken as bfloat16 bit patterns
                from .shlo.builder import f32_to_bf16_bits
                a = f32_to_bf16_bits(a.astype(np.float32)).reshape(a.shape)
            code = BF16
        else:
            if dtype is not None:
                a = a.astype(_DT_TO_NP[_NAME_TO_DT[dtype]])
            if a.dtype not in _NP_TO_DT:
                raise B200Error(f"unsupported host dtype {a.dtype}", INVALID_ARGUMENT)
            code = _NP_TO_DT[a.dtype]
        dims = (C.c_int64 * max(a.ndim, 1))(*a.shape)
        strides = (C.c_int64 * max(a.ndim, 1))(*a.strides)
        h = _P()
        ptr = a.ctypes.data_as(_P) if a.size else None
        _check(load_library().b200_buffer_from_host(self._h, ptr, code, dims, a.ndim, strides, C.byref(h), None))
        buf = Buffer(self, h.value)
        buf._host = a            # a pinned source is read asynchronously: keep it alive with the buffer
        return buf

    device_put = buffer_from_host

    def synchronize(self):
        _check(load_library().b200_client_synchronize(self._h))

    def compute_stream(self) -> int:
        return load_library().b200_client_compute_stream(self._h) or 0

    def set_profiling(self, on: bool):
        _check(load_library().b200_client_set_profiling(self._h, 1 if on else 0))

    def profile_report(self) -> list:
        """Per-step device times accumulated while profiling was on: [{'kind','key','ms','count'}]."""
        import json
        out = _P()
        lib = load_library()
        _check(lib.b200_client_profile_report(self._h, C.byref(out)))
        txt = C.string_at(out.value).decode()
        lib.b200_string_free(out)
        return json.loads(txt)

    def memories(self) -> list:
        """[{id, kind, debug_string, to_string, devices}] for the memory spaces of this client's device."""
        lib = load_library()
        out = []
        for k in range(lib.b200_device_num_memories(self._h)):
            ids, n = (C.c_int * 8)(), C.c_size_t(0)
            _check(lib.b200_memory_addressable_by_devices(self._h, k, ids, 8, C.byref(n)))
            out.append({"id": lib.b200_memory_id(self._h, k), "kind": lib.b200_memory_kind(self._h, k).decode(),
                        "debug_string": lib.b200_memory_debug_string(self._h, k).decode(),
                        "to_string": lib.b200_memory_to_string(self._h, k).decode(), "devices": list(ids[:n.value])})
        return out

    def topology(self) -> dict:
        lib = load_library()
        devs = []
        for k in range(lib.b200_topology_num_devices(self._h)):
            i, p, kind, dbg = C.c_int(), C.c_int(), C.c_char_p(), C.c_char_p()
            _check(lib.b200_topology_device_description(self._h, k, C.byref(i), C.byref(p), C.byref(kind), C.byref(dbg)))
            devs.append({"id": i.value, "process_index": p.value, "kind": kind.value.decode(), "debug_string": dbg.value.decode()})
        return {"platform_name": lib.b200_topology_platform_name(self._h).decode(),
                "platform_version": lib.b200_topology_platform_version(self._h).decode(),
                "fingerprint": lib.b200_topology_fingerprint(self._h), "devices": devs}

    def default_device_assignment(self, num_replicas: int, num_partitions: int) -> list:
        n = num_replicas * num_partitions
        arr = (C.c_int * max(n, 1))()
        _check(load_library().b200_client_default_device_assignment(self._h, num_replicas, num_partitions, arr, n))
        return [[arr[r * num_partitions + p] for p in range(num_partitions)] for r in range(num_replicas)]

    def debug_arm_wait_expiry(self, polls: int = 1000):
        """Test hook: the next execution starts with a bounded device-side wait that runs out."""
        _check(load_library().b200_client_debug_arm_wait_expiry(self._h, polls))

    def host_syncs(self) -> int:
        """Stream synchronisations inside executions so far (predicates of `while` / indices of `case` read by the host)."""
        return int(load_library().b200_client_host_syncs(self._h))

    def probe_tf32_mma_rate(self) -> float:
        """TFLOP/s of the TF32 tensor-core MMA on this device (issue loop alone); the 3xTF32 fp32 path tops out at a third."""
        out = C.c_double(0.0)
        _check(load_library().b200_client_probe_tf32_mma_rate(self._h, C.byref(out)))
        return out.value

    def launch_count(self) -> int:
        return load_library().b200_client_launch_count(self._h)

    def matmul_static_scratch(self, a: Buffer, b: Buffer, out: Buffer):
        """out[m,n] = a[m,k] @ b[k,n] (float32 buffers of this client) through the entry point that allocates
        nothing: the K-split partial sums use an 8 MiB array inside the library (m * n <= 1048576). Enqueued on
        the compute stream after the operands are ready; calls share the array, so do not overlap them."""
        (m, k), (k2, n) = a.shape, b.shape
        if k != k2 or out.shape != (m, n) or not (a.dtype == b.dtype == out.dtype == "f32"):
            raise B200Error("matmul_static_scratch wants f32 buffers a[m,k], b[k,n], out[m,n]", 3)
        for x in (a, b, out):
            x.block_until_ready()
        _check(load_library().b200_matmul_f32_static_scratch(a.device_pointer(), b.device_pointer(),
                                                             out.device_pointer(), m, n, k, self.compute_stream()))

    def close(self):
        if getattr(self, "_h", None) and self._owned:
            load_library().b200_client_destroy(self._h)
            self._h = None


class DeviceGroup:
    """Several local GPUs as the devices of this one process (the per-device lists of PJRT_LoadedExecutable_Execute):
    `devices[d]` is the client of device d (make buffers through it), `compile` gives one executable per device and
    `execute` takes one argument list per device."""

    def __init__(self, ordinals=None, num_devices: int | None = None):
        lib = load_library()
        n = len(ordinals) if ordinals is not None else int(num_devices)
        arr = (C.c_int * n)(*ordinals) if ordinals is not None else None
        h = _P()
        _check(lib.b200_device_group_create(arr, n, C.byref(h)))
        self._h = h.value
        self.devices = [Client._wrap(lib.b200_device_group_client(self._h, d)) for d in range(n)]

    def compile(self, text: str | bytes) -> list:
        code = text.encode() if isinstance(text, str) else text
        opts = _CompileOptions(C.sizeof(_CompileOptions), 0, 0)
        n = len(self.devices)
        exes = (_P * n)()
        _check(load_library().b200_device_group_compile(self._h, code, len(code), b"mlir", C.byref(opts), exes))
        return [Executable(self.devices[d], exes[d]) for d in range(n)]

    def execute(self, exes, argument_lists, donate: bool = False):
        """argument_lists[d][i]: argument i on device d. Returns (output_lists[d][k], device_complete_events[d])."""
        n = len(self.devices)
        num_args = len(argument_lists[0]) if argument_lists else 0
        exe_arr = (_P * n)(*[e._h for e in exes])
        arg_rows = [(_P * max(num_args, 1))(*[a._h for a in argument_lists[d]]) for d in range(n)]
        args = (C.POINTER(_P) * n)(*[C.cast(r, C.POINTER(_P)) for r in arg_rows])
        num_out = exes[0].num_outputs
        out_rows = [(_P * max(num_out, 1))() for _ in range(n)]
        outs = (C.POINTER(_P) * n)(*[C.cast(r, C.POINTER(_P)) for r in out_rows])
        events = (_P * n)()
        opts = _ExecuteOptions(C.sizeof(_ExecuteOptions), 1 if donate else 0)
        _check(load_library().b200_device_group_execute(self._h, exe_arr, args, num_args, outs, events, C.byref(opts)))
        return ([[Buffer(self.devices[d], out_rows[d][k]) for k in range(num_out)] for d in range(n)],
                [Event(events[d]) for d in range(n)])

    def close(self):
        if getattr(self, "_h", None):
            load_library().b200_device_group_destroy(self._h)
            self._h = None
            for c in self.devices:
                c._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

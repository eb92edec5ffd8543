/*
 * b200_core.h — C ABI of the B200 execution core behind the PJRT plugin.
 *
 * This is the drop-in boundary for the hot path of the reference plugin
 * (tillahoffmann/jax-mps): create a client, move host arrays to the device,
 * compile a StableHLO module, execute it, read results back. Every function
 * below names the reference entry point it stands in for (paths inside the
 * reference project). The PJRT veneer (GetPjrtApi function table,
 * src/pjrt_plugin/pjrt_api.cc:232-400) is a thin adapter over these calls;
 * it is built only where xla/pjrt/c/pjrt_c_api.h is available.
 *
 * Conventions (same as the reference's PJRT layer, pjrt_client.cc:17-31,
 * pjrt_types.h:137-140):
 *   - every call returns NULL on success or a heap b200_error* the caller
 *     frees with b200_error_destroy; no C++ exception crosses the boundary;
 *   - objects returned through out-parameters are owned by the caller and
 *     released with the matching *_destroy;
 *   - all calls are thread-safe; work on a device is stream-ordered.
 *
 * One process drives one GPU (data-parallel jobs run one process per GPU and
 * pass every process the same NCCL unique id); there is no CPU fallback: a
 * call that needs the GPU fails with B200_FAILED_PRECONDITION when no device
 * or no CUDA driver is present, and an unsupported operation is a compile
 * error.
 */
#ifndef B200_CORE_H_
#define B200_CORE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#pragma GCC visibility push(default)

typedef struct b200_client b200_client;
typedef struct b200_executable b200_executable;
typedef struct b200_buffer b200_buffer;
typedef struct b200_event b200_event;
typedef struct b200_error b200_error;

typedef enum {
  B200_OK = 0,
  B200_CANCELLED = 1,
  B200_UNKNOWN = 2,
  B200_INVALID_ARGUMENT = 3,
  B200_NOT_FOUND = 5,
  B200_RESOURCE_EXHAUSTED = 8,
  B200_FAILED_PRECONDITION = 9,
  B200_UNIMPLEMENTED = 12,
  B200_INTERNAL = 13
} b200_error_code;

/* Element types (the set the reference maps in PjrtDtypeToMlx, src/pjrt_plugin/mlx_buffer.cc:14-53,
 * plus F64; complex types are not supported). */
typedef enum {
  B200_INVALID = 0,
  B200_PRED = 1,
  B200_S8 = 2,
  B200_S16 = 3,
  B200_S32 = 4,
  B200_S64 = 5,
  B200_U8 = 6,
  B200_U16 = 7,
  B200_U32 = 8,
  B200_U64 = 9,
  B200_F16 = 10,
  B200_F32 = 11,
  B200_F64 = 12,
  B200_BF16 = 13
} b200_dtype;

/* ---- errors: PJRT_Error_Destroy / _Message / _GetCode (pjrt_client.cc:17-31) ---- */
void b200_error_destroy(b200_error* err);
const char* b200_error_message(const b200_error* err);
b200_error_code b200_error_get_code(const b200_error* err);

/* ---- client: PJRT_Client_Create (pjrt_client.cc:70-83), MlxClient (mlx_client.cc:19-66) ---- */
#define B200_NCCL_ID_BYTES 128
typedef struct {
  size_t struct_size;
  int device_ordinal;        /* CUDA device this process drives; -1 = LOCAL_RANK env or 0 */
  int process_index;         /* rank of this process in the data-parallel job */
  int num_processes;         /* 1 = single GPU */
  const char* nccl_unique_id;/* B200_NCCL_ID_BYTES bytes shared by all processes, or NULL when num_processes == 1 */
  size_t pool_release_threshold; /* bytes kept cached by the stream-ordered pool; 0 = keep everything */
} b200_client_options;

b200_error* b200_client_create(const b200_client_options* options, b200_client** client);
b200_error* b200_client_destroy(b200_client* client);                       /* PJRT_Client_Destroy */
const char* b200_client_platform_name(const b200_client* client);           /* PJRT_Client_PlatformName */
const char* b200_client_platform_version(const b200_client* client);        /* PJRT_Client_PlatformVersion */
int b200_client_process_index(const b200_client* client);                   /* PJRT_Client_ProcessIndex */
int b200_client_device_count(const b200_client* client);                    /* PJRT_Client_Devices: all processes */
int b200_client_addressable_device_count(const b200_client* client);        /* PJRT_Client_AddressableDevices */
/* Rank 0 makes the id that every process passes to b200_client_create. */
b200_error* b200_nccl_unique_id(char out[B200_NCCL_ID_BYTES]);

/* ---- device: pjrt_device.cc:12-147 ---- */
int b200_device_id(const b200_client* client);                               /* global id == process_index */
int b200_device_local_hardware_id(const b200_client* client);                /* CUDA ordinal */
const char* b200_device_kind(const b200_client* client);                     /* "NVIDIA B200" */
const char* b200_device_debug_string(const b200_client* client);
typedef struct {
  size_t struct_size;
  int64_t bytes_in_use;
  int64_t peak_bytes_in_use; int peak_bytes_in_use_is_set;
  int64_t bytes_limit; int bytes_limit_is_set;
  int64_t pool_bytes; int pool_bytes_is_set;
  int64_t peak_pool_bytes; int peak_pool_bytes_is_set;
  int64_t num_allocs; int num_allocs_is_set;
  int64_t largest_alloc_size; int largest_alloc_size_is_set;
} b200_memory_stats;
b200_error* b200_device_memory_stats(b200_client* client, b200_memory_stats* stats);   /* PJRT_Device_MemoryStats */

/* ---- memory spaces: pjrt_memory.cc:10-48, PJRT_Device_AddressableMemories / _DefaultMemory (pjrt_device.cc:88-109),
 *      PJRT_Client_AddressableMemories. Every device has one memory space, its HBM, of kind "device". ---- */
int b200_device_num_memories(const b200_client* client);                     /* 1 */
int b200_memory_id(const b200_client* client, int memory_index);             /* PJRT_Memory_Id: == the device's id */
const char* b200_memory_kind(const b200_client* client, int memory_index);   /* PJRT_Memory_Kind: "device" */
int b200_memory_kind_id(const b200_client* client, int memory_index);        /* PJRT_Memory_Kind_Id */
const char* b200_memory_debug_string(const b200_client* client, int memory_index);   /* PJRT_Memory_DebugString */
const char* b200_memory_to_string(const b200_client* client, int memory_index);      /* PJRT_Memory_ToString */
/* PJRT_Memory_AddressableByDevices: writes the ids of the devices that address the memory (one: its own device). */
b200_error* b200_memory_addressable_by_devices(const b200_client* client, int memory_index, int* device_ids, size_t capacity,
                                               size_t* num_devices);

/* ---- topology: PJRT_Client_TopologyDescription and PJRT_TopologyDescription_* (pjrt_topology.cc:10-70) ---- */
const char* b200_topology_platform_name(const b200_client* client);
const char* b200_topology_platform_version(const b200_client* client);
int b200_topology_num_devices(const b200_client* client);                    /* all processes of the job */
/* Device `index` of the job: its id (== index), the process that drives it, kind and debug string (owned by the client). */
b200_error* b200_topology_device_description(const b200_client* client, int index, int* id, int* process_index,
                                             const char** kind, const char** debug_string);
/* PJRT_TopologyDescription_Fingerprint: a hash of platform, device kind and device count (the reference returns a
 * constant for its one device); jax's compilation cache keys on it. */
uint64_t b200_topology_fingerprint(const b200_client* client);
/* PJRT_TopologyDescription_Serialize: B200_UNIMPLEMENTED, as in the reference. */
b200_error* b200_topology_serialize(const b200_client* client, char** bytes, size_t* size);

/* ---- device assignment: PJRT_Client_DefaultDeviceAssignment (pjrt_client.cc:259-265),
 *      PJRT_LoadedExecutable_GetDeviceAssignment (pjrt_executable.cc:290-313) ---- */
/* Fills assignment[replica * num_partitions + partition] with device ids 0, 1, ... in that order; fails when the job
 * has fewer devices than replicas * partitions. */
b200_error* b200_client_default_device_assignment(const b200_client* client, int num_replicas, int num_partitions,
                                                  int* assignment, size_t assignment_size);
/* Serialized xla.DeviceAssignmentProto (src/proto/device_assignment.proto:9-17) of the executable: replica_count,
 * computation_count (the partitions) and one ComputationDevice per partition listing the device of every replica.
 * `*bytes` is malloc'd: release it with b200_string_free. */
b200_error* b200_executable_device_assignment(const b200_executable* exe, char** bytes, size_t* size);
/* The same encoding for any assignment (device_ids[computation * replica_count + replica]); needs no device. */
b200_error* b200_encode_device_assignment(int replica_count, int computation_count, const int64_t* device_ids, char** bytes,
                                          size_t* size);
/* PJRT_Executable_OutputMemoryKinds (pjrt_executable.cc:66-99): one kind string per output ("device"); the arrays are
 * owned by the executable. */
b200_error* b200_executable_output_memory_kinds(const b200_executable* exe, const char* const** kinds, const size_t** kind_sizes,
                                                size_t* num_outputs);

/* ---- profiler extension stub: pjrt_profiler.cc:17-125. jaxlib probes the plugin for a profiler; like the reference this
 *      one accepts create / start / stop and hands back an empty trace. Device timings come from
 *      b200_client_set_profiling. ---- */
typedef struct b200_profiler b200_profiler;
b200_error* b200_profiler_create(const char* options, size_t options_size, b200_profiler** profiler);
b200_error* b200_profiler_start(b200_profiler* profiler);
b200_error* b200_profiler_stop(b200_profiler* profiler);
/* buffer == NULL: only *size is written (0: nothing was collected). */
b200_error* b200_profiler_collect_data(b200_profiler* profiler, void* buffer, size_t* size);
b200_error* b200_profiler_destroy(b200_profiler* profiler);

/* ---- compile: PJRT_Client_Compile (pjrt_client.cc:179-257) ---- */
typedef struct {
  size_t struct_size;
  int num_partitions;        /* 0 = take mhlo.num_partitions from the module */
  int disable_fusion;        /* one kernel per op (debugging; env B200_NO_FUSE=1 does the same) */
} b200_compile_options;
/* `format` is "mlir" (StableHLO text; generic operation form, or custom assembly for common ops). */
b200_error* b200_client_compile(b200_client* client, const char* code, size_t code_size, const char* format,
                                const b200_compile_options* options, b200_executable** executable);
b200_error* b200_executable_destroy(b200_executable* exe);                   /* PJRT_LoadedExecutable_Destroy */
const char* b200_executable_name(const b200_executable* exe);                /* PJRT_Executable_Name */
const char* b200_executable_fingerprint(const b200_executable* exe);         /* PJRT_Executable_Fingerprint */
int b200_executable_num_replicas(const b200_executable* exe);
int b200_executable_num_partitions(const b200_executable* exe);
size_t b200_executable_num_args(const b200_executable* exe);
size_t b200_executable_num_outputs(const b200_executable* exe);              /* PJRT_Executable_NumOutputs */
/* PJRT_Executable_OutputElementTypes / OutputDimensions; `dims` points at storage owned by the executable. */
b200_error* b200_executable_output_info(const b200_executable* exe, size_t index, b200_dtype* dtype,
                                        const int64_t** dims, size_t* num_dims);
b200_error* b200_executable_arg_info(const b200_executable* exe, size_t index, b200_dtype* dtype,
                                     const int64_t** dims, size_t* num_dims);
/* Kernel launches one execution performs (-1 when it depends on data), generated kernel count, arena bytes. */
int64_t b200_executable_launches_per_execute(const b200_executable* exe);
int64_t b200_executable_num_kernels(const b200_executable* exe);
int64_t b200_executable_temp_bytes(const b200_executable* exe);
/* Text of the kernel plan (what B200_DUMP_PLAN prints); owned by the executable. */
const char* b200_executable_plan_text(const b200_executable* exe);

/* Host-only compilation (no device needed): parses and plans the module and returns the plan text and
 * the generated CUDA source as malloc'd strings the caller releases with b200_string_free. With
 * `validate_kernels` & 1 the source is also compiled by NVRTC for sm_100a, so generator mistakes surface as
 * an error here; with `validate_kernels` & 2 the plan text ends with a table of the memory its steps name
 * (arguments, results, temporaries, constants with their bytes). Stands in for the reference's IR dump (JAX_MPS_DUMP_OPTIMIZED_IR,
 * src/pjrt_plugin/stablehlo_parser.cc:210-232), which its fusion tests read. */
b200_error* b200_compile_to_plan(const char* code, size_t code_size, const b200_compile_options* options,
                                 int num_processes, int process_index, int validate_kernels, char** plan_text,
                                 char** cuda_source);
void b200_string_free(char* s);

/* ---- buffers: PJRT_Client_BufferFromHostBuffer (pjrt_client.cc:267-322), pjrt_buffer.cc:13-188 ---- */
/* byte_strides may be NULL (dense row-major). `done_with_host_buffer` (may be NULL) becomes ready when
 * `data` may be reused. */
b200_error* b200_buffer_from_host(b200_client* client, const void* data, b200_dtype dtype, const int64_t* dims,
                                  size_t num_dims, const int64_t* byte_strides, b200_buffer** buffer,
                                  b200_event** done_with_host_buffer);
/* dst == NULL: only *dst_size is written (bytes needed). Otherwise starts an asynchronous copy; *event
 * (may be NULL: then the call blocks) is ready when dst holds the data. */
b200_error* b200_buffer_to_host(b200_buffer* buffer, void* dst, size_t* dst_size, b200_event** event);
b200_dtype b200_buffer_dtype(const b200_buffer* buffer);
size_t b200_buffer_num_dims(const b200_buffer* buffer);
const int64_t* b200_buffer_dims(const b200_buffer* buffer);
size_t b200_buffer_on_device_size(const b200_buffer* buffer);
int b200_buffer_device(const b200_buffer* buffer);
int b200_buffer_memory(const b200_buffer* buffer);                              /* PJRT_Buffer_Memory: the memory's id */
b200_error* b200_buffer_ready_event(b200_buffer* buffer, b200_event** event);   /* PJRT_Buffer_ReadyEvent */
b200_error* b200_buffer_copy(b200_buffer* buffer, b200_buffer** copy);          /* PJRT_Buffer_CopyToDevice (same device) */
b200_error* b200_buffer_delete(b200_buffer* buffer);                            /* PJRT_Buffer_Delete: frees device memory */
int b200_buffer_is_deleted(const b200_buffer* buffer);
b200_error* b200_buffer_destroy(b200_buffer* buffer);
/* Raw device address (PJRT_Buffer_UnsafePointer). */
void* b200_buffer_device_pointer(const b200_buffer* buffer);

/* ---- execute: PJRT_LoadedExecutable_Execute (pjrt_executable.cc:178-258) ---- */
typedef struct {
  size_t struct_size;
  int donate_arguments;      /* honour tf.aliasing_output: a donated argument is consumed. Its buffer is left deleted
                                and its memory returns to the stream-ordered pool behind this execution; results
                                are fresh allocations (they never share storage with an argument) */
} b200_execute_options;
/* `outputs` is a caller-allocated array of b200_executable_num_outputs pointers. `done` (may be NULL)
 * becomes ready when all outputs are computed. The call returns after enqueueing. Device-side waits are bounded: if
 * one runs out during the execution, b200_event_await / _error / _on_ready of `done`, and of the events of reads of
 * its outputs (b200_buffer_to_host, b200_buffer_ready_event), report B200_INTERNAL once the work has finished. The outputs of one call share
 * two device allocations (small and large results); each is deleted on its own and a shared allocation is
 * released with its last output. */
b200_error* b200_executable_execute(b200_executable* exe, b200_buffer* const* args, size_t num_args,
                                    b200_buffer** outputs, b200_event** done, const b200_execute_options* options);

/* ---- several GPUs as the devices of one process: the per-device lists of PJRT_LoadedExecutable_Execute
 *      (pjrt_executable.cc:178-258: argument_lists[d], output_lists[d], device_complete_events[d]; the reference reads
 *      index 0 only, it has one device) ---- */
typedef struct b200_device_group b200_device_group;
/* One client per listed CUDA ordinal (NULL: 0 .. num_devices - 1), their NCCL communicators made together in this
 * process. Device d of the group has id d. Buffers are made through b200_device_group_client(group, d). */
b200_error* b200_device_group_create(const int* ordinals, int num_devices, b200_device_group** group);
int b200_device_group_size(const b200_device_group* group);
b200_client* b200_device_group_client(const b200_device_group* group, int device);      /* owned by the group */
b200_error* b200_device_group_destroy(b200_device_group* group);
/* Compiles the module once per device (partition d of num_devices); `executables` has room for one per device. */
b200_error* b200_device_group_compile(b200_device_group* group, const char* code, size_t code_size, const char* format,
                                      const b200_compile_options* options, b200_executable** executables);
/* argument_lists[d][i] is argument i on device d, output_lists[d] a caller-allocated array of
 * b200_executable_num_outputs pointers, device_complete_events[d] (the array may be NULL) the completion event of
 * device d. Returns after every device's plan has been enqueued. */
b200_error* b200_device_group_execute(b200_device_group* group, b200_executable* const* executables,
                                      b200_buffer* const* const* argument_lists, size_t num_args, b200_buffer** const* output_lists,
                                      b200_event** device_complete_events, const b200_execute_options* options);

/* ---- events: pjrt_event.cc:101-193 ---- */
int b200_event_is_ready(b200_event* event);
b200_error* b200_event_await(b200_event* event);
b200_error* b200_event_error(b200_event* event);
typedef void (*b200_event_callback)(b200_error* error, void* user_arg);   /* the callback owns `error` */
b200_error* b200_event_on_ready(b200_event* event, b200_event_callback callback, void* user_arg);
b200_error* b200_event_destroy(b200_event* event);

/* Blocks until everything enqueued on the client's streams has finished. */
b200_error* b200_client_synchronize(b200_client* client);
/* CUDA stream the client launches on (cudaStream_t), for callers that time with events. */
void* b200_client_compute_stream(b200_client* client);
/* Per-step device timing (the reference's MPS_PROFILE counterpart, src/pjrt_plugin/mlx_executable.cc:381-454):
 * while enabled every plan step is bracketed by CUDA events on the compute stream and executions
 * synchronise at their end. b200_client_profile_report returns a malloc'd JSON array of
 * {"kind","key","ms","count"} accumulated since the last report (release with b200_string_free). */
b200_error* b200_client_set_profiling(b200_client* client, int enabled);
b200_error* b200_client_profile_report(b200_client* client, char** json);
/* Test hook: the next execution on this client starts with a kernel that waits, with a budget of `polls` polls, on a
 * barrier nothing arrives at. The wait runs out (nothing hangs, nothing faults) and the execution reports the failure
 * the way an expired tensor-core pipeline wait does. No counterpart in the reference. */
b200_error* b200_client_debug_arm_wait_expiry(b200_client* client, int polls);
/* How many times executions on this client have synchronised the compute stream to read a `while` predicate or a
 * `case` index back to the host (the reference does so on every iteration of a data-dependent loop,
 * src/pjrt_plugin/ops/control_flow.cc:505-536). Loops and cases whose bodies only launch kernels and device copies run
 * as conditional CUDA-graph nodes from their second execution on and add nothing here. A data-dependent loop that is
 * resident on the device ends with an error (reported like an expired device-side wait) once it has run for
 * B200_WHILE_TIME_LIMIT_S seconds (default 30). */
long long b200_client_host_syncs(const b200_client* client);
/* Measures the rate of tcgen05.mma.kind::tf32 on the client's device (TFLOP/s; issue loop alone, operands resident in
 * shared memory). The fp32-accurate contraction kernels issue three such MMAs per product: their ceiling is a third of
 * this figure. A measurement aid with no counterpart in the reference (its numbers come from MPS_PROFILE,
 * src/pjrt_plugin/mlx_executable.cc:381-454). */
b200_error* b200_client_probe_tf32_mma_rate(b200_client* client, double* tflops);
/* Total kernels launched by this client since creation (generated + static + collectives). */
int64_t b200_client_launch_count(const b200_client* client);

/* Split-K fp32 matrix product that allocates nothing: c[m,n] = a[m,k] * b[k,n], dense row-major DEVICE pointers,
 * enqueued on `cuda_stream` (a cudaStream_t; NULL = the default stream) of the current device. It has no
 * counterpart in the reference. It is for callers that must not allocate device memory when they need a product:
 * code inside a memory-pool callback or under a framework allocator's lock, and loops that may not take the
 * driver's allocation lock. The partial sums of the K splits live in an 8 MiB array inside the library image (held
 * by every GPU that loads the library, until exit), so 2 * m * n floats must fit in 8 MiB (m * n <= 1048576);
 * larger products are refused with B200_INVALID_ARGUMENT. The first call on each device loads the
 * library's device image (with the array) and looks up the array's device address, which does take the driver's
 * locks: make that call ahead of time, before entering the context that may not allocate and before any stream
 * capture. All calls share the array and it keeps the last
 * call's contents (each call overwrites the part it reads, nothing needs to start at zero): calls that overlap
 * in time on one device, from different streams or threads, race - serialise them. */
b200_error* b200_matmul_f32_static_scratch(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                                           void* cuda_stream);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
#endif /* B200_CORE_H_ */

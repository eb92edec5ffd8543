// Client, buffers, events, executable loading and plan execution, and the C
// ABI declared in include/b200_core.h.
//
// Reference counterparts: MlxClient (src/pjrt_plugin/mlx_client.cc:19-66),
// MlxBuffer (mlx_buffer.cc:104-335), PJRT_Event + CompletionService
// (pjrt_event.cc:28-150), MlxExecutable::Execute (mlx_executable.cc:799-1008)
// and the PJRT entry points in pjrt_client.cc / pjrt_buffer.cc /
// pjrt_executable.cc. Differences by design: one CUDA device per process,
// three streams (compute, host-to-device, device-to-host) ordered by events
// instead of one process-wide mutex around a lazy graph, a stream-ordered
// memory pool (cudaMallocAsync), pinned staging for pageable host arrays, a
// static kernel plan instead of trace-and-replay, NCCL for all_reduce.
#include <sstream>
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <nvrtc.h>

#include <atomic>
#include <condition_variable>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <thread>

#include "../../include/b200_core.h"
#include "kernels.h"
#include "plan.h"

using namespace b200;

struct b200_error {
  std::string message;
  b200_error_code code;
};

namespace {

b200_error* make_error(b200_error_code code, const std::string& msg) { return new b200_error{msg, code}; }

#define CUDA_TRY(expr)                                                                                   \
  do {                                                                                                   \
    cudaError_t _e = (expr);                                                                             \
    if (_e != cudaSuccess)                                                                               \
      return make_error(_e == cudaErrorMemoryAllocation ? B200_RESOURCE_EXHAUSTED : B200_INTERNAL,       \
                        std::string(#expr) + " failed: " + cudaGetErrorString(_e));                      \
  } while (0)

int log_level() {
  static int lvl = [] {
    const char* e = getenv("B200_LOG_LEVEL");
    return e ? atoi(e) : 1;
  }();
  return lvl;
}
void logf(int lvl, const char* fmt, ...) {
  if (lvl > log_level()) return;
  va_list ap;
  va_start(ap, fmt);
  fprintf(stderr, "[b200] ");
  vfprintf(stderr, fmt, ap);
  fprintf(stderr, "\n");
  va_end(ap);
}

// ---- driver / NVRTC / NCCL entry points, resolved at first use ----------------
struct DriverApi {
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void**, void**) = nullptr;
  CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;   // optional
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  std::string error;
  bool ok = false;
};

DriverApi& driver() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [&](const char* name, void** fn) {
      cudaDriverEntryPointQueryResult st;
      cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &st);
      if (e != cudaSuccess || st != cudaDriverEntryPointSuccess || !*fn) {
        api.error = std::string("CUDA driver entry point ") + name + " not available";
        return false;
      }
      return true;
    };
    api.ok = get("cuModuleLoadData", (void**)&api.ModuleLoadData) && get("cuModuleUnload", (void**)&api.ModuleUnload) &&
             get("cuModuleGetFunction", (void**)&api.ModuleGetFunction) &&
             get("cuLaunchKernel", (void**)&api.LaunchKernel) && get("cuGetErrorString", (void**)&api.GetErrorString);
    if (api.ok) {
      const std::string keep = api.error;
      if (!get("cuLaunchKernelEx", (void**)&api.LaunchKernelEx)) { api.LaunchKernelEx = nullptr; api.error = keep; }
    }
  });
  return api;
}

struct NvrtcApi {
  nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*);
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char*);
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char*);
  nvrtcResult (*DestroyProgram)(nvrtcProgram*);
  const char* (*GetErrorString)(nvrtcResult);
  std::string error;
  bool ok = false;
};

NvrtcApi& nvrtc() {
  static NvrtcApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = nullptr;
    const char* env = getenv("B200_NVRTC_PATH");
    const char* names[] = {env, "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so.12", "libnvrtc.so"};
    for (const char* n : names) {
      if (!n) continue;
      h = dlopen(n, RTLD_NOW | RTLD_LOCAL);
      if (h) break;
    }
    if (!h) {
      api.error = "cannot load libnvrtc.so.12 (set B200_NVRTC_PATH)";
      return;
    }
    bool ok = true;
    auto get = [&](const char* name, void** fn) {
      *fn = dlsym(h, name);
      if (!*fn) { ok = false; api.error = std::string("libnvrtc lacks ") + name; }
    };
    get("nvrtcCreateProgram", (void**)&api.CreateProgram);
    get("nvrtcCompileProgram", (void**)&api.CompileProgram);
    get("nvrtcGetCUBINSize", (void**)&api.GetCUBINSize);
    get("nvrtcGetCUBIN", (void**)&api.GetCUBIN);
    get("nvrtcGetProgramLogSize", (void**)&api.GetProgramLogSize);
    get("nvrtcGetProgramLog", (void**)&api.GetProgramLog);
    get("nvrtcDestroyProgram", (void**)&api.DestroyProgram);
    get("nvrtcGetErrorString", (void**)&api.GetErrorString);
    api.ok = ok;
  });
  return api;
}

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;   // optional
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*);
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*CommAbort)(ncclComm_t);
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
  ncclResult_t (*GroupStart)();
  ncclResult_t (*GroupEnd)();
  const char* (*GetErrorString)(ncclResult_t);
  std::string error;
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = nullptr;
    const char* env = getenv("B200_NCCL_PATH");
    const char* names[] = {env, "libnccl.so.2", "/usr/lib/x86_64-linux-gnu/libnccl.so.2"};
    for (const char* n : names) {
      if (!n) continue;
      h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (h) break;
    }
    if (!h) {
      api.error = "cannot load libnccl.so.2 (set B200_NCCL_PATH)";
      return;
    }
    bool ok = true;
    auto get = [&](const char* name, void** fn) {
      *fn = dlsym(h, name);
      if (!*fn) { ok = false; api.error = std::string("libnccl lacks ") + name; }
    };
    get("ncclGetUniqueId", (void**)&api.GetUniqueId);
    get("ncclCommInitRank", (void**)&api.CommInitRank);
    *(void**)&api.CommInitRankConfig = dlsym(h, "ncclCommInitRankConfig");      // optional (NCCL 2.17 and later)
    get("ncclCommInitAll", (void**)&api.CommInitAll);
    get("ncclAllReduce", (void**)&api.AllReduce);
    get("ncclAllGather", (void**)&api.AllGather);
    get("ncclCommDestroy", (void**)&api.CommDestroy);
    get("ncclCommAbort", (void**)&api.CommAbort);
    get("ncclCommGetAsyncError", (void**)&api.CommGetAsyncError);
    get("ncclGroupStart", (void**)&api.GroupStart);
    get("ncclGroupEnd", (void**)&api.GroupEnd);
    get("ncclGetErrorString", (void**)&api.GetErrorString);
    api.ok = ok;
  });
  return api;
}

size_t dtype_size(b200_dtype d) {
  switch (d) {
    case B200_PRED: case B200_S8: case B200_U8: return 1;
    case B200_S16: case B200_U16: case B200_F16: case B200_BF16: return 2;
    case B200_S32: case B200_U32: case B200_F32: return 4;
    case B200_S64: case B200_U64: case B200_F64: return 8;
    default: return 0;
  }
}
b200_dtype to_api(DT d) {
  switch (d) {
    case DT::PRED: return B200_PRED;
    case DT::I8: return B200_S8;
    case DT::I16: return B200_S16;
    case DT::I32: return B200_S32;
    case DT::I64: return B200_S64;
    case DT::U8: return B200_U8;
    case DT::U16: return B200_U16;
    case DT::U32: return B200_U32;
    case DT::U64: return B200_U64;
    case DT::F16: return B200_F16;
    case DT::F32: return B200_F32;
    case DT::F64: return B200_F64;
    case DT::BF16: return B200_BF16;
    default: return B200_INVALID;
  }
}

// ---- completion thread: fires on_ready callbacks (pjrt_event.cc:28-78) ----------
struct Completion {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::function<void()>> q;
  bool started = false;
  void post(std::function<void()> f) {
    std::lock_guard<std::mutex> l(mu);
    if (!started) {
      started = true;
      std::thread([this] {
        for (;;) {
          std::function<void()> f;
          {
            std::unique_lock<std::mutex> l(mu);
            cv.wait(l, [this] { return !q.empty(); });
            f = std::move(q.front());
            q.pop_front();
          }
          f();
        }
      }).detach();
    }
    q.push_back(std::move(f));
    cv.notify_one();
  }
};
Completion& completion() {
  static Completion* c = new Completion();   // never destroyed: the thread outlives static destructors
  return *c;
}

}  // namespace

// Error counter of the device as one execution saw it: the word before its first kernel and after its last, copied
// into pinned memory on the compute stream. The execution failed (a bounded device-side wait ran out) when the two
// differ once the copies have landed.
struct ExecStatus {
  volatile int* pair = nullptr;   // pinned: [0] before, [1] after
  std::function<void(volatile int*)> release;
  ~ExecStatus() { if (release && pair) release(pair); }
  bool failed() const { return pair && pair[1] != pair[0]; }
};

struct b200_event {
  cudaEvent_t ev = nullptr;       // null: ready at creation
  int device = 0;
  std::shared_ptr<ExecStatus> status;   // set on events of an execution and of reads of its results
  std::string error;              // non-empty: the event completed with an error
  b200_error_code code = B200_OK;
  ~b200_event() {
    if (ev) cudaEventDestroy(ev);
  }
};

struct PinnedBlock {
  void* ptr = nullptr;
  size_t size = 0;
  cudaEvent_t ev = nullptr;
  bool in_flight = false;
};

struct LoadedProgram {
  std::unique_ptr<CompiledProgram> prog;
  std::string text;                            // the module this plan was compiled from
  std::vector<const char*> output_kinds;       // PJRT_Executable_OutputMemoryKinds
  std::vector<size_t> output_kind_sizes;
  std::vector<CUmodule> modules;
  std::vector<CUfunction> functions;
  std::vector<void*> const_ptrs;
  std::vector<void*> arenas;
  void* const_block = nullptr;
  // Instantiated CUDA graphs of counted-loop bodies (two iterations each), per loop step and per set of slot
  // addresses the graph was captured with.
  struct LoopGraph { const void* step; std::vector<void*> ptrs; cudaGraphExec_t exec; int launches; };
  std::vector<LoopGraph> loop_graphs;
  // Graphs of data-dependent loops and cases (conditional nodes), per step and per set of addresses of the slots the
  // step and everything below it touches.
  std::vector<LoopGraph> cond_graphs;
  ~LoadedProgram() {
    for (auto& g : loop_graphs)
      if (g.exec) cudaGraphExecDestroy(g.exec);
    for (auto& g : cond_graphs)
      if (g.exec) cudaGraphExecDestroy(g.exec);
    for (auto* a : arenas)
      if (a) cudaFree(a);
    if (const_block) cudaFree(const_block);
    if (driver().ok)
      for (auto m : modules) driver().ModuleUnload(m);
  }
};

struct b200_client {
  int ordinal = 0, rank = 0, nprocs = 1;
  cudaStream_t compute = nullptr, h2d = nullptr, d2h = nullptr;
  cudaStream_t coll = nullptr;                      // collectives that overlap with compute (created with the communicator)
  cudaEvent_t coll_ready = nullptr, coll_done = nullptr;
  cudaMemPool_t pool = nullptr;
  ncclComm_t comm = nullptr;
  std::recursive_mutex mu;
  std::string kind, debug, version, memory_debug, memory_string;
  std::vector<std::string> topology_strings;
  std::atomic<int64_t> bytes_in_use{0}, peak_bytes{0}, num_allocs{0}, largest_alloc{0}, launches{0};
  // program text hash -> loaded plan. Entries are weak: the last executable handle releases the plan's arenas,
  // constants, modules and loop graphs (as PJRT_LoadedExecutable_Destroy does in the reference). A hit is confirmed
  // by comparing the text itself.
  std::map<std::string, std::weak_ptr<LoadedProgram>> cache;
  std::vector<PinnedBlock> pinned;
  unsigned char* pred_host = nullptr;   // pinned byte for while-loop predicates
  int* error_flag = nullptr;            // device word raised by kernels whose bounded waits expire
  unsigned long long* loop_guard = nullptr;   // device: start time of the data-dependent loop that is running
  double while_limit_s = 30.0;          // a device-resident data-dependent loop ends with an error after this long
  long long host_syncs = 0;             // stream synchronisations inside executions (predicates read back by the host)
  bool tensor_cores = true;
  bool profiling = false;
  // debugging switches of the contraction kernels and the loop executor, read from the environment once at creation
  struct Switches { bool no_vec_gather = false, no_seg_gather = false, no_tmem_a = false, no_half_ctas = false, narrow_tiles = false,
                    no_loop_graphs = false, no_tma_a = false, no_pdl = false, no_device_cf = false; } sw;
  int reported_errors = 0;              // value of the error word at the last b200_client_synchronize
  int armed_wait_polls = 0;             // test hook: the next execution starts with a wait that runs out
  int* status_block = nullptr;          // pinned pairs handed to executions
  std::vector<int> free_status;         // free pair indices
  static constexpr int kStatusPairs = 4096;
  struct ProfEntry { std::string kind; double ms = 0; long long count = 0; };
  std::map<std::string, ProfEntry> profile;
  int64_t total_mem = 0;

  void note_alloc(size_t n) {
    int64_t cur = bytes_in_use.fetch_add((int64_t)n) + (int64_t)n;
    int64_t pk = peak_bytes.load();
    while (cur > pk && !peak_bytes.compare_exchange_weak(pk, cur)) {}
    num_allocs++;
    int64_t lg = largest_alloc.load();
    while ((int64_t)n > lg && !largest_alloc.compare_exchange_weak(lg, (int64_t)n)) {}
  }
  void note_free(size_t n) { bytes_in_use.fetch_sub((int64_t)n); }
};

struct b200_buffer {
  b200_client* client = nullptr;
  std::shared_ptr<ExecStatus> status;          // the execution that produced this buffer
  void* ptr = nullptr;
  size_t bytes = 0;
  b200_dtype dtype = B200_INVALID;
  std::vector<int64_t> dims;
  cudaEvent_t ready = nullptr;                 // recorded on the producing stream
  cudaStream_t ready_on = nullptr;             // that stream: work issued to it later needs no wait
  struct Block { void* base; int refs; };      // one device allocation shared by several results of an execution
  Block* block = nullptr;                      // non-null: ptr lies inside block->base, freed with its last buffer
  std::vector<cudaEvent_t> reads;              // pending reads on other streams
  bool deleted = false;
};

struct b200_profiler {
  bool running = false;
};

struct b200_executable {
  b200_client* client = nullptr;
  std::shared_ptr<LoadedProgram> lp;
};

namespace {

b200_error* set_device(b200_client* c) {
  CUDA_TRY(cudaSetDevice(c->ordinal));
  return nullptr;
}

b200_error* device_alloc(b200_client* c, size_t bytes, cudaStream_t stream, void** out) {
  size_t n = std::max<size_t>(bytes, 16);
  cudaError_t e = cudaMallocAsync(out, n, stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return make_error(B200_RESOURCE_EXHAUSTED, "device allocation of " + std::to_string(n) + " bytes failed: " +
                                                   cudaGetErrorString(e));
  }
  c->note_alloc(n);
  return nullptr;
}

b200_event* new_event_on(b200_client* c, cudaStream_t stream, b200_error** err) {
  auto* e = new b200_event();
  e->device = c->ordinal;
  cudaError_t r = cudaEventCreateWithFlags(&e->ev, cudaEventDisableTiming);
  if (r == cudaSuccess) r = cudaEventRecord(e->ev, stream);
  if (r != cudaSuccess) {
    *err = make_error(B200_INTERNAL, std::string("event creation failed: ") + cudaGetErrorString(r));
    delete e;
    return nullptr;
  }
  return e;
}

// Pinned staging blocks are reused once the copy that read them has finished.
void* acquire_pinned(b200_client* c, size_t bytes, int* index) {
  for (size_t i = 0; i < c->pinned.size(); i++) {
    PinnedBlock& b = c->pinned[i];
    if (b.size < bytes) continue;
    if (b.in_flight) {
      if (cudaEventQuery(b.ev) != cudaSuccess) continue;
      b.in_flight = false;
    }
    *index = (int)i;
    return b.ptr;
  }
  PinnedBlock nb;
  size_t sz = 1 << 20;
  while (sz < bytes) sz <<= 1;
  if (cudaMallocHost(&nb.ptr, sz) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  nb.size = sz;
  cudaEventCreateWithFlags(&nb.ev, cudaEventDisableTiming);
  c->pinned.push_back(nb);
  *index = (int)c->pinned.size() - 1;
  return nb.ptr;
}

// Packs a strided host array into dense row-major order (mlx_buffer.cc:151-201 does the same row by row).
void pack_strided(const char* src, char* dst, const int64_t* dims, const int64_t* strides, size_t nd, size_t elem) {
  if (nd == 0) { memcpy(dst, src, elem); return; }
  std::vector<int64_t> idx(nd, 0);
  int64_t total = 1;
  for (size_t d = 0; d < nd; d++) total *= dims[d];
  bool inner_dense = strides[nd - 1] == (int64_t)elem;
  int64_t inner = dims[nd - 1];
  for (int64_t done = 0; done < total; done += inner) {
    const char* p = src;
    for (size_t d = 0; d + 1 < nd; d++) p += idx[d] * strides[d];
    if (inner_dense) memcpy(dst, p, (size_t)inner * elem);
    else
      for (int64_t i = 0; i < inner; i++) memcpy(dst + i * elem, p + i * strides[nd - 1], elem);
    dst += inner * elem;
    for (int d = (int)nd - 2; d >= 0; d--) {
      if (++idx[d] < dims[d]) break;
      idx[d] = 0;
    }
  }
}

ncclDataType_t nccl_type(DT d, bool* ok) {
  *ok = true;
  switch (d) {
    case DT::F32: return ncclFloat32;
    case DT::F64: return ncclFloat64;
    case DT::F16: return ncclFloat16;
    case DT::BF16: return ncclBfloat16;
    case DT::I32: return ncclInt32;
    case DT::U32: return ncclUint32;
    case DT::I64: return ncclInt64;
    case DT::U64: return ncclUint64;
    case DT::I8: return ncclInt8;
    case DT::U8: return ncclUint8;
    default: *ok = false; return ncclFloat32;
  }
}

// ---- NVRTC compilation of the generated kernels ------------------------------------
b200_error* build_kernels(LoadedProgram& lp) {
  CompiledProgram& p = *lp.prog;
  if (p.kernels.empty()) return nullptr;
  NvrtcApi& rt = nvrtc();
  if (!rt.ok) return make_error(B200_FAILED_PRECONDITION, "NVRTC unavailable: " + rt.error);
  DriverApi& drv = driver();
  if (!drv.ok) return make_error(B200_FAILED_PRECONDITION, drv.error);
  size_t n = p.kernels.size();
  unsigned hw = std::max(1u, std::thread::hardware_concurrency());
  size_t chunks = std::min<size_t>(std::min<size_t>(hw, 16), (n + 7) / 8);
  chunks = std::max<size_t>(chunks, 1);
  std::vector<std::string> cubins(chunks), errors(chunks);
  std::vector<std::thread> threads;
  for (size_t c = 0; c < chunks; c++) {
    threads.emplace_back([&, c] {
      std::string src = codegen_prelude();
      for (size_t k = c; k < n; k += chunks) src += p.kernels[k].body + "\n";
      nvrtcProgram prog;
      if (rt.CreateProgram(&prog, src.c_str(), "b200_fused.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS) {
        errors[c] = "nvrtcCreateProgram failed";
        return;
      }
      const char* opts[] = {"--gpu-architecture=sm_100a", "-std=c++17", "-lineinfo", "-w"};
      nvrtcResult r = rt.CompileProgram(prog, 4, opts);
      if (r != NVRTC_SUCCESS) {
        size_t ls = 0;
        rt.GetProgramLogSize(prog, &ls);
        std::string log(ls, '\0');
        if (ls) rt.GetProgramLog(prog, &log[0]);
        errors[c] = std::string("NVRTC: ") + rt.GetErrorString(r) + "\n" + log.substr(0, 4000);
        rt.DestroyProgram(&prog);
        return;
      }
      size_t cs = 0;
      rt.GetCUBINSize(prog, &cs);
      cubins[c].resize(cs);
      rt.GetCUBIN(prog, &cubins[c][0]);
      rt.DestroyProgram(&prog);
    });
  }
  for (auto& t : threads) t.join();
  for (auto& e : errors)
    if (!e.empty()) return make_error(B200_INTERNAL, "kernel generation failed: " + e);
  lp.functions.assign(n, nullptr);
  for (size_t c = 0; c < chunks; c++) {
    CUmodule mod;
    CUresult r = drv.ModuleLoadData(&mod, cubins[c].data());
    if (r != CUDA_SUCCESS) {
      const char* s = nullptr;
      drv.GetErrorString(r, &s);
      return make_error(B200_INTERNAL, std::string("cuModuleLoadData failed: ") + (s ? s : "?"));
    }
    lp.modules.push_back(mod);
    for (size_t k = c; k < n; k += chunks) {
      r = drv.ModuleGetFunction(&lp.functions[k], mod, p.kernels[k].name.c_str());
      if (r != CUDA_SUCCESS) return make_error(B200_INTERNAL, "generated kernel " + p.kernels[k].name + " not found in module");
    }
  }
  return nullptr;
}

struct ExecCtx {
  b200_client* c;
  LoadedProgram* lp;
  std::vector<void*> ptrs;
  int launches = 0;
  bool plain_launch = false;            // while the bodies of conditional graph nodes are recorded: no programmatic launches
  bool coll_pending = false;            // work on the collective stream that the compute stream has not waited for yet
  cudaStream_t coll_stream = nullptr;   // set while the members of an all-reduce group are issued
  struct Timed { std::string kind, key; cudaEvent_t a, b; };
  std::vector<Timed> timed;
};

b200_error* run_plan(ExecCtx& x, const Plan& plan);

// A plan can be recorded into a CUDA graph when it only launches kernels and device copies: no host round trip
// (data-dependent loops, case), no collective.
bool graph_safe(const Plan& plan) {
  for (const Step& s : plan.steps) {
    switch (s.kind) {
      case Step::KERNEL: case Step::IGEMM: case Step::MEMCPY: case Step::GEMM16: case Step::REPACK16: case Step::TRANSPOSE: break;
      case Step::WHILE:
        if (s.trip_count < 0 || !graph_safe(*s.sub[1])) return false;
        break;
      default: return false;
    }
  }
  return true;
}

// Addresses of every slot a step and the plans below it refer to, in a fixed order.
void touched_addresses(const ExecCtx& x, const Step& s, std::vector<void*>& out, bool top = true) {
  for (int a : s.args) out.push_back(x.ptrs[a]);
  for (int a : s.state) out.push_back(x.ptrs[a]);
  if (!top) for (int a : s.init) out.push_back(x.ptrs[a]);      // the outermost loop's initial values are copied in front of the graph
  for (int a : s.next) out.push_back(x.ptrs[a]);
  if (s.pred >= 0) out.push_back(x.ptrs[s.pred]);
  for (auto& p : s.sub)
    if (p) for (const Step& t : p->steps) touched_addresses(x, t, out, false);
}

b200_error* run_step(ExecCtx& x, const Step& s) {
  b200_client* c = x.c;
  cudaStream_t st = c->compute;
  switch (s.kind) {
    case Step::KERNEL: {
      void* vals[512];
      void* argv[512];
      size_t n = s.args.size();
      if (n > 512) return make_error(B200_INTERNAL, "kernel with more than 512 parameters");
      for (size_t k = 0; k < n; k++) {
        vals[k] = x.ptrs[s.args[k]];
        argv[k] = &vals[k];
      }
      CUresult r;
      if (driver().LaunchKernelEx && !c->sw.no_pdl && !x.plain_launch) {
        // programmatic stream serialization: the kernel is scheduled while the one in front of it drains, and waits for
        // it (first statement of every generated kernel) before it reads or writes anything
        CUlaunchConfig cfg = {};
        cfg.gridDimX = s.grid[0]; cfg.gridDimY = s.grid[1]; cfg.gridDimZ = s.grid[2];
        cfg.blockDimX = s.block[0]; cfg.blockDimY = s.block[1]; cfg.blockDimZ = s.block[2];
        cfg.sharedMemBytes = 0;
        cfg.hStream = (CUstream)st;
        CUlaunchAttribute attr[1];
        attr[0].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr[0].value.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        r = driver().LaunchKernelEx(&cfg, x.lp->functions[s.kernel], argv, nullptr);
      } else {
        r = driver().LaunchKernel(x.lp->functions[s.kernel], s.grid[0], s.grid[1], s.grid[2], s.block[0], s.block[1], s.block[2], 0,
                                  (CUstream)st, argv, nullptr);
      }
      if (r != CUDA_SUCCESS) {
        const char* msg = nullptr;
        driver().GetErrorString(r, &msg);
        return make_error(B200_INTERNAL, "launch of " + s.label + " failed: " + (msg ? msg : "?"));
      }
      x.launches++;
      return nullptr;
    }
    case Step::IGEMM: {
      IGemmLaunch p;
      p.M = s.ig.M; p.N = s.ig.N; p.K = s.ig.K; p.groups = s.ig.groups; p.split_k = s.ig.split_k;
      p.Hd = s.ig.Hd; p.Wd = s.ig.Wd; p.ldh = s.ig.ldh; p.ldw = s.ig.ldw;
      p.a_sh = s.ig.a_sh; p.a_sw = s.ig.a_sw;
      p.a_mcontig = s.ig.a_contig; p.b_kcontig = s.ig.b_contig; p.mask = s.ig.needs_mask;
      // tiny products stay on the fp32 FMA kernel; everything else goes to the tensor cores (3xTF32)
      p.vec = s.ig.vec && !c->sw.no_vec_gather;
      p.c_vec = s.ig.c_vec;
      p.seg = p.vec && s.ig.seg && !c->sw.no_seg_gather;
      p.tmem_a = c->sw.no_tmem_a ? 0 : 1;
      p.half_ctas = c->sw.no_half_ctas ? 0 : 1;
      p.wide_n = c->sw.narrow_tiles ? 0 : 1;
      p.tensor_cores = c->tensor_cores && (long long)s.ig.M * s.ig.N * s.ig.K * s.ig.groups >= (1LL << 18) && s.ig.K >= 16;
      const void* tables[9];
      for (int k = 0; k < 9; k++) tables[k] = x.ptrs[s.args[3 + k]];
      void* partial = s.ig.split_k > 1 ? x.ptrs[s.args[12]] : nullptr;
      p.kt_stride = s.ig.kt_stride;
      p.a_tma = s.ig.a_tma && p.seg && p.tmem_a && !c->sw.no_tma_a;
      p.tma_c = s.ig.tma_c; p.tma_w = s.ig.tma_w; p.tma_h = s.ig.tma_h; p.tma_n = s.ig.tma_n;
      p.tma_ow = s.ig.tma_ow; p.tma_oh = s.ig.tma_oh; p.tma_box_h = s.ig.tma_box_h; p.tma_box_n = s.ig.tma_box_n;
      p.tma_kw = s.ig.tma_kw; p.tma_pad_h = s.ig.tma_pad_h; p.tma_pad_w = s.ig.tma_pad_w;
      p.tma_rdil_h = s.ig.tma_rdil_h; p.tma_rdil_w = s.ig.tma_rdil_w;
      const int* kt_table = s.ig.kt_stride > 0 ? (const int*)x.ptrs[s.args.back()] : nullptr;
      cudaError_t e = launch_igemm_f32(p, x.ptrs[s.args[0]], x.ptrs[s.args[1]], x.ptrs[s.args[2]], tables, partial,
                                       kt_table, c->error_flag, st, &x.launches);
      if (e != cudaSuccess) return make_error(B200_INTERNAL, "launch of " + s.label + " failed: " + cudaGetErrorString(e));
      return nullptr;
    }
    case Step::GEMM16: {
      size_t next = 3;
      float* scratch = s.iparams[0] ? (float*)x.ptrs[s.args[next++]] : nullptr;
      int* counters = s.iparams[1] ? (int*)x.ptrs[s.args[next++]] : nullptr;
      const char* why = nullptr;
      cudaError_t e = launch_gemm16(s.g16, x.ptrs[s.args[0]], x.ptrs[s.args[1]], x.ptrs[s.args[2]], scratch, counters,
                                    c->error_flag, st, &x.launches, &why);
      if (e != cudaSuccess)
        return make_error(B200_INTERNAL, "launch of " + s.label + " failed: " + (why ? why : cudaGetErrorString(e)));
      return nullptr;
    }
    case Step::TRANSPOSE: {
      char* dst = (char*)x.ptrs[s.args[0]] + s.iparams[6] * s.iparams[0];
      cudaError_t e = launch_transpose2d(dst, x.ptrs[s.args[1]], (int)s.iparams[0], s.iparams[1], s.iparams[2], s.iparams[3],
                                         s.iparams[4], s.iparams[5], st, &x.launches);
      if (e != cudaSuccess) return make_error(B200_INTERNAL, "launch of " + s.label + " failed: " + cudaGetErrorString(e));
      return nullptr;
    }
    case Step::REPACK16: {
      cudaError_t e = launch_repack_rows16(x.ptrs[s.args[0]], x.ptrs[s.args[1]], s.iparams[0], s.iparams[1], s.iparams[2],
                                           s.iparams[3], st, &x.launches);
      if (e != cudaSuccess) return make_error(B200_INTERNAL, "launch of " + s.label + " failed: " + cudaGetErrorString(e));
      return nullptr;
    }
    case Step::MEMCPY: {
      if (s.bytes && x.ptrs[s.args[0]] != x.ptrs[s.args[1]])
        CUDA_TRY(cudaMemcpyAsync(x.ptrs[s.args[0]], x.ptrs[s.args[1]], s.bytes, cudaMemcpyDeviceToDevice, st));
      return nullptr;
    }
    case Step::ALL_REDUCE: {
      void* in = x.ptrs[s.args[0]];
      void* out = x.ptrs[s.args[1]];
      if (c->nprocs == 1) {
        // one partition: identity (src/pjrt_plugin/ops/collectives.cc:41-47)
        if (in != out && s.bytes) CUDA_TRY(cudaMemcpyAsync(out, in, s.bytes, cudaMemcpyDeviceToDevice, st));
        return nullptr;
      }
      bool ok;
      ncclDataType_t t = nccl_type(s.dtype, &ok);
      if (!ok) return make_error(B200_UNIMPLEMENTED, "all_reduce of this element type");
      ncclResult_t r = nccl().AllReduce(in, out, s.bytes / dt_size(s.dtype), t, ncclSum, c->comm, x.coll_stream ? x.coll_stream : st);
      if (r != ncclSuccess) return make_error(B200_INTERNAL, std::string("ncclAllReduce failed: ") + nccl().GetErrorString(r));
      x.launches++;
      return nullptr;
    }
    case Step::ALL_GATHER: {
      void *in = x.ptrs[s.args[0]], *out = x.ptrs[s.args[1]];
      if (c->nprocs == 1) {
        if (in != out && s.bytes) CUDA_TRY(cudaMemcpyAsync(out, in, s.bytes, cudaMemcpyDeviceToDevice, st));
        return nullptr;
      }
      // bytes move as they are: gathered as unsigned bytes whatever the element type
      const long long rows = s.iparams[0], row_bytes = s.iparams[1];
      void* dst = rows > 1 ? x.ptrs[s.args[2]] : out;
      ncclResult_t r = nccl().AllGather(in, dst, s.bytes, ncclUint8, c->comm, st);
      if (r != ncclSuccess) return make_error(B200_INTERNAL, std::string("ncclAllGather failed: ") + nccl().GetErrorString(r));
      x.launches++;
      if (rows > 1) {
        // staging holds [partition][row][row_bytes]; the result wants [row][partition][row_bytes]
        for (int p2 = 0; p2 < c->nprocs; p2++)
          CUDA_TRY(cudaMemcpy2DAsync((char*)out + (size_t)p2 * row_bytes, (size_t)c->nprocs * row_bytes,
                                     (char*)dst + (size_t)p2 * s.bytes, (size_t)row_bytes, (size_t)row_bytes, (size_t)rows,
                                     cudaMemcpyDeviceToDevice, st));
      }
      return nullptr;
    }
    case Step::WHILE: {
      size_t n = s.state.size();
      for (size_t k = 0; k < n; k++) {
        void *d = x.ptrs[s.state[k]], *src = x.ptrs[s.init[k]];
        size_t b = x.lp->prog->slots[s.state[k]].type.bytes();
        if (d != src && b) CUDA_TRY(cudaMemcpyAsync(d, src, b, cudaMemcpyDeviceToDevice, st));
      }
      // carried values marked for exchange trade pointers with their next value after every iteration; when the
      // loop ends the pointers go back and a value left in the other buffer is copied home once
      std::vector<void*> home_state(n), home_next(n);
      for (size_t k = 0; k < n; k++) {
        home_state[k] = x.ptrs[s.state[k]];
        home_next[k] = x.ptrs[s.next[k]];
      }
      auto iterate = [&]() -> b200_error* {
        if (auto* e = run_plan(x, *s.sub[1])) return e;
        for (size_t k = 0; k < n; k++) {
          if (k < s.swap.size() && s.swap[k]) {
            std::swap(x.ptrs[s.state[k]], x.ptrs[s.next[k]]);
            continue;
          }
          void *d = x.ptrs[s.state[k]], *src = x.ptrs[s.next[k]];
          size_t b = x.lp->prog->slots[s.state[k]].type.bytes();
          if (d != src && b) CUDA_TRY(cudaMemcpyAsync(d, src, b, cudaMemcpyDeviceToDevice, st));
        }
        return nullptr;
      };
      auto finish = [&]() -> b200_error* {
        for (size_t k = 0; k < n; k++) {
          if (!(k < s.swap.size() && s.swap[k])) continue;
          void* cur = x.ptrs[s.state[k]];
          x.ptrs[s.state[k]] = home_state[k];
          x.ptrs[s.next[k]] = home_next[k];
          size_t b = x.lp->prog->slots[s.state[k]].type.bytes();
          if (cur != home_state[k] && b) CUDA_TRY(cudaMemcpyAsync(home_state[k], cur, b, cudaMemcpyDeviceToDevice, st));
        }
        return nullptr;
      };
      if (s.trip_count >= 0) {
        // counted loop: trip count known at compile time, no host round trip
        // (the reference's counted path, src/pjrt_plugin/ops/control_flow.cc:476-503)
        long long done = 0;
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        CUDA_TRY(cudaStreamIsCapturing(st, &capturing));
        if (s.trip_count >= 4 && !c->profiling && capturing == cudaStreamCaptureStatusNone && graph_safe(*s.sub[1]) &&
            !c->sw.no_loop_graphs) {
          // Two iterations (after which exchanged pointers are back where they started) are recorded once as a
          // CUDA graph and replayed: the host issues one launch per pair instead of one per kernel, and the
          // dependent kernels of a latency-bound body follow each other without a host round trip.
          const long long pairs = s.trip_count / 2;
          long long replayed = 0;
          LoadedProgram::LoopGraph* hit = nullptr;
          for (auto& g : x.lp->loop_graphs)
            if (g.step == &s && g.ptrs == x.ptrs) { hit = &g; break; }
          if (!hit) {
            if (x.lp->loop_graphs.size() >= 16) {
              // bounded cache: let the device finish with the oldest graph before it goes
              CUDA_TRY(cudaStreamSynchronize(st));
              cudaGraphExecDestroy(x.lp->loop_graphs.front().exec);
              x.lp->loop_graphs.erase(x.lp->loop_graphs.begin());
            }
            const std::vector<void*> at_start = x.ptrs;
            // the first pair runs directly, so that every kernel of the body has been loaded and configured
            // before anything is recorded
            if (auto* e = iterate()) return e;
            if (auto* e = iterate()) return e;
            replayed = 1;
            const int before = x.launches;
            CUDA_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed));
            b200_error* err = iterate();
            if (!err) err = iterate();
            cudaGraph_t graph = nullptr;
            cudaError_t ce = cudaStreamEndCapture(st, &graph);
            if (err) {
              if (graph) cudaGraphDestroy(graph);
              return err;
            }
            CUDA_TRY(ce);
            cudaGraphExec_t exec = nullptr;
            ce = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            CUDA_TRY(ce);
            if (x.ptrs != at_start) {
              cudaGraphExecDestroy(exec);
              return make_error(B200_INTERNAL, "loop state pointers did not return after two iterations");
            }
            x.lp->loop_graphs.push_back({&s, at_start, exec, x.launches - before});
            x.launches = before;
            hit = &x.lp->loop_graphs.back();
          }
          for (long long i = replayed; i < pairs; i++) CUDA_TRY(cudaGraphLaunch(hit->exec, st));
          x.launches += (int)(hit->launches * (pairs - replayed));
          done = 2 * pairs;
        }
        for (long long i = done; i < s.trip_count; i++)
          if (auto* e = iterate()) return e;
        return finish();
      }
      // Data-dependent loop. On the device when condition and body only launch kernels and device copies: a CUDA graph
      // of [condition, handle] -> while node { body, copies of the carried values, condition, handle }, where
      // `handle` is a one-thread kernel that sets the node's handle from the predicate (the reference pays a host
      // read-back per iteration, src/pjrt_plugin/ops/control_flow.cc:505-536). Inside the graph carried values are
      // copied, not exchanged (the addresses are part of the recording). The first execution of a loop with a given
      // set of addresses runs through the host, which also loads every kernel; the graph is recorded after it.
      cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
      CUDA_TRY(cudaStreamIsCapturing(st, &capturing));
      const bool on_device = !c->sw.no_device_cf && !c->profiling && capturing == cudaStreamCaptureStatusNone &&
                             graph_safe(*s.sub[0]) && graph_safe(*s.sub[1]);
      std::vector<void*> touched;
      if (on_device) {
        touched_addresses(x, s, touched);
        for (auto& g : x.lp->cond_graphs)
          if (g.step == &s && g.ptrs == touched) {
            CUDA_TRY(cudaGraphLaunch(g.exec, st));
            x.launches += g.launches;
            return nullptr;
          }
      }
      const std::vector<void*> at_start = x.ptrs;
      long long trips = 0;
      for (long long it = 0;; it++) {
        if (auto* e = run_plan(x, *s.sub[0])) return e;
        CUDA_TRY(cudaMemcpyAsync(c->pred_host, x.ptrs[s.pred], 1, cudaMemcpyDeviceToHost, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        c->host_syncs++;
        if (!*c->pred_host) break;
        if (auto* e = iterate()) return e;
        trips++;
      }
      if (auto* e = finish()) return e;
      if (on_device && trips > 0 && x.ptrs == at_start) {
        if (x.lp->cond_graphs.size() >= 16) {
          CUDA_TRY(cudaStreamSynchronize(st));
          cudaGraphExecDestroy(x.lp->cond_graphs.front().exec);
          x.lp->cond_graphs.erase(x.lp->cond_graphs.begin());
        }
        // the loop has just run with these addresses: recording changes nothing on the device
        const int before = x.launches;
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        b200_error* err = nullptr;
        auto fail = [&](cudaError_t ce, const char* what) {
          if (!err) err = make_error(B200_INTERNAL, std::string("recording a device-resident loop: ") + what + ": " + cudaGetErrorString(ce));
        };
        x.plain_launch = true;
        set_programmatic_launch(false);
        set_igemm_programmatic_launch(false);
        cudaError_t ce = cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed);
        if (ce != cudaSuccess) fail(ce, "begin capture");
        else {
          cudaStreamCaptureStatus status;
          const cudaGraphNode_t* deps = nullptr;
          size_t ndeps = 0;
          cudaGraphConditionalHandle handle = 0;
          cudaGraph_t body = nullptr;
          ce = cudaStreamGetCaptureInfo(st, &status, nullptr, &graph, &deps, &ndeps);
          if (ce != cudaSuccess) fail(ce, "capture info");
          if (!err && (ce = cudaGraphConditionalHandleCreate(&handle, graph, 0, cudaGraphCondAssignDefault)) != cudaSuccess) fail(ce, "handle");
          if (!err) err = run_plan(x, *s.sub[0]);
          if (!err && (ce = launch_while_handle(handle, x.ptrs[s.pred], c->loop_guard, c->while_limit_s, true, c->error_flag, st)) != cudaSuccess)
            fail(ce, "handle kernel");
          if (!err && (ce = cudaStreamGetCaptureInfo(st, &status, nullptr, nullptr, &deps, &ndeps)) != cudaSuccess) fail(ce, "capture info");
          if (!err) {
            cudaGraphNodeParams np = {};
            np.type = cudaGraphNodeTypeConditional;
            np.conditional.handle = handle;
            np.conditional.type = cudaGraphCondTypeWhile;
            np.conditional.size = 1;
            cudaGraphNode_t node = nullptr;
            if ((ce = cudaGraphAddNode(&node, graph, deps, ndeps, &np)) != cudaSuccess) fail(ce, "while node");
            else {
              body = np.conditional.phGraph_out[0];
              if ((ce = cudaStreamUpdateCaptureDependencies(st, &node, 1, cudaStreamSetCaptureDependencies)) != cudaSuccess) fail(ce, "dependencies");
            }
          }
          cudaGraph_t ended = nullptr;
          ce = cudaStreamEndCapture(st, &ended);
          if (ce != cudaSuccess) fail(ce, "end capture");
          graph = ended;                              // null when the capture was invalidated: nothing to destroy then
          if (!err && body) {
            if ((ce = cudaStreamBeginCaptureToGraph(st, body, nullptr, nullptr, 0, cudaStreamCaptureModeRelaxed)) != cudaSuccess) fail(ce, "begin body");
            else {
              err = run_plan(x, *s.sub[1]);
              for (size_t k = 0; k < n && !err; k++) {
                void *d = x.ptrs[s.state[k]], *src = x.ptrs[s.next[k]];
                size_t b = x.lp->prog->slots[s.state[k]].type.bytes();
                if (d != src && b && (ce = cudaMemcpyAsync(d, src, b, cudaMemcpyDeviceToDevice, st)) != cudaSuccess) fail(ce, "state copy");
              }
              if (!err) err = run_plan(x, *s.sub[0]);
              if (!err && (ce = launch_while_handle(handle, x.ptrs[s.pred], c->loop_guard, c->while_limit_s, false, c->error_flag, st)) != cudaSuccess)
                fail(ce, "handle kernel");
              ce = cudaStreamEndCapture(st, nullptr);
              if (ce != cudaSuccess) fail(ce, "end body");
            }
          }
          if (!err && (ce = cudaGraphInstantiate(&exec, graph, 0)) != cudaSuccess) fail(ce, "instantiate");
        }
        x.plain_launch = false;
        set_programmatic_launch(!c->sw.no_pdl);
        set_igemm_programmatic_launch(!c->sw.no_pdl && !getenv("B200_NO_IGEMM_PDL"));
        if (graph) cudaGraphDestroy(graph);
        const int recorded = x.launches - before;
        x.launches = before;
        if (err) {
          // a loop that cannot be recorded keeps the host path (the result of this execution is already complete)
          logf(1, "%s", err->message.c_str());
          b200_error_destroy(err);
          cudaGetLastError();
        } else {
          x.lp->cond_graphs.push_back({&s, touched, exec, recorded});
        }
      }
      return nullptr;
    }
    case Step::SCATTER: {
      void *operand = x.ptrs[s.args[0]], *out = x.ptrs[s.args[3]];
      if (operand != out && s.bytes) CUDA_TRY(cudaMemcpyAsync(out, operand, s.bytes, cudaMemcpyDeviceToDevice, st));
      const int ek = s.dtype == DT::F32 ? 0 : s.dtype == DT::BF16 ? 1 : 2;
      if (s.iparams.size() > 5 && s.iparams[5] == 1) {
        // general form: the key kernel in front of this step has filled the scratch with (destination, update) pairs
        cudaError_t e = launch_scatter_elems(ek, (int)s.iparams[4], s.iparams[0], (int)s.iparams[2], out, x.ptrs[s.args[2]],
                                             (int*)x.ptrs[s.args[4]], st, &x.launches);
        if (e != cudaSuccess) return make_error(B200_INTERNAL, "launch of " + s.label + " failed: " + cudaGetErrorString(e));
        return nullptr;
      }
      cudaError_t e = launch_scatter_rows(ek, (int)s.iparams[3], (int)s.iparams[4], s.iparams[0], s.iparams[1], (int)s.iparams[2], out,
                                          x.ptrs[s.args[1]], x.ptrs[s.args[2]], (int*)x.ptrs[s.args[4]], st, &x.launches);
      if (e != cudaSuccess) return make_error(B200_INTERNAL, "launch of " + s.label + " failed: " + cudaGetErrorString(e));
      return nullptr;
    }
    case Step::CASE: {
      const int n = (int)s.sub.size();
      // On the device when every branch only launches generated kernels and device copies: a switch node whose handle
      // a one-thread kernel sets from the index (out of range selects the last branch, as on the host path;
      // src/pjrt_plugin/ops/control_flow.cc:600-699). Recorded after the first execution through the host.
      cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
      CUDA_TRY(cudaStreamIsCapturing(st, &capturing));
      bool on_device = !c->sw.no_device_cf && !c->profiling && capturing == cudaStreamCaptureStatusNone && n >= 1;
      for (int b = 0; b < n && on_device; b++)
        for (const Step& bs : s.sub[b]->steps) on_device = on_device && (bs.kind == Step::KERNEL || bs.kind == Step::MEMCPY);
      std::vector<void*> touched;
      if (on_device) {
        touched_addresses(x, s, touched);
        for (auto& g : x.lp->cond_graphs)
          if (g.step == &s && g.ptrs == touched) {
            CUDA_TRY(cudaGraphLaunch(g.exec, st));
            x.launches += g.launches;
            return nullptr;
          }
      }
      int32_t index = 0;
      CUDA_TRY(cudaMemcpyAsync(c->pred_host, x.ptrs[s.pred], 4, cudaMemcpyDeviceToHost, st));
      CUDA_TRY(cudaStreamSynchronize(st));
      c->host_syncs++;
      memcpy(&index, c->pred_host, 4);
      if (index < 0 || index >= n) index = n - 1;
      if (auto* e = run_plan(x, *s.sub[index])) return e;
      if (on_device) {
        if (x.lp->cond_graphs.size() >= 16) {
          CUDA_TRY(cudaStreamSynchronize(st));
          cudaGraphExecDestroy(x.lp->cond_graphs.front().exec);
          x.lp->cond_graphs.erase(x.lp->cond_graphs.begin());
        }
        const int before = x.launches;
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        b200_error* err = nullptr;
        auto fail = [&](cudaError_t ce, const char* what) {
          if (!err) err = make_error(B200_INTERNAL, std::string("recording a device-resident case: ") + what + ": " + cudaGetErrorString(ce));
        };
        x.plain_launch = true;
        std::vector<cudaGraph_t> bodies;
        cudaError_t ce = cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed);
        if (ce != cudaSuccess) fail(ce, "begin capture");
        else {
          cudaStreamCaptureStatus status;
          const cudaGraphNode_t* deps = nullptr;
          size_t ndeps = 0;
          cudaGraphConditionalHandle handle = 0;
          ce = cudaStreamGetCaptureInfo(st, &status, nullptr, &graph, &deps, &ndeps);
          if (ce != cudaSuccess) fail(ce, "capture info");
          if (!err && (ce = cudaGraphConditionalHandleCreate(&handle, graph, 0, cudaGraphCondAssignDefault)) != cudaSuccess) fail(ce, "handle");
          if (!err && (ce = launch_switch_handle(handle, x.ptrs[s.pred], n, st)) != cudaSuccess) fail(ce, "handle kernel");
          if (!err && (ce = cudaStreamGetCaptureInfo(st, &status, nullptr, nullptr, &deps, &ndeps)) != cudaSuccess) fail(ce, "capture info");
          if (!err) {
            cudaGraphNodeParams np = {};
            np.type = cudaGraphNodeTypeConditional;
            np.conditional.handle = handle;
            np.conditional.type = cudaGraphCondTypeSwitch;
            np.conditional.size = (unsigned)n;
            cudaGraphNode_t node = nullptr;
            if ((ce = cudaGraphAddNode(&node, graph, deps, ndeps, &np)) != cudaSuccess) fail(ce, "switch node");
            else {
              for (int b = 0; b < n; b++) bodies.push_back(np.conditional.phGraph_out[b]);
              if ((ce = cudaStreamUpdateCaptureDependencies(st, &node, 1, cudaStreamSetCaptureDependencies)) != cudaSuccess) fail(ce, "dependencies");
            }
          }
          cudaGraph_t ended = nullptr;
          ce = cudaStreamEndCapture(st, &ended);
          if (ce != cudaSuccess) fail(ce, "end capture");
          graph = ended;
          for (int b = 0; b < n && !err && (int)bodies.size() == n; b++) {
            if ((ce = cudaStreamBeginCaptureToGraph(st, bodies[b], nullptr, nullptr, 0, cudaStreamCaptureModeRelaxed)) != cudaSuccess) { fail(ce, "begin branch"); break; }
            err = run_plan(x, *s.sub[b]);
            ce = cudaStreamEndCapture(st, nullptr);
            if (ce != cudaSuccess) fail(ce, "end branch");
          }
          if (!err && (ce = cudaGraphInstantiate(&exec, graph, 0)) != cudaSuccess) fail(ce, "instantiate");
        }
        x.plain_launch = false;
        if (graph) cudaGraphDestroy(graph);
        const int recorded = n > 0 ? (x.launches - before) / n : 0;
        x.launches = before;
        if (err) {
          logf(1, "%s", err->message.c_str());
          b200_error_destroy(err);
          cudaGetLastError();
        } else {
          x.lp->cond_graphs.push_back({&s, touched, exec, recorded});
        }
      }
      return nullptr;
    }
    default:
      return make_error(B200_UNIMPLEMENTED, "plan step kind not implemented: " + s.label);
  }
}

b200_error* run_plan(ExecCtx& x, const Plan& plan) {
  for (size_t si = 0; si < plan.steps.size(); ++si) {
    const Step& s = plan.steps[si];
    if (s.kind == Step::JOIN) {
      // the compute stream waits for everything issued on the collective stream so far
      if (x.c->nprocs > 1 && x.coll_pending) {
        CUDA_TRY(cudaStreamWaitEvent(x.c->compute, x.c->coll_done, 0));
        x.coll_pending = false;
      }
      continue;
    }
    if (s.kind == Step::ALL_REDUCE && x.c->nprocs > 1) {
      // consecutive all-reduces (the gradient leaves of a data-parallel step) go out as one NCCL group: one
      // fused launch instead of one per leaf
      size_t sj = si;
      size_t bytes = 0;
      while (sj < plan.steps.size() && plan.steps[sj].kind == Step::ALL_REDUCE) bytes += plan.steps[sj++].bytes;
      ExecCtx::Timed t;
      if (x.c->profiling) {
        t.kind = "all_reduce";
        t.key = "all_reduce group of " + std::to_string(sj - si) + ", " + std::to_string(bytes) + " bytes";
        cudaEventCreate(&t.a);
        cudaEventCreate(&t.b);
        cudaEventRecord(t.a, x.c->compute);
      }
      // the compiler lays the run's inputs and outputs out back to back (256-byte granules): when it did, the run
      // is one all-reduce over one flat buffer; the padding between leaves is summed along and never read
      // an overlapped run goes to the collective stream behind everything the compute stream has been given so far
      cudaStream_t cst = x.c->compute;
      const bool overlapped = s.overlapped && x.c->coll && !x.c->profiling;
      if (overlapped) {
        cst = x.c->coll;
        CUDA_TRY(cudaEventRecord(x.c->coll_ready, x.c->compute));
        CUDA_TRY(cudaStreamWaitEvent(cst, x.c->coll_ready, 0));
      }
      auto after_issue = [&]() -> b200_error* {
        if (overlapped) {
          CUDA_TRY(cudaEventRecord(x.c->coll_done, cst));
          x.coll_pending = true;
        }
        return nullptr;
      };
      {
        bool flat = sj - si >= 2;
        size_t total = 0;
        const Step& f = plan.steps[si];
        char *in0 = (char*)x.ptrs[f.args[0]], *out0 = (char*)x.ptrs[f.args[1]];
        for (size_t k = si; k < sj && flat; ++k) {
          const Step& q = plan.steps[k];
          flat = q.dtype == f.dtype && (char*)x.ptrs[q.args[0]] == in0 + total && (char*)x.ptrs[q.args[1]] == out0 + total;
          // leaves sit in 256-byte granules; the last one counts with its own size, so that the reduction never
          // reaches past the end of the last allocation
          total += k + 1 < sj ? (q.bytes + 255) & ~(size_t)255 : q.bytes;
        }
        bool ok = false;
        ncclDataType_t nt = nccl_type(f.dtype, &ok);
        if (flat && ok) {
          ncclResult_t r = nccl().AllReduce(in0, out0, total / dt_size(f.dtype), nt, ncclSum, x.c->comm, cst);
          if (r != ncclSuccess) return make_error(B200_INTERNAL, std::string("ncclAllReduce failed: ") + nccl().GetErrorString(r));
          if (auto* e = after_issue()) return e;
          x.launches += 1;
          if (x.c->profiling) {
            cudaEventRecord(t.b, x.c->compute);
            x.timed.push_back(t);
          }
          si = sj - 1;
          continue;
        }
      }
      const int before = x.launches;
      nccl().GroupStart();
      b200_error* err = nullptr;
      x.coll_stream = cst;
      for (size_t k = si; k < sj && !err; ++k) err = run_step(x, plan.steps[k]);
      x.coll_stream = nullptr;
      ncclResult_t r = nccl().GroupEnd();
      if (err) return err;
      if (r != ncclSuccess) return make_error(B200_INTERNAL, std::string("ncclGroupEnd failed: ") + nccl().GetErrorString(r));
      if (auto* e = after_issue()) return e;
      x.launches = before + 1;
      if (x.c->profiling) {
        cudaEventRecord(t.b, x.c->compute);
        x.timed.push_back(t);
      }
      si = sj - 1;
      continue;
    }
    bool timed = x.c->profiling && s.kind != Step::WHILE && s.kind != Step::CASE;
    ExecCtx::Timed t;
    if (timed) {
      switch (s.kind) {
        case Step::KERNEL:
          t.kind = s.label.rfind("reduce_fusion", 0) == 0 ? "reduce" : "fused";
          t.key = s.label + " grid=" + std::to_string(s.grid[0]) + "x" + std::to_string(s.grid[1]);
          break;
        case Step::IGEMM:
          t.kind = "igemm";
          t.key = "igemm M=" + std::to_string(s.ig.M) + " N=" + std::to_string(s.ig.N) + " K=" + std::to_string(s.ig.K) +
                  " G=" + std::to_string(s.ig.groups) + " splitK=" + std::to_string(s.ig.split_k) + " a_mcontig=" +
                  std::to_string(s.ig.a_contig) + " b_kcontig=" + std::to_string(s.ig.b_contig) + " mask=" +
                  std::to_string(s.ig.needs_mask) + " ld=" + std::to_string(s.ig.ldh) + "x" + std::to_string(s.ig.ldw) + " vec=" + std::to_string(s.ig.vec) + " seg=" + std::to_string(s.ig.seg);
          if (!(x.c->tensor_cores && (long long)s.ig.M * s.ig.N * s.ig.K * s.ig.groups >= (1LL << 18) && s.ig.K >= 16))
            t.kind = "igemm_fma";
          break;
        case Step::ALL_REDUCE: t.kind = "all_reduce"; t.key = "all_reduce " + std::to_string(s.bytes); break;
        case Step::GEMM16:
          t.kind = s.g16.path == 0 ? "gemm16" : "gemv16";
          t.key = t.kind + " M=" + std::to_string(s.g16.M) + " N=" + std::to_string(s.g16.N) + " K=" + std::to_string(s.g16.K) +
                  " G=" + std::to_string(s.g16.G) + " a_kcontig=" + std::to_string(s.g16.a_ks == 1) + " b_kcontig=" +
                  std::to_string(s.g16.b_ks == 1) + " bn=" + std::to_string(s.g16.bn) + " splitK=" + std::to_string(s.g16.split_k);
          break;
        default: t.kind = "copy"; t.key = s.label; break;
      }
      cudaEventCreate(&t.a);
      cudaEventCreate(&t.b);
      cudaEventRecord(t.a, x.c->compute);
    }
    if (auto* e = run_step(x, s)) return e;
    if (timed) {
      cudaEventRecord(t.b, x.c->compute);
      x.timed.push_back(t);
    }
  }
  return nullptr;
}

uint64_t hash_text(const char* s, size_t n, uint64_t seed) {
  uint64_t h = 1469598103934665603ull ^ seed;
  for (size_t i = 0; i < n; i++) { h ^= (unsigned char)s[i]; h *= 1099511628211ull; }
  return h;
}

}  // namespace

// ===========================================================================
// C ABI
// ===========================================================================
extern "C" {

void b200_error_destroy(b200_error* err) { delete err; }
const char* b200_error_message(const b200_error* err) { return err ? err->message.c_str() : ""; }
b200_error_code b200_error_get_code(const b200_error* err) { return err ? err->code : B200_OK; }

b200_error* b200_nccl_unique_id(char out[B200_NCCL_ID_BYTES]) {
  NcclApi& n = nccl();
  if (!n.ok) return make_error(B200_FAILED_PRECONDITION, n.error);
  ncclUniqueId id;
  static_assert(sizeof(ncclUniqueId) == B200_NCCL_ID_BYTES, "NCCL id size");
  ncclResult_t r = n.GetUniqueId(&id);
  if (r != ncclSuccess) return make_error(B200_INTERNAL, std::string("ncclGetUniqueId: ") + n.GetErrorString(r));
  memcpy(out, &id, sizeof id);
  return nullptr;
}

namespace {
b200_error* create_client(const b200_client_options* o, ncclComm_t given_comm, b200_client** out);
}

b200_error* b200_client_create(const b200_client_options* o, b200_client** out) { return create_client(o, nullptr, out); }

namespace {
// `given_comm`: a communicator made for this device by ncclCommInitAll (several devices in one process); otherwise
// a job of several processes builds its own from the shared unique id.
b200_error* create_client(const b200_client_options* o, ncclComm_t given_comm, b200_client** out) {
  if (!out) return make_error(B200_INVALID_ARGUMENT, "client out-pointer is null");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return make_error(B200_FAILED_PRECONDITION,
                      std::string("no CUDA device available (this plugin has no CPU fallback): ") +
                          (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
  }
  auto c = std::make_unique<b200_client>();
  int ord = o ? o->device_ordinal : -1;
  if (ord < 0) {
    const char* lr = getenv("LOCAL_RANK");
    ord = lr ? atoi(lr) % count : 0;
  }
  if (ord >= count) return make_error(B200_INVALID_ARGUMENT, "device ordinal " + std::to_string(ord) + " out of range");
  c->ordinal = ord;
  c->rank = o ? o->process_index : 0;
  c->nprocs = (o && o->num_processes > 0) ? o->num_processes : 1;
  CUDA_TRY(cudaSetDevice(ord));
  CUDA_TRY(cudaFree(0));
  cudaDeviceProp prop;
  CUDA_TRY(cudaGetDeviceProperties(&prop, ord));
  c->kind = prop.name;
  c->total_mem = (int64_t)prop.totalGlobalMem;
  c->memory_debug = "B200 HBM of device " + std::to_string(c->rank) + " (" + std::to_string(prop.totalGlobalMem >> 20) + " MiB)";
  c->memory_string = "B200Memory(id=" + std::to_string(c->rank) + ", kind=device)";
  c->debug = "B200:" + std::to_string(c->rank) + " (cuda:" + std::to_string(ord) + ", sm_" + std::to_string(prop.major) +
             std::to_string(prop.minor) + ")";
  int rtv = 0;
  cudaRuntimeGetVersion(&rtv);
  c->version = "cuda " + std::to_string(rtv / 1000) + "." + std::to_string((rtv % 1000) / 10);
  if (prop.major != 10)
    logf(1, "warning: device %d is sm_%d%d; generated kernels target sm_100a", ord, prop.major, prop.minor);
  CUDA_TRY(cudaStreamCreateWithFlags(&c->compute, cudaStreamNonBlocking));
  CUDA_TRY(cudaStreamCreateWithFlags(&c->h2d, cudaStreamNonBlocking));
  CUDA_TRY(cudaStreamCreateWithFlags(&c->d2h, cudaStreamNonBlocking));
  CUDA_TRY(cudaDeviceGetDefaultMemPool(&c->pool, ord));
  uint64_t thr = (o && o->pool_release_threshold) ? o->pool_release_threshold : UINT64_MAX;
  CUDA_TRY(cudaMemPoolSetAttribute(c->pool, cudaMemPoolAttrReleaseThreshold, &thr));
  CUDA_TRY(cudaMallocHost((void**)&c->pred_host, 64));
  CUDA_TRY(cudaMalloc((void**)&c->error_flag, sizeof(int)));
  CUDA_TRY(cudaMalloc((void**)&c->loop_guard, sizeof(unsigned long long)));
  CUDA_TRY(cudaMemset(c->error_flag, 0, sizeof(int)));
  CUDA_TRY(cudaMallocHost((void**)&c->status_block, 2 * sizeof(int) * b200_client::kStatusPairs));
  memset(c->status_block, 0, 2 * sizeof(int) * b200_client::kStatusPairs);
  for (int k = b200_client::kStatusPairs - 1; k >= 0; k--) c->free_status.push_back(k);
  if (const char* e2 = getenv("B200_NO_TENSOR_CORES")) c->tensor_cores = atoi(e2) == 0;
  c->sw.no_vec_gather = getenv("B200_NO_VEC_GATHER") != nullptr;
  c->sw.no_seg_gather = getenv("B200_NO_SEG_GATHER") != nullptr;
  c->sw.no_tmem_a = getenv("B200_NO_TMEM_A") != nullptr;
  c->sw.no_half_ctas = getenv("B200_NO_HALF_CTAS") != nullptr;
  c->sw.narrow_tiles = getenv("B200_NARROW_TILES") != nullptr;
  c->sw.no_loop_graphs = getenv("B200_NO_LOOP_GRAPHS") != nullptr;
  c->sw.no_tma_a = getenv("B200_NO_TMA_A") != nullptr;
  c->sw.no_pdl = getenv("B200_NO_PDL") != nullptr;
  c->sw.no_device_cf = getenv("B200_NO_DEVICE_CONTROL_FLOW") != nullptr;
  if (const char* lim = getenv("B200_WHILE_TIME_LIMIT_S")) c->while_limit_s = std::max(0.001, atof(lim));
  set_programmatic_launch(!c->sw.no_pdl);
  set_igemm_programmatic_launch(!c->sw.no_pdl && !getenv("B200_NO_IGEMM_PDL"));
  if (!driver().ok) return make_error(B200_FAILED_PRECONDITION, driver().error);
  if (c->nprocs > 1) {
    NcclApi& n = nccl();
    if (!n.ok) return make_error(B200_FAILED_PRECONDITION, n.error);
    if (given_comm) c->comm = given_comm;
    else {
      if (!o->nccl_unique_id) return make_error(B200_INVALID_ARGUMENT, "num_processes > 1 needs nccl_unique_id");
      ncclUniqueId id;
      memcpy(&id, o->nccl_unique_id, sizeof id);
      // A small CTA budget for the communicator leaves the SMs to the backward pass while a gradient bucket is in
      // flight (the all-reduce then takes longer but hides under compute); B200_NCCL_MAX_CTAS sets it.
      const char* max_ctas = getenv("B200_NCCL_MAX_CTAS");
      ncclResult_t r;
      if (max_ctas && n.CommInitRankConfig && atoi(max_ctas) > 0) {
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.maxCTAs = atoi(max_ctas);
        cfg.minCTAs = 1;
        r = n.CommInitRankConfig(&c->comm, c->nprocs, id, c->rank, &cfg);
      } else {
        r = n.CommInitRank(&c->comm, c->nprocs, id, c->rank);
      }
      if (r != ncclSuccess) return make_error(B200_INTERNAL, std::string("ncclCommInitRank: ") + n.GetErrorString(r));
    }
    // collectives that overlap with compute run on a stream of their own, at the highest priority so that their
    // few CTAs find a place as soon as compute CTAs retire
    int lo = 0, hi = 0;
    CUDA_TRY(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    CUDA_TRY(cudaStreamCreateWithPriority(&c->coll, cudaStreamNonBlocking, hi));
    CUDA_TRY(cudaEventCreateWithFlags(&c->coll_ready, cudaEventDisableTiming));
    CUDA_TRY(cudaEventCreateWithFlags(&c->coll_done, cudaEventDisableTiming));
  }
  *out = c.release();
  return nullptr;
}
}  // namespace

b200_error* b200_client_destroy(b200_client* c) {
  if (!c) return nullptr;
  cudaSetDevice(c->ordinal);
  cudaDeviceSynchronize();
  c->cache.clear();
  if (c->comm) nccl().CommDestroy(c->comm);
  for (auto& b : c->pinned) {
    cudaFreeHost(b.ptr);
    cudaEventDestroy(b.ev);
  }
  if (c->pred_host) cudaFreeHost(c->pred_host);
  if (c->loop_guard) cudaFree(c->loop_guard);
  if (c->status_block) cudaFreeHost(c->status_block);
  if (c->error_flag) cudaFree(c->error_flag);
  if (c->coll) cudaStreamDestroy(c->coll);
  if (c->coll_ready) cudaEventDestroy(c->coll_ready);
  if (c->coll_done) cudaEventDestroy(c->coll_done);
  cudaStreamDestroy(c->compute);
  cudaStreamDestroy(c->h2d);
  cudaStreamDestroy(c->d2h);
  delete c;
  return nullptr;
}

const char* b200_client_platform_name(const b200_client*) { return "b200"; }
const char* b200_client_platform_version(const b200_client* c) { return c->version.c_str(); }
int b200_client_process_index(const b200_client* c) { return c->rank; }
int b200_client_device_count(const b200_client* c) { return c->nprocs; }
int b200_client_addressable_device_count(const b200_client*) { return 1; }
int b200_device_id(const b200_client* c) { return c->rank; }
int b200_device_local_hardware_id(const b200_client* c) { return c->ordinal; }
const char* b200_device_kind(const b200_client* c) { return c->kind.c_str(); }
const char* b200_device_debug_string(const b200_client* c) { return c->debug.c_str(); }
void* b200_client_compute_stream(b200_client* c) { return (void*)c->compute; }
int64_t b200_client_launch_count(const b200_client* c) { return c->launches.load(); }

b200_error* b200_device_memory_stats(b200_client* c, b200_memory_stats* s) {
  if (!c || !s) return make_error(B200_INVALID_ARGUMENT, "null argument");
  if (auto* e = set_device(c)) return e;
  s->bytes_in_use = c->bytes_in_use.load();
  s->peak_bytes_in_use = c->peak_bytes.load(); s->peak_bytes_in_use_is_set = 1;
  s->bytes_limit = c->total_mem; s->bytes_limit_is_set = 1;
  uint64_t v = 0;
  s->pool_bytes_is_set = cudaMemPoolGetAttribute(c->pool, cudaMemPoolAttrReservedMemCurrent, &v) == cudaSuccess;
  s->pool_bytes = (int64_t)v;
  s->peak_pool_bytes_is_set = cudaMemPoolGetAttribute(c->pool, cudaMemPoolAttrReservedMemHigh, &v) == cudaSuccess;
  s->peak_pool_bytes = (int64_t)v;
  s->num_allocs = c->num_allocs.load(); s->num_allocs_is_set = 1;
  s->largest_alloc_size = c->largest_alloc.load(); s->largest_alloc_size_is_set = 1;
  return nullptr;
}

b200_error* b200_client_set_profiling(b200_client* c, int enabled) {
  if (!c) return make_error(B200_INVALID_ARGUMENT, "null client");
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  c->profiling = enabled != 0;
  return nullptr;
}

b200_error* b200_client_profile_report(b200_client* c, char** json) {
  if (!c || !json) return make_error(B200_INVALID_ARGUMENT, "null argument");
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  std::string out = "[";
  bool first = true;
  for (auto& kv : c->profile) {
    std::string key;
    for (char ch : kv.first) { if (ch == '"' || ch == '\\') key += '\\'; key += ch; }
    char buf[64];
    snprintf(buf, sizeof buf, "%.6f", kv.second.ms);
    out += std::string(first ? "" : ",") + "{\"kind\":\"" + kv.second.kind + "\",\"key\":\"" + key + "\",\"ms\":" + buf +
           ",\"count\":" + std::to_string(kv.second.count) + "}";
    first = false;
  }
  out += "]";
  c->profile.clear();
  *json = strdup(out.c_str());
  return nullptr;
}

b200_error* b200_client_synchronize(b200_client* c) {
  if (auto* e = set_device(c)) return e;
  CUDA_TRY(cudaStreamSynchronize(c->h2d));
  CUDA_TRY(cudaStreamSynchronize(c->compute));
  CUDA_TRY(cudaStreamSynchronize(c->d2h));
  int flag = 0;
  CUDA_TRY(cudaMemcpy(&flag, c->error_flag, sizeof(int), cudaMemcpyDeviceToHost));
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (flag != c->reported_errors) {
    c->reported_errors = flag;
    return make_error(B200_INTERNAL, "a kernel gave up on a bounded wait (tensor-core pipeline did not complete); "
                                     "results of the affected execution are invalid");
  }
  return nullptr;
}

// ---- compile -------------------------------------------------------------------
b200_error* b200_client_compile(b200_client* c, const char* code, size_t code_size, const char* format,
                                const b200_compile_options* o, b200_executable** out) {
  if (!c || !code || !out) return make_error(B200_INVALID_ARGUMENT, "null argument");
  *out = nullptr;
  std::string fmt = format ? format : "mlir";
  if (fmt != "mlir" && fmt != "hlo" && fmt != "hlo_with_config")
    return make_error(B200_INVALID_ARGUMENT, "unknown program format '" + fmt + "'");
  if (code_size >= 4 && memcmp(code, "ML\xefR", 4) == 0)
    return make_error(B200_UNIMPLEMENTED,
                      "MLIR bytecode (VHLO portable artifact) cannot be read without the StableHLO libraries; "
                      "pass the module as text");
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (auto* e = set_device(c)) return e;
  CompileOptions co;
  co.fuse = !(o && o->disable_fusion) && !(getenv("B200_NO_FUSE") && atoi(getenv("B200_NO_FUSE")));
  co.partition_id = c->rank;
  co.num_partitions = c->nprocs;
  char key[64];
  // planning switches read from the environment are part of the key (a plan made with one setting must not answer
  // for another)
  unsigned env_bits = 0;
  {
    static const char* names[] = {"B200_NO_WINDOW_UPDATE", "B200_NO_FLAT_ALL_REDUCE", "B200_NO_GEMM16", "B200_NO_ROW_FUSION",
                                  "B200_NO_WEIGHT_HOIST", "B200_NO_LICM", "B200_NO_CSE", "B200_NO_HOIST", "B200_NO_BUNDLES",
                                  "B200_NO_TILED_TRANSPOSE", "B200_NO_ALL_REDUCE_OVERLAP", "B200_DEBUG_NO_REUSE", "B200_NO_COL4",
                                  "B200_NO_ATTENTION_FUSION", "B200_NO_WIDE_POINTWISE", "B200_NO_WIDE_ROWS"};
    for (size_t k = 0; k < sizeof names / sizeof names[0]; k++)
      if (getenv(names[k])) env_bits |= 1u << k;
  }
  snprintf(key, sizeof key, "%016llx-%d-%d-%d-%x", (unsigned long long)hash_text(code, code_size, 0), (int)co.fuse, c->rank,
           c->nprocs, env_bits);
  auto hit = c->cache.find(key);
  std::shared_ptr<LoadedProgram> lp;
  if (hit != c->cache.end()) {
    lp = hit->second.lock();
    if (lp && (lp->text.size() != code_size || memcmp(lp->text.data(), code, code_size) != 0)) lp.reset();   // same hash, other text
  }
  if (!lp) {
    lp = std::make_shared<LoadedProgram>();
    lp->text.assign(code, code_size);
    try {
      auto m = parse_module(code, code_size);
      int np = (o && o->num_partitions > 0) ? o->num_partitions : 0;
      if (np == 0 && m->attrs.count("mhlo.num_partitions")) np = (int)attr_int(m->attrs.at("mhlo.num_partitions"));
      if (np > 1 && np != c->nprocs)
        return make_error(B200_INVALID_ARGUMENT, "program wants " + std::to_string(np) + " partitions but the job has " +
                                                     std::to_string(c->nprocs) + " processes");
      lp->prog = compile_module(*m, co);
    } catch (const CompileError& e) {
      return make_error(B200_INVALID_ARGUMENT, e.what());
    } catch (const std::exception& e) {
      return make_error(B200_INTERNAL, std::string("compiler failure: ") + e.what());
    }
    if (const char* d = getenv("B200_DUMP_PLAN")) {
      if (FILE* f = fopen(d, "a")) { fputs(lp->prog->dump.c_str(), f); fclose(f); }
      else fputs(lp->prog->dump.c_str(), stderr);
    }
    if (auto* e = build_kernels(*lp)) return e;
    // constants: one device block, uploaded once
    CompiledProgram& p = *lp->prog;
    size_t total = 0;
    std::vector<size_t> offs(p.consts.size());
    for (size_t k = 0; k < p.consts.size(); k++) {
      offs[k] = total;
      total += (p.consts[k].bytes.size() + 255) & ~(size_t)255;
    }
    if (total) {
      CUDA_TRY(cudaMalloc(&lp->const_block, total));
      std::vector<uint8_t> host(total, 0);
      for (size_t k = 0; k < p.consts.size(); k++)
        memcpy(host.data() + offs[k], p.consts[k].bytes.data(), p.consts[k].bytes.size());
      CUDA_TRY(cudaMemcpy(lp->const_block, host.data(), total, cudaMemcpyHostToDevice));
    }
    for (size_t k = 0; k < p.consts.size(); k++) lp->const_ptrs.push_back((char*)lp->const_block + offs[k]);
    for (size_t a = 0; a < p.arena_bytes.size(); a++) {
      void* ptr = nullptr;
      if (p.arena_bytes[a]) {
        cudaError_t e = cudaMalloc(&ptr, p.arena_bytes[a]);
        if (e != cudaSuccess) {
          cudaGetLastError();
          return make_error(B200_RESOURCE_EXHAUSTED, "cannot allocate " + std::to_string(p.arena_bytes[a]) +
                                                         " bytes of temporaries: " + cudaGetErrorString(e));
        }
      }
      lp->arenas.push_back(ptr);
    }
    c->cache[key] = lp;
    logf(2, "compiled %s: %zu generated kernels, %zu constants, arena %zu bytes", p.name.c_str(), p.kernels.size(),
         p.consts.size(), p.arena_bytes[0]);
  }
  auto* exe = new b200_executable();
  exe->client = c;
  exe->lp = lp;
  *out = exe;
  return nullptr;
}

void b200_string_free(char* s) { free(s); }

b200_error* b200_compile_to_plan(const char* code, size_t code_size, const b200_compile_options* o, int num_processes,
                                 int process_index, int validate_kernels, char** plan_text, char** cuda_source) {
  if (!code) return make_error(B200_INVALID_ARGUMENT, "null program");
  if (plan_text) *plan_text = nullptr;
  if (cuda_source) *cuda_source = nullptr;
  CompileOptions co;
  co.fuse = !(o && o->disable_fusion) && !(getenv("B200_NO_FUSE") && atoi(getenv("B200_NO_FUSE")));
  co.num_partitions = num_processes > 0 ? num_processes : 1;
  co.partition_id = process_index;
  std::unique_ptr<CompiledProgram> prog;
  try {
    auto m = parse_module(code, code_size);
    prog = compile_module(*m, co);
  } catch (const CompileError& e) {
    return make_error(B200_INVALID_ARGUMENT, e.what());
  } catch (const std::exception& e) {
    return make_error(B200_INTERNAL, std::string("compiler failure: ") + e.what());
  }
  std::string src = codegen_prelude();
  for (auto& k : prog->kernels) src += k.body + "\n";
  if ((validate_kernels & 1) && !prog->kernels.empty()) {
    NvrtcApi& rt = nvrtc();
    if (!rt.ok) return make_error(B200_FAILED_PRECONDITION, "NVRTC unavailable: " + rt.error);
    nvrtcProgram np;
    if (rt.CreateProgram(&np, src.c_str(), "b200_fused.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
      return make_error(B200_INTERNAL, "nvrtcCreateProgram failed");
    const char* opts[] = {"--gpu-architecture=sm_100a", "-std=c++17", "-w"};
    nvrtcResult r = rt.CompileProgram(np, 3, opts);
    if (r != NVRTC_SUCCESS) {
      size_t ls = 0;
      rt.GetProgramLogSize(np, &ls);
      std::string log(ls, '\0');
      if (ls) rt.GetProgramLog(np, &log[0]);
      rt.DestroyProgram(&np);
      return make_error(B200_INTERNAL, std::string("generated kernels do not compile: ") + log.substr(0, 4000));
    }
    rt.DestroyProgram(&np);
  }
  std::string text = prog->dump;
  if (validate_kernels & 2) {
    // the memory the plan's steps name: arguments, results, constants with their bytes, temporaries
    static const char* kinds[] = {"arg", "const", "temp", "result"};
    std::ostringstream os;
    os << "slots:\n";
    for (size_t k = 0; k < prog->slots.size(); k++) {
      const Slot& sl = prog->slots[k];
      os << "  slot " << k << " " << kinds[(int)sl.kind] << " index=" << sl.index << " arena=" << sl.arena << " offset=" << sl.offset
         << " bytes=" << sl.bytes << " " << sl.type.str();
      if (sl.kind == Slot::CONST && sl.index >= 0 && (size_t)sl.index < prog->consts.size()) {
        const auto& b = prog->consts[sl.index].bytes;
        os << " hex=";
        if (b.size() <= (1u << 20)) {
          static const char* digits = "0123456789abcdef";
          for (uint8_t c : b) os << digits[c >> 4] << digits[c & 15];
        } else os << "-";
      }
      os << "\n";
    }
    for (size_t k = 0; k < prog->results.size(); k++) os << "  result " << k << " slot=" << prog->results[k].slot << " " << prog->results[k].type.str() << "\n";
    // the top-level steps with every argument (the plan text above abbreviates long argument lists)
    os << "launches:\n";
    for (const Step& st : prog->main.steps) {
      if (st.kind == Step::KERNEL) {
        os << "  kernel " << prog->kernels[st.kernel].name << " grid=" << st.grid[0] << "x" << st.grid[1] << "x" << st.grid[2] << " block="
           << st.block[0] << "x" << st.block[1] << "x" << st.block[2] << " args=[";
        for (size_t k = 0; k < st.args.size(); k++) os << (k ? "," : "") << st.args[k];
        os << "]\n";
      } else if (st.kind == Step::MEMCPY) {
        os << "  memcpy bytes=" << st.bytes << " args=[" << st.args[0] << "," << st.args[1] << "]\n";
      } else if (st.kind == Step::SCATTER && st.iparams.size() > 5 && st.iparams[5] == 1) {
        // the general scatter between its generated key kernel and (for update computations of their own) its generated
        // apply kernel: sorts the (destination, update) pairs in the scratch and, for a built-in computation, applies them
        os << "  scatter_elems numel=" << st.iparams[0] << " updates=" << st.iparams[2] << " computation=" << st.iparams[4] << " bytes=" << st.bytes
           << " args=[";
        for (size_t k = 0; k < st.args.size(); k++) os << (k ? "," : "") << st.args[k];
        os << "]\n";
      } else {
        os << "  other kind=" << (int)st.kind << " " << st.label << "\n";
      }
    }
    text += os.str();
  }
  if (plan_text) *plan_text = strdup(text.c_str());
  if (cuda_source) *cuda_source = strdup(src.c_str());
  return nullptr;
}

b200_error* b200_executable_destroy(b200_executable* e) {
  if (!e) return nullptr;
  b200_client* c = e->client;
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (e->lp.use_count() == 1) {
    // the last handle: the device must be done with the plan's memory before it is freed
    cudaSetDevice(c->ordinal);
    cudaStreamSynchronize(c->compute);
  }
  delete e;
  return nullptr;
}
const char* b200_executable_name(const b200_executable* e) { return e->lp->prog->name.c_str(); }
const char* b200_executable_fingerprint(const b200_executable* e) { return e->lp->prog->fingerprint.c_str(); }
int b200_executable_num_replicas(const b200_executable* e) { return e->lp->prog->num_replicas; }
int b200_executable_num_partitions(const b200_executable* e) { return e->lp->prog->num_partitions; }
size_t b200_executable_num_args(const b200_executable* e) { return e->lp->prog->arg_types.size(); }
size_t b200_executable_num_outputs(const b200_executable* e) { return e->lp->prog->results.size(); }
int64_t b200_executable_launches_per_execute(const b200_executable* e) { return e->lp->prog->launches_per_execute; }
int64_t b200_executable_num_kernels(const b200_executable* e) { return (int64_t)e->lp->prog->kernels.size(); }
int64_t b200_executable_temp_bytes(const b200_executable* e) {
  int64_t t = 0;
  for (auto b : e->lp->prog->arena_bytes) t += (int64_t)b;
  return t;
}
const char* b200_executable_plan_text(const b200_executable* e) { return e->lp->prog->dump.c_str(); }

b200_error* b200_executable_output_info(const b200_executable* e, size_t i, b200_dtype* dt, const int64_t** dims,
                                        size_t* nd) {
  auto& r = e->lp->prog->results;
  if (i >= r.size()) return make_error(B200_INVALID_ARGUMENT, "output index out of range");
  if (dt) *dt = to_api(r[i].type.dt);
  if (dims) *dims = r[i].type.dims.data();
  if (nd) *nd = r[i].type.dims.size();
  return nullptr;
}
b200_error* b200_executable_arg_info(const b200_executable* e, size_t i, b200_dtype* dt, const int64_t** dims, size_t* nd) {
  auto& a = e->lp->prog->arg_types;
  if (i >= a.size()) return make_error(B200_INVALID_ARGUMENT, "argument index out of range");
  if (dt) *dt = to_api(a[i].dt);
  if (dims) *dims = a[i].dims.data();
  if (nd) *nd = a[i].dims.size();
  return nullptr;
}

// ---- buffers ----------------------------------------------------------------------
b200_error* b200_buffer_from_host(b200_client* c, const void* data, b200_dtype dtype, const int64_t* dims, size_t nd,
                                  const int64_t* byte_strides, b200_buffer** out, b200_event** done) {
  if (!c || !out) return make_error(B200_INVALID_ARGUMENT, "null argument");
  *out = nullptr;
  if (done) *done = nullptr;
  size_t es = dtype_size(dtype);
  if (!es) return make_error(B200_INVALID_ARGUMENT, "unsupported element type " + std::to_string((int)dtype));
  size_t count = 1;
  for (size_t d = 0; d < nd; d++) {
    if (dims[d] < 0) return make_error(B200_INVALID_ARGUMENT, "negative dimension");
    count *= (size_t)dims[d];
  }
  size_t bytes = count * es;
  // null data only for zero-size arrays (pjrt_client.cc:285-295)
  if (!data && bytes) return make_error(B200_INVALID_ARGUMENT, "host data pointer is null for a non-empty array");
  bool dense = true;
  if (byte_strides) {
    int64_t st = (int64_t)es;
    for (int d = (int)nd - 1; d >= 0; d--) {
      if (byte_strides[d] < 0) return make_error(B200_INVALID_ARGUMENT, "negative byte strides are not supported");   // mlx_buffer.cc:157-163
      if (dims[d] > 1 && byte_strides[d] != st) dense = false;
      st *= dims[d];
    }
  }
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (auto* e = set_device(c)) return e;
  auto b = std::make_unique<b200_buffer>();
  b->client = c;
  b->dtype = dtype;
  b->dims.assign(dims, dims + nd);
  b->bytes = bytes;
  if (auto* e = device_alloc(c, bytes, c->h2d, &b->ptr)) return e;
  bool host_ready_now = true;
  if (bytes) {
    cudaPointerAttributes attr;
    bool pinned = dense && cudaPointerGetAttributes(&attr, data) == cudaSuccess && attr.type == cudaMemoryTypeHost;
    cudaGetLastError();
    if (pinned) {
      CUDA_TRY(cudaMemcpyAsync(b->ptr, data, bytes, cudaMemcpyHostToDevice, c->h2d));
      host_ready_now = false;
    } else if (bytes <= (256u << 20)) {
      int idx = -1;
      void* stage = acquire_pinned(c, bytes, &idx);
      if (!stage) return make_error(B200_RESOURCE_EXHAUSTED, "cannot allocate pinned staging memory");
      if (dense) memcpy(stage, data, bytes);
      else pack_strided((const char*)data, (char*)stage, dims, byte_strides, nd, es);
      CUDA_TRY(cudaMemcpyAsync(b->ptr, stage, bytes, cudaMemcpyHostToDevice, c->h2d));
      CUDA_TRY(cudaEventRecord(c->pinned[idx].ev, c->h2d));
      c->pinned[idx].in_flight = true;
    } else {
      std::vector<char> tmp;
      const void* src = data;
      if (!dense) {
        tmp.resize(bytes);
        pack_strided((const char*)data, tmp.data(), dims, byte_strides, nd, es);
        src = tmp.data();
      }
      CUDA_TRY(cudaMemcpyAsync(b->ptr, src, bytes, cudaMemcpyHostToDevice, c->h2d));
      CUDA_TRY(cudaStreamSynchronize(c->h2d));
    }
  }
  CUDA_TRY(cudaEventCreateWithFlags(&b->ready, cudaEventDisableTiming));
  CUDA_TRY(cudaEventRecord(b->ready, c->h2d));
  b->ready_on = c->h2d;
  if (done) {
    if (host_ready_now) *done = new b200_event();
    else {
      b200_error* err = nullptr;
      *done = new_event_on(c, c->h2d, &err);
      if (err) return err;
    }
  }
  *out = b.release();
  return nullptr;
}

b200_error* b200_buffer_to_host(b200_buffer* b, void* dst, size_t* dst_size, b200_event** event) {
  if (!b) return make_error(B200_INVALID_ARGUMENT, "null buffer");
  if (event) *event = nullptr;
  if (!dst) {
    if (dst_size) *dst_size = b->bytes;
    return nullptr;
  }
  if (b->deleted) return make_error(B200_INVALID_ARGUMENT, "buffer has been deleted or donated");
  if (dst_size && *dst_size < b->bytes) return make_error(B200_INVALID_ARGUMENT, "destination too small");
  b200_client* c = b->client;
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (auto* e = set_device(c)) return e;
  CUDA_TRY(cudaStreamWaitEvent(c->d2h, b->ready, 0));
  if (b->bytes) CUDA_TRY(cudaMemcpyAsync(dst, b->ptr, b->bytes, cudaMemcpyDeviceToHost, c->d2h));
  cudaEvent_t rd;
  CUDA_TRY(cudaEventCreateWithFlags(&rd, cudaEventDisableTiming));
  CUDA_TRY(cudaEventRecord(rd, c->d2h));
  // drop finished read markers, keep this one so deletion waits for the copy
  for (auto it = b->reads.begin(); it != b->reads.end();) {
    if (cudaEventQuery(*it) == cudaSuccess) { cudaEventDestroy(*it); it = b->reads.erase(it); }
    else ++it;
  }
  b->reads.push_back(rd);
  if (event) {
    b200_error* err = nullptr;
    *event = new_event_on(c, c->d2h, &err);
    if (err) return err;
    (*event)->status = b->status;
  } else {
    CUDA_TRY(cudaStreamSynchronize(c->d2h));
    if (b->status && b->status->failed())
      return make_error(B200_INTERNAL, "the execution that produced this buffer gave up on a bounded device-side wait; its results are invalid");
  }
  return nullptr;
}

b200_dtype b200_buffer_dtype(const b200_buffer* b) { return b->dtype; }
size_t b200_buffer_num_dims(const b200_buffer* b) { return b->dims.size(); }
const int64_t* b200_buffer_dims(const b200_buffer* b) { return b->dims.data(); }
size_t b200_buffer_on_device_size(const b200_buffer* b) { return b->bytes; }
int b200_buffer_device(const b200_buffer* b) { return b->client->rank; }
void* b200_buffer_device_pointer(const b200_buffer* b) { return b->deleted ? nullptr : b->ptr; }
int b200_buffer_is_deleted(const b200_buffer* b) { return b->deleted ? 1 : 0; }

b200_error* b200_buffer_ready_event(b200_buffer* b, b200_event** event) {
  if (!b || !event) return make_error(B200_INVALID_ARGUMENT, "null argument");
  if (b->deleted) return make_error(B200_INVALID_ARGUMENT, "buffer has been deleted or donated");
  b200_client* c = b->client;
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (auto* e = set_device(c)) return e;
  // a fresh event on the d2h stream ordered after the buffer's producer
  CUDA_TRY(cudaStreamWaitEvent(c->d2h, b->ready, 0));
  b200_error* err = nullptr;
  *event = new_event_on(c, c->d2h, &err);
  if (*event) (*event)->status = b->status;
  return err;
}

b200_error* b200_buffer_delete(b200_buffer* b) {
  if (!b || b->deleted) return nullptr;
  b200_client* c = b->client;
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (auto* e = set_device(c)) return e;
  b->deleted = true;
  if (b->ptr) {
    // the free is ordered on the compute stream: only a producer on another stream needs a wait
    if (b->ready && b->ready_on != c->compute) cudaStreamWaitEvent(c->compute, b->ready, 0);
    for (auto ev : b->reads) {
      cudaStreamWaitEvent(c->compute, ev, 0);
      cudaEventDestroy(ev);
    }
    b->reads.clear();
    if (b->block) {
      if (--b->block->refs == 0) {
        cudaFreeAsync(b->block->base, c->compute);
        delete b->block;
      }
      b->block = nullptr;
    } else {
      cudaFreeAsync(b->ptr, c->compute);
    }
    c->note_free(std::max<size_t>(b->bytes, 16));
    b->ptr = nullptr;
  }
  return nullptr;
}

b200_error* b200_buffer_destroy(b200_buffer* b) {
  if (!b) return nullptr;
  b200_error* e = b200_buffer_delete(b);
  if (b->ready) cudaEventDestroy(b->ready);
  for (auto ev : b->reads) cudaEventDestroy(ev);
  delete b;
  return e;
}

b200_error* b200_buffer_copy(b200_buffer* b, b200_buffer** out) {
  if (!b || !out) return make_error(B200_INVALID_ARGUMENT, "null argument");
  if (b->deleted) return make_error(B200_INVALID_ARGUMENT, "buffer has been deleted or donated");
  b200_client* c = b->client;
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (auto* e = set_device(c)) return e;
  auto n = std::make_unique<b200_buffer>();
  n->client = c;
  n->dtype = b->dtype;
  n->dims = b->dims;
  n->bytes = b->bytes;
  if (auto* e = device_alloc(c, b->bytes, c->compute, &n->ptr)) return e;
  CUDA_TRY(cudaStreamWaitEvent(c->compute, b->ready, 0));
  if (b->bytes) CUDA_TRY(cudaMemcpyAsync(n->ptr, b->ptr, b->bytes, cudaMemcpyDeviceToDevice, c->compute));
  CUDA_TRY(cudaEventCreateWithFlags(&n->ready, cudaEventDisableTiming));
  CUDA_TRY(cudaEventRecord(n->ready, c->compute));
  n->ready_on = c->compute;
  *out = n.release();
  return nullptr;
}

// ---- execute -------------------------------------------------------------------------
b200_error* b200_executable_execute(b200_executable* exe, b200_buffer* const* args, size_t num_args, b200_buffer** outputs,
                                    b200_event** done, const b200_execute_options* opts) {
  if (!exe || (!outputs && !exe->lp->prog->results.empty())) return make_error(B200_INVALID_ARGUMENT, "null argument");
  if (done) *done = nullptr;
  b200_client* c = exe->client;
  CompiledProgram& p = *exe->lp->prog;
  if (num_args != p.arg_types.size())
    return make_error(B200_INVALID_ARGUMENT, "executable takes " + std::to_string(p.arg_types.size()) + " arguments, got " +
                                                 std::to_string(num_args));
  for (size_t k = 0; k < num_args; k++) {
    b200_buffer* b = args[k];
    if (!b) return make_error(B200_INVALID_ARGUMENT, "argument " + std::to_string(k) + " is null");
    if (b->deleted) return make_error(B200_INVALID_ARGUMENT, "argument " + std::to_string(k) + " has been deleted or donated");
    if (b->client != c) return make_error(B200_INVALID_ARGUMENT, "argument " + std::to_string(k) + " lives on another client");
    const TensorType& t = p.arg_types[k];
    if (t.dt == DT::TOKEN) continue;
    if (to_api(t.dt) != b->dtype || t.dims != b->dims)
      return make_error(B200_INVALID_ARGUMENT, "argument " + std::to_string(k) + " does not match the program's " + t.str());
  }
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (auto* e = set_device(c)) return e;
  bool donate = opts && opts->donate_arguments;
  ExecCtx x;
  x.c = c;
  x.lp = exe->lp.get();
  x.ptrs.assign(p.slots.size(), nullptr);
  // arguments produced on the compute stream itself (the outputs of earlier executions) are ordered already
  for (size_t k = 0; k < num_args; k++)
    if (args[k]->ready_on != c->compute) CUDA_TRY(cudaStreamWaitEvent(c->compute, args[k]->ready, 0));
  std::vector<std::unique_ptr<b200_buffer>> outs(p.results.size());
  // Donation (tf.aliasing_output on an argument): the argument is consumed. Its buffer is left deleted and its memory
  // goes back to the stream-ordered pool behind this execution, where the next allocation of the stream finds it; the
  // results themselves are fresh allocations (the kernels are free to write a result before they have read all of
  // the argument, so the two never share storage).
  std::vector<bool> arg_taken(num_args, false);
  // the error counter as this execution sees it before its first and after its last kernel
  auto status = std::make_shared<ExecStatus>();
  if (!c->free_status.empty()) {
    const int slot = c->free_status.back();
    c->free_status.pop_back();
    status->pair = c->status_block + 2 * slot;
    status->pair[0] = status->pair[1] = 0;
    status->release = [c, slot](volatile int*) { std::lock_guard<std::recursive_mutex> l(c->mu); c->free_status.push_back(slot); };
    CUDA_TRY(cudaMemcpyAsync((void*)&status->pair[0], c->error_flag, sizeof(int), cudaMemcpyDeviceToHost, c->compute));
  }
  if (c->armed_wait_polls > 0) {
    cudaError_t he = b200::launch_expiring_wait(c->armed_wait_polls, c->error_flag, c->compute);
    c->armed_wait_polls = 0;
    if (he != cudaSuccess) return make_error(B200_INTERNAL, std::string("test hook launch failed: ") + cudaGetErrorString(he));
  }
  for (size_t k = 0; k < p.results.size(); k++) {
    auto b = std::make_unique<b200_buffer>();
    b->client = c;
    b->dtype = to_api(p.results[k].type.dt);
    b->dims = p.results[k].type.dims;
    b->bytes = p.results[k].type.bytes();
    b->status = status;
    int da = p.results[k].donated_arg;
    if (donate && da >= 0 && (size_t)da < num_args) arg_taken[da] = true;
    outs[k] = std::move(b);
  }
  // Results come out of two allocations per execution instead of one each: one block for the small results (under
  // 64 KB: scalars, statistics vectors) and one for the large ones (parameters, optimizer state), each freed when
  // its last buffer is deleted. A scalar that the caller keeps (a loss) therefore pins the small block only.
  {
    size_t total[2] = {0, 0};
    int count[2] = {0, 0};
    auto cls = [](size_t bytes) { return bytes < 65536 ? 0 : 1; };
    auto padded = [](size_t bytes) { return (std::max<size_t>(bytes, 16) + 255) & ~(size_t)255; };
    for (auto& b : outs) { total[cls(b->bytes)] += padded(b->bytes); count[cls(b->bytes)]++; }
    b200_buffer::Block* blocks[2] = {nullptr, nullptr};
    for (int g = 0; g < 2; g++) {
      if (count[g] < 2) continue;
      void* base = nullptr;
      cudaError_t e = cudaMallocAsync(&base, total[g], c->compute);
      if (e != cudaSuccess) {
        cudaGetLastError();
        if (blocks[0]) { cudaFreeAsync(blocks[0]->base, c->compute); delete blocks[0]; }
        return make_error(B200_RESOURCE_EXHAUSTED, "device allocation of " + std::to_string(total[g]) + " bytes for " +
                                                       std::to_string(count[g]) + " results failed: " + cudaGetErrorString(e));
      }
      blocks[g] = new b200_buffer::Block{base, 0};
    }
    size_t at[2] = {0, 0};
    for (auto& b : outs) {
      const int g = cls(b->bytes);
      if (!blocks[g]) continue;
      b->block = blocks[g];
      b->ptr = (char*)blocks[g]->base + at[g];
      at[g] += padded(b->bytes);
      blocks[g]->refs++;
      c->note_alloc(std::max<size_t>(b->bytes, 16));
    }
    for (auto& b : outs) {
      if (b->ptr) continue;
      if (auto* e = device_alloc(c, b->bytes, c->compute, &b->ptr)) {
        for (auto& o : outs)
          if (o->ptr) b200_buffer_delete(o.get());
        return e;
      }
    }
  }
  for (size_t s = 0; s < p.slots.size(); s++) {
    const Slot& sl = p.slots[s];
    switch (sl.kind) {
      case Slot::ARG: x.ptrs[s] = args[sl.index]->ptr; break;
      case Slot::CONST: x.ptrs[s] = exe->lp->const_ptrs[sl.index]; break;
      case Slot::TEMP: x.ptrs[s] = (char*)exe->lp->arenas[sl.arena] + sl.offset; break;
      case Slot::RESULT: x.ptrs[s] = outs[sl.index]->ptr; break;
    }
  }
  b200_error* err = run_plan(x, p.main);
  if (x.coll_pending) cudaStreamWaitEvent(c->compute, c->coll_done, 0);   // a plan that ended early still joins
  c->launches += x.launches;
  if (!x.timed.empty()) {
    cudaStreamSynchronize(c->compute);
    for (auto& t : x.timed) {
      float ms = 0;
      cudaEventElapsedTime(&ms, t.a, t.b);
      auto& pe = c->profile[t.key];
      pe.kind = t.kind;
      pe.ms += ms;
      pe.count++;
      cudaEventDestroy(t.a);
      cudaEventDestroy(t.b);
    }
  }
  if (err) {
    for (auto& b : outs)
      if (b && b->ptr) b200_buffer_delete(b.get());
    return err;
  }
  for (size_t k = 0; k < outs.size(); k++) {
    CUDA_TRY(cudaEventCreateWithFlags(&outs[k]->ready, cudaEventDisableTiming));
    CUDA_TRY(cudaEventRecord(outs[k]->ready, c->compute));
    outs[k]->ready_on = c->compute;
  }
  if (donate) {
    // donated arguments are consumed (PJRT semantics): their memory returns to the pool in stream order
    for (size_t k = 0; k < num_args; k++)
      if (arg_taken[k]) b200_buffer_delete(args[k]);
  }
  if (status->pair)
    CUDA_TRY(cudaMemcpyAsync((void*)&status->pair[1], c->error_flag, sizeof(int), cudaMemcpyDeviceToHost, c->compute));
  if (done) {
    b200_error* e2 = nullptr;
    *done = new_event_on(c, c->compute, &e2);
    if (e2) return e2;
    (*done)->status = status;
  }
  for (size_t k = 0; k < outs.size(); k++) outputs[k] = outs[k].release();
  return nullptr;
}

// ---- events ------------------------------------------------------------------------------
int b200_event_is_ready(b200_event* e) {
  if (!e || !e->ev) return 1;
  return cudaEventQuery(e->ev) != cudaErrorNotReady;
}

b200_error* b200_event_await(b200_event* e) {
  if (!e) return make_error(B200_INVALID_ARGUMENT, "null event");
  if (e->ev) {
    cudaError_t r = cudaEventSynchronize(e->ev);
    if (r != cudaSuccess) {
      e->error = std::string("device work failed: ") + cudaGetErrorString(r);
      e->code = B200_INTERNAL;
    }
  }
  return b200_event_error(e);
}

b200_error* b200_event_error(b200_event* e) {
  if (!e) return nullptr;
  if (e->error.empty() && e->status && e->status->failed() && (!e->ev || cudaEventQuery(e->ev) == cudaSuccess)) {
    e->error = "the execution gave up on a bounded device-side wait (a tensor-core pipeline did not complete); its results are invalid";
    e->code = B200_INTERNAL;
  }
  if (e->error.empty()) return nullptr;
  return make_error(e->code, e->error);
}

b200_error* b200_event_on_ready(b200_event* e, b200_event_callback cb, void* user_arg) {
  if (!e || !cb) return make_error(B200_INVALID_ARGUMENT, "null argument");
  if (!e->ev) {
    cb(b200_event_error(e), user_arg);
    return nullptr;
  }
  cudaEvent_t ev = e->ev;
  int dev = e->device;
  std::shared_ptr<ExecStatus> status = e->status;
  // The waiter needs its own handle on completion: record-independent wait through a second event
  // is not possible, so the callback thread synchronises on the same CUDA event; destroying the
  // b200_event before the callback fired is therefore not allowed (same rule as PJRT).
  completion().post([ev, dev, cb, user_arg, status] {
    cudaSetDevice(dev);
    cudaError_t r = cudaEventSynchronize(ev);
    b200_error* err = r == cudaSuccess ? nullptr : make_error(B200_INTERNAL, std::string("device work failed: ") + cudaGetErrorString(r));
    if (!err && status && status->failed())
      err = make_error(B200_INTERNAL, "the execution gave up on a bounded device-side wait; its results are invalid");
    cb(err, user_arg);
  });
  return nullptr;
}

b200_error* b200_event_destroy(b200_event* e) {
  delete e;
  return nullptr;
}

// ---- memory spaces, topology, device assignment, profiler stub ---------------------------------------------------
int b200_device_num_memories(const b200_client*) { return 1; }
int b200_memory_id(const b200_client* c, int) { return c->rank; }
const char* b200_memory_kind(const b200_client*, int) { return "device"; }
int b200_memory_kind_id(const b200_client*, int) { return 0; }
const char* b200_memory_debug_string(const b200_client* c, int) { return c->memory_debug.c_str(); }
const char* b200_memory_to_string(const b200_client* c, int) { return c->memory_string.c_str(); }
int b200_buffer_memory(const b200_buffer* b) { return b->client->rank; }

b200_error* b200_memory_addressable_by_devices(const b200_client* c, int memory_index, int* device_ids, size_t capacity,
                                               size_t* num_devices) {
  if (!c || !num_devices) return make_error(B200_INVALID_ARGUMENT, "null argument");
  if (memory_index != 0) return make_error(B200_INVALID_ARGUMENT, "a device has one memory space (index 0)");
  *num_devices = 1;
  if (device_ids && capacity >= 1) device_ids[0] = c->rank;
  return nullptr;
}

const char* b200_topology_platform_name(const b200_client*) { return "b200"; }
const char* b200_topology_platform_version(const b200_client* c) { return c->version.c_str(); }
int b200_topology_num_devices(const b200_client* c) { return c->nprocs; }

b200_error* b200_topology_device_description(const b200_client* c, int index, int* id, int* process_index, const char** kind,
                                             const char** debug_string) {
  if (!c) return make_error(B200_INVALID_ARGUMENT, "null client");
  if (index < 0 || index >= c->nprocs) return make_error(B200_INVALID_ARGUMENT, "device index out of range");
  if (id) *id = index;
  if (process_index) *process_index = index;          // one process drives one device
  if (kind) *kind = c->kind.c_str();
  if (debug_string) {
    std::lock_guard<std::recursive_mutex> lock(const_cast<b200_client*>(c)->mu);
    auto& cache = const_cast<b200_client*>(c)->topology_strings;
    if ((int)cache.size() < c->nprocs) cache.resize(c->nprocs);
    if (cache[index].empty()) cache[index] = "B200:" + std::to_string(index) + (index == c->rank ? " (this process)" : " (process " + std::to_string(index) + ")");
    *debug_string = cache[index].c_str();
  }
  return nullptr;
}

uint64_t b200_topology_fingerprint(const b200_client* c) {
  const std::string text = std::string("b200|") + c->kind + "|" + std::to_string(c->nprocs);
  return hash_text(text.data(), text.size(), 0x42323030ull);
}

b200_error* b200_topology_serialize(const b200_client*, char**, size_t*) {
  return make_error(B200_UNIMPLEMENTED, "TopologyDescription_Serialize is not implemented");
}

b200_error* b200_client_default_device_assignment(const b200_client* c, int num_replicas, int num_partitions, int* assignment,
                                                  size_t assignment_size) {
  if (!c || !assignment) return make_error(B200_INVALID_ARGUMENT, "null argument");
  if (num_replicas < 1 || num_partitions < 1) return make_error(B200_INVALID_ARGUMENT, "replica and partition counts must be positive");
  const size_t n = (size_t)num_replicas * (size_t)num_partitions;
  if (assignment_size < n) return make_error(B200_INVALID_ARGUMENT, "assignment array is too small");
  if (n > (size_t)c->nprocs)
    return make_error(B200_INVALID_ARGUMENT, "the job has " + std::to_string(c->nprocs) + " devices, " + std::to_string(n) + " were asked for");
  for (size_t k = 0; k < n; k++) assignment[k] = (int)k;
  return nullptr;
}

namespace {
void put_varint(std::string& out, uint64_t v) {
  while (v >= 0x80) { out.push_back((char)((v & 0x7F) | 0x80)); v >>= 7; }
  out.push_back((char)v);
}
// xla.DeviceAssignmentProto by hand: 1 replica_count, 2 computation_count, 3 repeated ComputationDevice
// { 1 repeated int64 replica_device_ids (packed) }; proto3 leaves out scalars that are zero.
std::string encode_device_assignment(int replicas, int computations, const int64_t* ids) {
  std::string out;
  if (replicas) { out.push_back(0x08); put_varint(out, (uint64_t)replicas); }
  if (computations) { out.push_back(0x10); put_varint(out, (uint64_t)computations); }
  for (int cidx = 0; cidx < computations; cidx++) {
    std::string packed;
    for (int r = 0; r < replicas; r++) put_varint(packed, (uint64_t)ids[(size_t)cidx * replicas + r]);
    std::string msg;
    if (!packed.empty()) { msg.push_back(0x0A); put_varint(msg, packed.size()); msg += packed; }
    out.push_back(0x1A);
    put_varint(out, msg.size());
    out += msg;
  }
  return out;
}
b200_error* hand_out(const std::string& data, char** bytes, size_t* size) {
  char* p = (char*)malloc(std::max<size_t>(data.size(), 1));
  if (!p) return make_error(B200_RESOURCE_EXHAUSTED, "out of host memory");
  memcpy(p, data.data(), data.size());
  *bytes = p;
  *size = data.size();
  return nullptr;
}
}  // namespace

b200_error* b200_encode_device_assignment(int replica_count, int computation_count, const int64_t* device_ids, char** bytes,
                                          size_t* size) {
  if (!bytes || !size || (!device_ids && replica_count * computation_count > 0)) return make_error(B200_INVALID_ARGUMENT, "null argument");
  if (replica_count < 0 || computation_count < 0) return make_error(B200_INVALID_ARGUMENT, "negative count");
  return hand_out(encode_device_assignment(replica_count, computation_count, device_ids), bytes, size);
}

b200_error* b200_executable_device_assignment(const b200_executable* e, char** bytes, size_t* size) {
  if (!e || !bytes || !size) return make_error(B200_INVALID_ARGUMENT, "null argument");
  const int replicas = std::max(1, e->lp->prog->num_replicas);
  const int parts = std::max(1, e->client->nprocs > 1 ? e->client->nprocs : e->lp->prog->num_partitions);
  std::vector<int64_t> ids((size_t)replicas * parts);
  for (int p2 = 0; p2 < parts; p2++)
    for (int r = 0; r < replicas; r++) ids[(size_t)p2 * replicas + r] = (int64_t)p2 * replicas + r;
  if (parts == 1 && replicas == 1) ids[0] = e->client->rank;
  return hand_out(encode_device_assignment(replicas, parts, ids.data()), bytes, size);
}

b200_error* b200_executable_output_memory_kinds(const b200_executable* e, const char* const** kinds, const size_t** kind_sizes,
                                                size_t* num_outputs) {
  if (!e || !num_outputs) return make_error(B200_INVALID_ARGUMENT, "null argument");
  static const char* const kDevice = "device";
  std::lock_guard<std::recursive_mutex> lock(e->client->mu);
  auto& lp = *e->lp;
  const size_t n = lp.prog->results.size();
  if (lp.output_kinds.size() != n) {
    lp.output_kinds.assign(n, kDevice);
    lp.output_kind_sizes.assign(n, 6);
  }
  *num_outputs = n;
  if (kinds) *kinds = lp.output_kinds.data();
  if (kind_sizes) *kind_sizes = lp.output_kind_sizes.data();
  return nullptr;
}

// ---- several GPUs as the devices of one process ------------------------------------------------------------------
// PJRT_LoadedExecutable_Execute hands the plugin one argument list per addressable device
// (src/pjrt_plugin/pjrt_executable.cc:178-258 reads argument_lists[0] only: the reference has one device). A device
// group is that shape on this side: one client per local GPU, their NCCL communicators made together in this process
// (ncclCommInitAll), one executable per device compiled from the same module, and an execute call that takes
// per-device argument and output lists and returns one completion event per device. Each device's plan is issued
// by a thread of its own, so that the collectives of the plans meet the way they do between processes.
struct b200_device_group {
  std::vector<b200_client*> clients;
};

b200_error* b200_device_group_create(const int* ordinals, int num_devices, b200_device_group** out) {
  if (!out || num_devices < 1) return make_error(B200_INVALID_ARGUMENT, "a device group needs at least one device");
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();
    return make_error(B200_FAILED_PRECONDITION, "no CUDA device available (this plugin has no CPU fallback)");
  }
  std::vector<int> devs(num_devices);
  for (int d = 0; d < num_devices; d++) {
    devs[d] = ordinals ? ordinals[d] : d;
    if (devs[d] < 0 || devs[d] >= count) return make_error(B200_INVALID_ARGUMENT, "device ordinal " + std::to_string(devs[d]) + " out of range");
    for (int q = 0; q < d; q++) if (devs[q] == devs[d]) return make_error(B200_INVALID_ARGUMENT, "a device appears twice in the group");
  }
  std::vector<ncclComm_t> comms(num_devices, nullptr);
  if (num_devices > 1) {
    NcclApi& n = nccl();
    if (!n.ok) return make_error(B200_FAILED_PRECONDITION, n.error);
    ncclResult_t r = n.CommInitAll(comms.data(), num_devices, devs.data());
    if (r != ncclSuccess) return make_error(B200_INTERNAL, std::string("ncclCommInitAll: ") + n.GetErrorString(r));
  }
  auto g = std::make_unique<b200_device_group>();
  for (int d = 0; d < num_devices; d++) {
    b200_client_options o;
    memset(&o, 0, sizeof o);
    o.struct_size = sizeof o;
    o.device_ordinal = devs[d];
    o.process_index = d;
    o.num_processes = num_devices;
    b200_client* c = nullptr;
    if (auto* e = create_client(&o, comms[d], &c)) {
      for (auto* made : g->clients) b200_client_destroy(made);
      return e;
    }
    g->clients.push_back(c);
  }
  *out = g.release();
  return nullptr;
}

int b200_device_group_size(const b200_device_group* g) { return g ? (int)g->clients.size() : 0; }
b200_client* b200_device_group_client(const b200_device_group* g, int device) {
  return (g && device >= 0 && device < (int)g->clients.size()) ? g->clients[device] : nullptr;
}

b200_error* b200_device_group_destroy(b200_device_group* g) {
  if (!g) return nullptr;
  for (auto* c : g->clients) b200_client_destroy(c);
  delete g;
  return nullptr;
}

b200_error* b200_device_group_compile(b200_device_group* g, const char* code, size_t code_size, const char* format,
                                      const b200_compile_options* options, b200_executable** executables) {
  if (!g || !executables) return make_error(B200_INVALID_ARGUMENT, "null argument");
  const size_t n = g->clients.size();
  std::vector<b200_error*> errs(n, nullptr);
  std::vector<std::thread> threads;
  for (size_t d = 0; d < n; d++) {
    executables[d] = nullptr;
    threads.emplace_back([&, d] { errs[d] = b200_client_compile(g->clients[d], code, code_size, format, options, &executables[d]); });
  }
  for (auto& t : threads) t.join();
  b200_error* first = nullptr;
  for (size_t d = 0; d < n; d++) {
    if (!errs[d]) continue;
    if (!first) first = errs[d];
    else b200_error_destroy(errs[d]);
  }
  if (first)
    for (size_t d = 0; d < n; d++)
      if (executables[d]) { b200_executable_destroy(executables[d]); executables[d] = nullptr; }
  return first;
}

b200_error* b200_device_group_execute(b200_device_group* g, b200_executable* const* executables,
                                      b200_buffer* const* const* argument_lists, size_t num_args, b200_buffer** const* output_lists,
                                      b200_event** device_complete_events, const b200_execute_options* options) {
  if (!g || !executables || !output_lists || (num_args && !argument_lists)) return make_error(B200_INVALID_ARGUMENT, "null argument");
  const size_t n = g->clients.size();
  for (size_t d = 0; d < n; d++)
    if (!executables[d] || executables[d]->client != g->clients[d])
      return make_error(B200_INVALID_ARGUMENT, "executable " + std::to_string(d) + " does not belong to device " + std::to_string(d) + " of the group");
  std::vector<b200_error*> errs(n, nullptr);
  std::vector<std::thread> threads;
  for (size_t d = 0; d < n; d++)
    threads.emplace_back([&, d] {
      errs[d] = b200_executable_execute(executables[d], num_args ? argument_lists[d] : nullptr, num_args, output_lists[d],
                                        device_complete_events ? &device_complete_events[d] : nullptr, options);
    });
  for (auto& t : threads) t.join();
  b200_error* first = nullptr;
  for (size_t d = 0; d < n; d++) {
    if (!errs[d]) continue;
    if (!first) first = make_error(errs[d]->code, "device " + std::to_string(d) + ": " + errs[d]->message);
    b200_error_destroy(errs[d]);
  }
  return first;
}

b200_error* b200_client_debug_arm_wait_expiry(b200_client* c, int polls) {
  if (!c || polls <= 0) return make_error(B200_INVALID_ARGUMENT, "client and a positive poll budget are required");
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  c->armed_wait_polls = polls;
  return nullptr;
}

long long b200_client_host_syncs(const b200_client* c) { return c ? c->host_syncs : 0; }

b200_error* b200_client_probe_tf32_mma_rate(b200_client* c, double* tflops) {
  if (!c || !tflops) return make_error(B200_INVALID_ARGUMENT, "null argument");
  std::lock_guard<std::recursive_mutex> lock(c->mu);
  if (auto* e = set_device(c)) return e;
  cudaError_t e = b200::probe_tf32_mma_rate(c->error_flag, c->compute, tflops);
  if (e != cudaSuccess) return make_error(B200_INTERNAL, std::string("tensor-core rate probe failed: ") + cudaGetErrorString(e));
  return nullptr;
}

// profiler extension stub (pjrt_profiler.cc:17-125)
b200_error* b200_profiler_create(const char*, size_t, b200_profiler** profiler) {
  if (!profiler) return make_error(B200_INVALID_ARGUMENT, "null argument");
  *profiler = new b200_profiler();
  return nullptr;
}
b200_error* b200_profiler_start(b200_profiler* p) {
  if (!p) return make_error(B200_INVALID_ARGUMENT, "null profiler");
  if (p->running) return make_error(B200_FAILED_PRECONDITION, "profiler already started");
  p->running = true;
  return nullptr;
}
b200_error* b200_profiler_stop(b200_profiler* p) {
  if (!p) return make_error(B200_INVALID_ARGUMENT, "null profiler");
  if (!p->running) return make_error(B200_FAILED_PRECONDITION, "profiler was not started");
  p->running = false;
  return nullptr;
}
b200_error* b200_profiler_collect_data(b200_profiler* p, void*, size_t* size) {
  if (!p || !size) return make_error(B200_INVALID_ARGUMENT, "null argument");
  *size = 0;
  return nullptr;
}
b200_error* b200_profiler_destroy(b200_profiler* p) {
  delete p;
  return nullptr;
}

b200_error* b200_matmul_f32_static_scratch(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                                           void* cuda_stream) {
  if (!a || !b || !c) return make_error(B200_INVALID_ARGUMENT, "null operand pointer");
  // (the kernel rounds K up to whole chunks in 32-bit arithmetic: keep a margin below INT32_MAX)
  if (m <= 0 || n <= 0 || k <= 0 || m > INT32_MAX || n > INT32_MAX || k > INT32_MAX - 4096 || m * k > INT32_MAX * 64ll ||
      k * n > INT32_MAX * 64ll)
    return make_error(B200_INVALID_ARGUMENT, "matrix extents must be positive and fit the kernel's index range");
  const char* why = nullptr;
  cudaError_t e = b200::matmul_f32_static_scratch(a, b, c, (int)m, (int)n, (int)k, (cudaStream_t)cuda_stream, &why);
  if (e == cudaSuccess) return nullptr;
  std::string msg = why ? why : cudaGetErrorString(e);
  if (e == cudaErrorInvalidValue && why)
    return make_error(B200_INVALID_ARGUMENT, msg + " (m=" + std::to_string(m) + ", n=" + std::to_string(n) + ", limit " +
                                                 std::to_string(b200::static_scratch_bytes()) + " bytes)");
  return make_error(B200_INTERNAL, "static-scratch product failed: " + msg);
}

}  // extern "C"

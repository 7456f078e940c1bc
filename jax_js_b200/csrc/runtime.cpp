// libjaxcuda.so runtime: contexts, ref-counted slots over a caching device allocator, the
// NVRTC kernel cache, dispatch, readback, event timing and the NCCL gradient sum.
//
// Shape of the reference it stands behind: the slot map and allocator of the Wasm backend
// (src/backend/wasm.ts:57-123, src/backend/wasm/allocator.ts:73-90), the buffer pool and
// pipeline cache of the WebGPU backend (src/backend/webgpu.ts:224-247, :655-760), and the
// dispatch-order guarantee of the interface (src/backend.ts:203-210) -- here one CUDA stream.
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nvrtc.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../include/jaxcuda.h"
#include "emit.hpp"
#include "gemm_tc.hpp"
#include "ir.hpp"
#include "scatter.hpp"
#include "linalg.hpp"
#include "fft.hpp"

#include <sstream>
#include <unordered_set>

extern "C" size_t jaxcuda_sort_work_bytes(int argsort, int dtype, int64_t batch, int64_t n);
extern "C" int jaxcuda_sort_launch(void* stream, int argsort, const void* x, void* y, int32_t* yi, int dtype,
                                   int64_t batch, int64_t n, void* work, int* launches);

using namespace jaxcuda;

namespace jaxcuda_rt {

std::string g_create_error;

struct Driver {
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                           CUstream, void**, void**) = nullptr;
  CUresult (*LaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;   // optional: cluster launches
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  void* TensorMapEncodeTiled = nullptr;
  bool loaded = false;
};

bool load_driver(Driver& d, std::string& err) {
  auto get = [&](const char* name, void** fn) {
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !*fn) {
      err = std::string("driver entry point ") + name + " unavailable";
      return false;
    }
    return true;
  };
  if (!get("cuModuleLoadData", (void**)&d.ModuleLoadData)) return false;
  if (!get("cuModuleUnload", (void**)&d.ModuleUnload)) return false;
  if (!get("cuModuleGetFunction", (void**)&d.ModuleGetFunction)) return false;
  if (!get("cuLaunchKernel", (void**)&d.LaunchKernel)) return false;
  if (!get("cuFuncSetAttribute", (void**)&d.FuncSetAttribute)) return false;
  if (!get("cuGetErrorString", (void**)&d.GetErrorString)) return false;
  if (!get("cuTensorMapEncodeTiled", &d.TensorMapEncodeTiled)) return false;
  {
    std::string ignored;
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuLaunchKernelEx", &fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      d.LaunchKernelEx = (CUresult (*)(const CUlaunchConfig*, CUfunction, void**, void**))fn;
  }
  d.loaded = true;
  return true;
}

// Size-class caching allocator.  Everything a context does is ordered on one stream, so a
// block returned to the free list may be handed out again at once: any kernel that still
// reads it was enqueued before whatever the next owner enqueues.
struct Allocator {
  std::map<size_t, std::vector<void*>> free_lists;
  size_t reserved = 0, in_use = 0;
  // Blocks that a captured graph has baked into its kernel parameters belong to that graph until
  // it is destroyed: `owner` maps such a block to its graph, `idle` holds the owned blocks that no
  // slot is using at the moment.  While `capturing` is non-zero every block that is handed out or
  // handed back is adopted by the graph being captured, and reuse happens among adopted blocks only.
  std::unordered_map<void*, int> owner;
  std::unordered_map<int, std::map<size_t, std::vector<void*>>> idle;
  int capturing = 0;

  static size_t round_size(size_t n) {
    if (n <= 512) return 512;
    size_t p = 512;
    while (p < n) p <<= 1;
    const size_t step = p >> 3;  // eight classes per octave: at most 12.5 % slack
    return (n + step - 1) / step * step;
  }
  cudaError_t get(size_t n, void** out) {
    const size_t cls = round_size(n);
    if (capturing) {
      auto& mine = idle[capturing][cls];
      if (!mine.empty()) {
        *out = mine.back();
        mine.pop_back();
        in_use += cls;
        return cudaSuccess;
      }
    }
    auto it = free_lists.find(cls);
    if (it != free_lists.end() && !it->second.empty()) {
      *out = it->second.back();
      it->second.pop_back();
      in_use += cls;
      if (capturing) owner[*out] = capturing;
      return cudaSuccess;
    }
    cudaError_t e = cudaMalloc(out, cls);
    if (e != cudaSuccess) {  // give cached blocks back to the driver and retry once
      cudaGetLastError();
      release_cached();
      e = cudaMalloc(out, cls);
    }
    if (e == cudaSuccess) {
      reserved += cls;
      in_use += cls;
      if (capturing) owner[*out] = capturing;
    }
    return e;
  }
  void put(void* p, size_t n) {
    const size_t cls = round_size(n);
    in_use -= cls;
    if (capturing) owner[p] = capturing;  // a block released inside a capture may be reused by it: adopt it
    auto it = owner.find(p);
    if (it != owner.end()) idle[it->second][cls].push_back(p);
    else free_lists[cls].push_back(p);
  }
  // The graph is gone: its idle blocks return to the pool, its blocks still behind live slots
  // become ordinary blocks.
  void release_graph(int id) {
    for (auto& kv : idle[id])
      for (void* p : kv.second) free_lists[kv.first].push_back(p);
    idle.erase(id);
    for (auto it = owner.begin(); it != owner.end();) it = (it->second == id) ? owner.erase(it) : std::next(it);
  }
  void release_cached() {
    for (auto& kv : free_lists) {
      for (void* p : kv.second) { cudaFree(p); reserved -= kv.first; }
      kv.second.clear();
    }
  }
};

struct SlotRec {
  void* ptr = nullptr;
  size_t bytes = 0;
  int refs = 0;
  uint64_t read_ticket = 0;  // last asynchronous read of this slot (a later upload into it waits for that read)
};

}  // namespace jaxcuda_rt
using namespace jaxcuda_rt;

struct jaxcuda_exe {
  jaxcuda_ctx* ctx = nullptr;
  int kind = 0;  // 0 kernel, 1 Sort, 2 Argsort, 3 Scatter
  jaxcuda_scatter_desc scatter = {};
  int handles = 0;
  uint64_t hash = 0;
  KernelIR ir;
  Plan plan;
  CUmodule module = nullptr;
  std::vector<CUfunction> fns;
  // routine
  int rt_dtype = 0;
  int64_t rt_batch = 0, rt_n = 0;
  int64_t rt_m = 0, rt_rows = 0;  // linalg routines: rows of a rectangular matrix; right-hand sides per matrix
  int rt_flag = 0;                // TriangularSolve: unitDiagonal; JacobiEigh: maxSweeps; Fft: inverse
  double rt_tolerance = 0.0;      // JacobiEigh
  std::vector<int> rt_factors;    // Fft
  std::string describe;
  void* persistent_scratch = nullptr;  // zero-initialised once; reused by every dispatch (stream-ordered)
  std::vector<int> fuse_params;        // row program: buffer (of the group's table) behind each pointer parameter
};

struct jaxcuda_graph {
  jaxcuda_ctx* ctx = nullptr;
  int id = 0;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t kernels = 0;  // kernel launches recorded in the graph
  double algo_bytes = 0;  // algorithmic bytes of those launches (a fused kernel counts what it reads and writes itself)
  int fused_groups = 0;
};

// A Kernel dispatched inside a capture is not launched at once: the list is kept until something
// other than a Kernel needs the stream (or the capture ends), so that runs of Kernels over the rows
// of one array can be replaced by one row-resident kernel (emit.hpp, plan_row_fusion).
struct PendingDispatch {
  jaxcuda_exe* exe = nullptr;
  std::vector<void*> in;
  std::vector<size_t> in_bytes;
  void* out = nullptr;
  size_t out_bytes = 0;
  bool out_freed = false;  // the output's slot was released before the list was flushed: nobody else can read it
  size_t freed_at = (size_t)-1;  // ... after this many dispatches of the list (later users of the address see another array)
  LoPlanes lo;             // 3xTF32 GEMMs: remainder planes kept across the GEMMs of the list (see plane_ticket)
};

struct jaxcuda_ctx {
  int device = 0;
  int next_graph_id = 1;
  uint64_t capture_launches0 = 0;
  std::vector<PendingDispatch> pending;
  bool fuse_rows = true;          // JAXCUDA_FUSE=0: captured Kernels are launched one by one
  // Remainder planes lo = x - tf32(x) of arrays that 3xTF32 GEMMs of the step list being captured
  // read, by the array's address: an activation is the operand of a forward GEMM and of a
  // weight-gradient GEMM, a weight of a forward and a backward one, and is split once.  Entries are
  // made and dropped in program order (at dispatch, at the release or overwrite of the array), the
  // order in which the deferred launches then happen.
  struct LoPlane { void* plane; size_t bytes; uint64_t len; };
  std::unordered_map<void*, LoPlane> lo_planes;
  bool keep_lo_planes = true;     // JAXCUDA_TC_PLANE_CACHE=0: every GEMM splits its own operands
  double capture_bytes = 0;
  int capture_groups = 0;
  std::map<std::string, std::unique_ptr<jaxcuda_exe>> fused;  // compiled row programs by wiring
  cudaStream_t stream = nullptr;
  Driver drv;
  Allocator alloc;
  std::unordered_map<uint32_t, SlotRec> slots;
  uint32_t next_slot = 1;
  std::unordered_map<uint64_t, std::unique_ptr<jaxcuda_exe>> kernels;
  std::vector<std::unique_ptr<jaxcuda_exe>> routines;
  std::string last_error;
  Options opt;
  std::vector<cudaEvent_t> events;  // created on first use of an index
  uint64_t launches = 0;
  int debug = 0;
  // Kernels whose bounded waits give up write a code to `status_dev` (device memory: every CTA
  // polls it, which must not cross PCIe); it is copied to the pinned `status_host` before a sync.
  int* status_host = nullptr;
  int* status_dev = nullptr;
  unsigned* oob_dev = nullptr;   // checked build: the two counters of jx_ix
  bool tc_dispatched = false;
  // NCCL (resolved with dlopen so that the library loads where NCCL is absent)
  void* nccl_lib = nullptr;
  void* comm = nullptr;
  int nranks = 1;
  // second stream for sums that run under later kernels (jaxcuda_allreduce_sum_f32_async)
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t comm_fork = nullptr, comm_done = nullptr;
  cudaEvent_t wait_compute = nullptr, wait_comm = nullptr;   // jaxcuda_comm_wait's probes
  // Tracing: while it is on, every eager dispatch is bracketed by a pair of timing events.
  struct TraceRec { jaxcuda_exe* exe; std::string name; cudaEvent_t begin, end; };
  bool tracing = false;
  cudaEvent_t trace_origin = nullptr;
  std::vector<TraceRec> trace;
  std::vector<cudaEvent_t> trace_events;   // pool, reused by the next trace
  size_t trace_events_used = 0;
  bool comm_pending = false;
  // copy streams of the asynchronous read / write calls, so that uploads, kernels and downloads of
  // consecutive steps overlap (the GPU has separate copy engines per direction)
  cudaStream_t up_stream = nullptr, down_stream = nullptr;
  cudaEvent_t copy_fork = nullptr, up_done = nullptr;
  std::vector<cudaEvent_t> tickets;  // ticket t = tickets[t - 1]
  std::vector<uint64_t> free_tickets;
  std::vector<char> ticket_pending;  // read_async issued, read_wait not yet returned
  std::unordered_set<void*> comm_ptrs;  // blocks a sum on the second stream is still working on
  // ... and, per block, the event behind the sum that works on it: a Kernel that reads the block makes
  // the compute stream wait for exactly that sum (not for those begun after it)
  std::unordered_map<void*, cudaEvent_t> comm_ptr_event;
  std::vector<cudaEvent_t> comm_events;   // pool; the first comm_events_used are taken
  size_t comm_events_used = 0;
  uint64_t order_waits = 0;          // times the compute stream was made to wait for a copy or a sum (see order_after_users)
  // direction of the next streaming kernel's walk over its grid (JAXCUDA_SWEEP=0: always forward)
  int sweep = 0;
  bool sweep_alternate = true;
  // SMs a persistent GEMM leaves free while such a sum is in flight (JAXCUDA_COMM_SMS).  Off by default:
  // on 8 GPUs 8 SMs changed nothing and 24 or 32 cost more GEMM time than the sum took.
  int comm_sms = 0;
};

namespace {

int fail(jaxcuda_ctx* ctx, int status, const char* fmt, ...) {
  char buf[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->last_error = buf; else g_create_error = buf;
  return status;
}

#define CUDA_TRY(ctx, call)                                                                        \
  do {                                                                                             \
    cudaError_t e__ = (call);                                                                      \
    if (e__ != cudaSuccess) return fail(ctx, JAXCUDA_ECUDA, "%s: %s", #call, cudaGetErrorString(e__)); \
  } while (0)

int drv_fail(jaxcuda_ctx* ctx, const char* what, CUresult r) {
  const char* s = nullptr;
  if (ctx->drv.GetErrorString) ctx->drv.GetErrorString(r, &s);
  return fail(ctx, JAXCUDA_ECUDA, "%s: %s", what, s ? s : "unknown driver error");
}

SlotRec* find_slot(jaxcuda_ctx* ctx, jaxcuda_slot s) {
  auto it = ctx->slots.find(s);
  return it == ctx->slots.end() ? nullptr : &it->second;
}

int slot_error(jaxcuda_ctx* ctx, jaxcuda_slot s) {
  // wording of SlotError, src/backend.ts:222-226
  return fail(ctx, JAXCUDA_ESLOT, "Used a buffer that is invalid or already freed: %u", s);
}

// The caching allocator hands a released block out again at once, and a write or a dispatch may
// target a slot directly; both are ordered on the compute stream only.  A download on the copy
// stream or a sum on the second stream that still uses the block is not, so before the block
// changes hands (or is written) the compute stream is made to wait for them.
int order_after_users(jaxcuda_ctx* ctx, SlotRec* s) {
  if (s->read_ticket && s->read_ticket <= ctx->ticket_pending.size() && ctx->ticket_pending[s->read_ticket - 1]) {
    CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->tickets[s->read_ticket - 1], 0));
    ctx->order_waits++;
    s->read_ticket = 0;
  }
  if (ctx->comm_pending && s->ptr && ctx->comm_ptrs.count(s->ptr)) {
    ctx->order_waits++;
    return jaxcuda_comm_join(ctx);
  }
  return JAXCUDA_OK;
}

// After a stream sync: has a kernel abandoned a bounded wait?
int check_device_status(jaxcuda_ctx* ctx) {
  if (ctx->status_host && *ctx->status_host != 0) {
    const int code = *ctx->status_host;
    *ctx->status_host = 0;
    cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), ctx->stream);
    return fail(ctx, JAXCUDA_ECUDA, "tcgen05 GEMM pipeline wait timed out (role %d: 1 producer, 2/3 mma, 4 epilogue, 5 patch gatherer, 6 remainder tiles); "
                "results of that dispatch are invalid", code);
  }
  return JAXCUDA_OK;
}

uint64_t fnv1a(const uint8_t* p, size_t n) {
  uint64_t h = 0xcbf29ce484222325ull;
  for (size_t i = 0; i < n; i++) h = (h ^ p[i]) * 0x100000001b3ull;
  return h;
}

// NVRTC: CUDA C -> sm_100a cubin.  Needs no GPU.
bool nvrtc_compile(const std::string& src_in, std::vector<char>& cubin, std::string& err, const void* oob_words = nullptr) {
  nvrtcProgram prog;
  std::string src = src_in;
  if (emit_checked()) {   // the checked build's counters live at a fixed device address of the context
    char head[96];
    snprintf(head, sizeof head, "#define JX_CHECKED 1\n#define JX_OOB_ADDR 0x%llxull\n", (unsigned long long)(uintptr_t)oob_words);
    src = head + src;
  }
  if (nvrtcCreateProgram(&prog, src.c_str(), "jaxcuda_kernel.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS) {
    err = "nvrtcCreateProgram failed";
    return false;
  }
  const char* opts[] = {"--gpu-architecture=sm_100a", "-std=c++17", "-lineinfo", "--fmad=true"};
  nvrtcResult r = nvrtcCompileProgram(prog, 4, opts);
  if (r != NVRTC_SUCCESS) {
    size_t n = 0;
    nvrtcGetProgramLogSize(prog, &n);
    std::string log(n, '\0');
    nvrtcGetProgramLog(prog, &log[0]);
    nvrtcDestroyProgram(&prog);
    err = "NVRTC: " + log + "\n---- generated source ----\n" + src;
    return false;
  }
  size_t n = 0;
  nvrtcGetCUBINSize(prog, &n);
  cubin.resize(n);
  nvrtcGetCUBIN(prog, cubin.data());
  nvrtcDestroyProgram(&prog);
  return true;
}

int compile_plan(jaxcuda_ctx* ctx, jaxcuda_exe* exe) {
  std::vector<char> cubin;
  if (!nvrtc_compile(exe->plan.source, cubin, ctx->last_error, ctx->oob_dev)) return JAXCUDA_ECOMPILE;
  CUresult cr = ctx->drv.ModuleLoadData(&exe->module, cubin.data());
  if (cr != CUDA_SUCCESS) return drv_fail(ctx, "cuModuleLoadData", cr);
  for (const Stage& st : exe->plan.stages) {
    CUfunction fn;
    cr = ctx->drv.ModuleGetFunction(&fn, exe->module, st.entry.c_str());
    if (cr != CUDA_SUCCESS) return drv_fail(ctx, "cuModuleGetFunction", cr);
    if (st.smem > 48 * 1024) {
      cr = ctx->drv.FuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)st.smem);
      if (cr != CUDA_SUCCESS) return drv_fail(ctx, "cuFuncSetAttribute", cr);
    }
    exe->fns.push_back(fn);
  }
  return JAXCUDA_OK;
}

void free_exe(jaxcuda_ctx* ctx, jaxcuda_exe* exe) {
  if (exe->persistent_scratch) ctx->alloc.put(exe->persistent_scratch, exe->plan.scratch_bytes);
  exe->persistent_scratch = nullptr;
  if (exe->module && ctx->drv.ModuleUnload) ctx->drv.ModuleUnload(exe->module);
  exe->module = nullptr;
}

int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : dflt;
}

}  // namespace

static int launch_kernel(jaxcuda_ctx* ctx, jaxcuda_exe* exe, const std::vector<void*>& inptr, void* outptr, const LoPlanes* lo = nullptr);
static int flush_pending(jaxcuda_ctx* ctx);

// A dispatch is about to read `s`: if a sum on the second stream still works on it, everything
// dispatched from here on waits for that sum.
static int order_after_sum(jaxcuda_ctx* ctx, SlotRec* s) {
  if (!ctx->comm_pending || !s->ptr) return JAXCUDA_OK;
  auto it = ctx->comm_ptr_event.find(s->ptr);
  if (it == ctx->comm_ptr_event.end()) return JAXCUDA_OK;
  if (int rc = flush_pending(ctx)) return rc;
  CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, it->second, 0));
  ctx->order_waits++;
  // sums complete in the order they were begun: every block of this sum and of earlier ones is settled
  const cudaEvent_t waited = it->second;
  size_t upto = 0;
  while (upto < ctx->comm_events_used && ctx->comm_events[upto] != waited) upto++;
  for (auto e = ctx->comm_ptr_event.begin(); e != ctx->comm_ptr_event.end();) {
    size_t at = 0;
    while (at < ctx->comm_events_used && ctx->comm_events[at] != e->second) at++;
    if (at <= upto) { ctx->comm_ptrs.erase(e->first); e = ctx->comm_ptr_event.erase(e); }
    else ++e;
  }
  return JAXCUDA_OK;
}



extern "C" {

int jaxcuda_max_args(void) { return 64; }

const char* jaxcuda_last_error(jaxcuda_ctx* ctx) { return ctx ? ctx->last_error.c_str() : g_create_error.c_str(); }

int jaxcuda_create(int device, jaxcuda_ctx** out) {
  if (!out) return fail(nullptr, JAXCUDA_EINVAL, "null out pointer");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(nullptr, JAXCUDA_ECUDA, "no CUDA device available (%s); the cuda backend has no CPU fallback",
                e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
  if (device < 0) device = env_int("JAXCUDA_DEVICE", 0);
  if (device >= count) return fail(nullptr, JAXCUDA_EINVAL, "device %d out of range (%d devices)", device, count);
  std::unique_ptr<jaxcuda_ctx> ctx(new jaxcuda_ctx);
  ctx->device = device;
  if ((e = cudaSetDevice(device)) != cudaSuccess || (e = cudaFree(0)) != cudaSuccess)
    return fail(nullptr, JAXCUDA_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
  cudaDeviceProp prop;
  if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess)
    return fail(nullptr, JAXCUDA_ECUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return fail(nullptr, JAXCUDA_ECUDA, "device %d is sm_%d%d; this backend is built for sm_100a only", device,
                prop.major, prop.minor);
  std::string err;
  if (!load_driver(ctx->drv, err)) return fail(nullptr, JAXCUDA_ECUDA, "%s", err.c_str());
  if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail(nullptr, JAXCUDA_ECUDA, "cudaStreamCreate: %s", cudaGetErrorString(e));
  if ((e = cudaHostAlloc((void**)&ctx->status_host, sizeof(int), cudaHostAllocDefault)) != cudaSuccess ||
      (e = cudaMalloc((void**)&ctx->status_dev, sizeof(int))) != cudaSuccess ||
      (e = cudaMemset(ctx->status_dev, 0, sizeof(int))) != cudaSuccess)
    return fail(nullptr, JAXCUDA_ECUDA, "status word: %s", cudaGetErrorString(e));
  *ctx->status_host = 0;
  if (emit_checked() && ((e = cudaMalloc((void**)&ctx->oob_dev, 2 * sizeof(unsigned))) != cudaSuccess ||
                         (e = cudaMemset(ctx->oob_dev, 0, 2 * sizeof(unsigned))) != cudaSuccess))
    return fail(nullptr, JAXCUDA_ECUDA, "checked build counters: %s", cudaGetErrorString(e));
  ctx->opt.sm_count = prop.multiProcessorCount;
  ctx->opt.ew_ilp = env_int("JAXCUDA_EW_ILP", ctx->opt.ew_ilp);
  ctx->opt.ew_blocks_per_sm = env_int("JAXCUDA_EW_BLOCKS_PER_SM", ctx->opt.ew_blocks_per_sm);
  ctx->opt.allow_tc = env_int("JAXCUDA_NO_TC", 0) == 0;
  ctx->opt.force_skeleton = env_int("JAXCUDA_FORCE_SKELETON", -1);
  ctx->opt.exact_math = env_int("JAXCUDA_EXACT_MATH", ctx->opt.exact_math);
  ctx->opt.ld_hint = env_int("JAXCUDA_LD_HINT", ctx->opt.ld_hint);
  ctx->opt.conv_implicit = env_int("JAXCUDA_CONV_IMPLICIT", ctx->opt.conv_implicit);
  ctx->opt.tc_lo_in_kernel = env_int("JAXCUDA_TC_LO_IN_KERNEL", ctx->opt.tc_lo_in_kernel);
  ctx->opt.tc_half_last = env_int("JAXCUDA_TC_HALF_LAST", ctx->opt.tc_half_last);
  ctx->opt.tc_pair = ctx->drv.LaunchKernelEx ? env_int("JAXCUDA_TC_PAIR", ctx->opt.tc_pair) : 0;
  ctx->opt.row_tpr = env_int("JAXCUDA_ROW_TPR", ctx->opt.row_tpr);
  ctx->opt.row_unroll = env_int("JAXCUDA_ROW_UNROLL", ctx->opt.row_unroll);
  ctx->opt.col_threads = env_int("JAXCUDA_COL_THREADS", ctx->opt.col_threads);
  ctx->opt.col_ctas_per_sm = env_int("JAXCUDA_COL_CTAS_PER_SM", ctx->opt.col_ctas_per_sm);
  ctx->opt.col_ty = env_int("JAXCUDA_COL_TY", ctx->opt.col_ty);
  ctx->opt.col_unroll = env_int("JAXCUDA_COL_UNROLL", ctx->opt.col_unroll);
  ctx->comm_sms = env_int("JAXCUDA_COMM_SMS", ctx->comm_sms);
  ctx->opt.tc_bn = env_int("JAXCUDA_TC_BN", 0);
  ctx->opt.tc_streamk = env_int("JAXCUDA_TC_STREAMK", ctx->opt.tc_streamk);
  ctx->opt.tc_spin_limit = env_int("JAXCUDA_TC_SPIN_LIMIT", ctx->opt.tc_spin_limit);
  ctx->opt.tc_fault = env_int("JAXCUDA_TC_FAULT", 0);
  ctx->sweep_alternate = env_int("JAXCUDA_SWEEP", 1) != 0;
  ctx->fuse_rows = env_int("JAXCUDA_FUSE", 1) != 0;
  ctx->keep_lo_planes = env_int("JAXCUDA_TC_PLANE_CACHE", 1) != 0;
  ctx->opt.fuse_chunks = env_int("JAXCUDA_FUSE_CHUNKS", ctx->opt.fuse_chunks);
  ctx->opt.fuse_min_ctas = env_int("JAXCUDA_FUSE_MIN_CTAS", ctx->opt.fuse_min_ctas);
  ctx->debug = env_int("JAXCUDA_DEBUG", 0);
  *out = ctx.release();
  return JAXCUDA_OK;
}

int jaxcuda_destroy(jaxcuda_ctx* ctx) {
  if (!ctx) return JAXCUDA_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->up_stream) {
    cudaStreamSynchronize(ctx->up_stream);
    cudaStreamSynchronize(ctx->down_stream);
    for (cudaEvent_t ev : ctx->tickets) cudaEventDestroy(ev);
    cudaEventDestroy(ctx->copy_fork);
    cudaEventDestroy(ctx->up_done);
    cudaStreamDestroy(ctx->up_stream);
    cudaStreamDestroy(ctx->down_stream);
  }
  if (ctx->comm_stream) {
    cudaStreamSynchronize(ctx->comm_stream);
    cudaEventDestroy(ctx->comm_fork);
    cudaEventDestroy(ctx->comm_done);
    for (cudaEvent_t ev : ctx->comm_events) cudaEventDestroy(ev);
    cudaStreamDestroy(ctx->comm_stream);
  }
  for (cudaEvent_t ev : ctx->trace_events) cudaEventDestroy(ev);
  if (ctx->trace_origin) cudaEventDestroy(ctx->trace_origin);
  if (ctx->wait_compute) cudaEventDestroy(ctx->wait_compute);
  if (ctx->wait_comm) cudaEventDestroy(ctx->wait_comm);
  jaxcuda_comm_destroy(ctx);
  for (auto& kv : ctx->kernels) free_exe(ctx, kv.second.get());
  for (auto& ev : ctx->events) if (ev) cudaEventDestroy(ev);
  for (auto& kv : ctx->slots) if (kv.second.ptr) ctx->alloc.put(kv.second.ptr, kv.second.bytes);
  ctx->alloc.release_cached();
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  if (ctx->status_dev) cudaFree(ctx->status_dev);
  if (ctx->oob_dev) cudaFree(ctx->oob_dev);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return JAXCUDA_OK;
}

int jaxcuda_malloc(jaxcuda_ctx* ctx, size_t bytes, const void* init, size_t init_bytes, jaxcuda_slot* out) {
  if (!ctx || !out) return JAXCUDA_EINVAL;
  if (init && init_bytes != bytes)
    return fail(ctx, JAXCUDA_EINVAL, "initialData size %zu does not match buffer size %zu", init_bytes, bytes);
  if (init && ctx->alloc.capturing)
    return fail(ctx, JAXCUDA_EINVAL, "malloc with initialData inside a capture: upload before jaxcuda_capture_begin");
  cudaSetDevice(ctx->device);
  SlotRec rec;
  rec.bytes = bytes;
  rec.refs = 1;
  if (bytes) {
    cudaError_t e = ctx->alloc.get(bytes, &rec.ptr);
    if (e != cudaSuccess) return fail(ctx, JAXCUDA_ENOMEM, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    if (init) {
      e = cudaMemcpyAsync(rec.ptr, init, bytes, cudaMemcpyHostToDevice, ctx->stream);
      // The caller may reuse `init` as soon as malloc returns (it is a JS typed array).
      if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
      if (e != cudaSuccess) {
        ctx->alloc.put(rec.ptr, bytes);
        return fail(ctx, JAXCUDA_ECUDA, "upload failed: %s", cudaGetErrorString(e));
      }
    }
  }
  const jaxcuda_slot id = ctx->next_slot++;
  ctx->slots[id] = rec;
  *out = id;
  return JAXCUDA_OK;
}

// The array at `ptr` is about to change or to go away: its remainder plane is of no use any more.
static void drop_lo_plane(jaxcuda_ctx* ctx, void* ptr) {
  if (ctx->lo_planes.empty()) return;
  auto it = ctx->lo_planes.find(ptr);
  if (it == ctx->lo_planes.end()) return;
  ctx->alloc.put(it->second.plane, it->second.bytes);
  ctx->lo_planes.erase(it);
}
static void drop_all_lo_planes(jaxcuda_ctx* ctx) {
  for (auto& kv : ctx->lo_planes) ctx->alloc.put(kv.second.plane, kv.second.bytes);
  ctx->lo_planes.clear();
}
// The plane of the operand at `ptr` (`len` elements): the one an earlier GEMM of the list made, or a
// new one that this GEMM fills.
static int plane_ticket(jaxcuda_ctx* ctx, void* ptr, uint64_t len, float*& plane, bool& compute) {
  auto it = ctx->lo_planes.find(ptr);
  if (it != ctx->lo_planes.end() && it->second.len == len) { plane = (float*)it->second.plane; compute = false; return JAXCUDA_OK; }
  if (it != ctx->lo_planes.end()) drop_lo_plane(ctx, ptr);
  const size_t bytes = (size_t)((len + 63) / 64 * 64) * 4;
  void* p = nullptr;
  cudaError_t e = ctx->alloc.get(bytes, &p);
  if (e != cudaSuccess) return fail(ctx, JAXCUDA_ENOMEM, "remainder plane of %zu bytes: %s", bytes, cudaGetErrorString(e));
  ctx->lo_planes[ptr] = jaxcuda_ctx::LoPlane{p, bytes, len};
  plane = (float*)p;
  compute = true;
  return JAXCUDA_OK;
}

int jaxcuda_incref(jaxcuda_ctx* ctx, jaxcuda_slot slot) {
  SlotRec* s = find_slot(ctx, slot);
  if (!s) return slot_error(ctx, slot);
  s->refs++;
  return JAXCUDA_OK;
}

int jaxcuda_decref(jaxcuda_ctx* ctx, jaxcuda_slot slot) {
  SlotRec* s = find_slot(ctx, slot);
  if (!s) return slot_error(ctx, slot);
  if (--s->refs == 0) {
    if (int rc = order_after_users(ctx, s)) return rc;
    for (size_t i = ctx->pending.size(); i-- > 0;)   // the latest pending writer of this block produced it
      if (ctx->pending[i].out == s->ptr) { ctx->pending[i].out_freed = true; ctx->pending[i].freed_at = ctx->pending.size(); break; }
    if (s->ptr) { drop_lo_plane(ctx, s->ptr); ctx->alloc.put(s->ptr, s->bytes); }
    ctx->slots.erase(slot);
  }
  return JAXCUDA_OK;
}

int jaxcuda_slot_size(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t* bytes) {
  SlotRec* s = find_slot(ctx, slot);
  if (!s) return slot_error(ctx, slot);
  *bytes = s->bytes;
  return JAXCUDA_OK;
}

int jaxcuda_read(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t start, size_t count, void* dst) {
  SlotRec* s = find_slot(ctx, slot);
  if (!s) return slot_error(ctx, slot);
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "read inside a capture: reads synchronise the stream");
  if (start > s->bytes) return fail(ctx, JAXCUDA_EINVAL, "read start %zu beyond buffer of %zu bytes", start, s->bytes);
  if (count == SIZE_MAX) count = s->bytes - start;
  if (count > s->bytes - start) return fail(ctx, JAXCUDA_EINVAL, "read of %zu bytes at %zu beyond buffer of %zu bytes", count, start, s->bytes);
  cudaSetDevice(ctx->device);
  if (int rc = jaxcuda_comm_join(ctx)) return rc;
  if (count) {
    if (!dst) return fail(ctx, JAXCUDA_EINVAL, "null destination");
    CUDA_TRY(ctx, cudaMemcpyAsync(dst, (const char*)s->ptr + start, count, cudaMemcpyDeviceToHost, ctx->stream));
  }
  if (ctx->tc_dispatched) {  // only contexts that ran the tensor-core skeleton have anything to report
    CUDA_TRY(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    ctx->tc_dispatched = false;
  }
  CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  return check_device_status(ctx);
}

int jaxcuda_write(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t start, size_t count, const void* src) {
  SlotRec* s = find_slot(ctx, slot);
  if (!s) return slot_error(ctx, slot);
  if (start > s->bytes || count > s->bytes - start)
    return fail(ctx, JAXCUDA_EINVAL, "write of %zu bytes at %zu beyond buffer of %zu bytes", count, start, s->bytes);
  cudaSetDevice(ctx->device);
  if (int rc = flush_pending(ctx)) return rc;
  if (int rc = order_after_users(ctx, s)) return rc;
  drop_lo_plane(ctx, s->ptr);
  if (count) CUDA_TRY(ctx, cudaMemcpyAsync((char*)s->ptr + start, src, count, cudaMemcpyHostToDevice, ctx->stream));
  return JAXCUDA_OK;
}

static int copy_streams(jaxcuda_ctx* ctx) {
  if (ctx->up_stream) return JAXCUDA_OK;
  CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->up_stream, cudaStreamNonBlocking));
  CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->down_stream, cudaStreamNonBlocking));
  CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->copy_fork, cudaEventDisableTiming));
  CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->up_done, cudaEventDisableTiming));
  return JAXCUDA_OK;
}

int jaxcuda_write_async(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t start, size_t count, const void* src) {
  SlotRec* s = find_slot(ctx, slot);
  if (!s) return slot_error(ctx, slot);
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "write_async inside a capture");
  if (start > s->bytes || count > s->bytes - start)
    return fail(ctx, JAXCUDA_EINVAL, "write of %zu bytes at %zu beyond buffer of %zu bytes", count, start, s->bytes);
  cudaSetDevice(ctx->device);
  if (!count) return JAXCUDA_OK;
  if (int rc = copy_streams(ctx)) return rc;
  // after everything dispatched so far (earlier kernels may still read the slot) ...
  CUDA_TRY(ctx, cudaEventRecord(ctx->copy_fork, ctx->stream));
  CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->up_stream, ctx->copy_fork, 0));
  if (s->read_ticket)  // ... and after a download of this very slot that may still be in flight
    CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->up_stream, ctx->tickets[s->read_ticket - 1], 0));
  CUDA_TRY(ctx, cudaMemcpyAsync((char*)s->ptr + start, src, count, cudaMemcpyHostToDevice, ctx->up_stream));
  // ... and before everything dispatched from now on
  CUDA_TRY(ctx, cudaEventRecord(ctx->up_done, ctx->up_stream));
  CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->up_done, 0));
  return JAXCUDA_OK;
}

int jaxcuda_read_async(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t start, size_t count, void* dst, uint64_t* ticket) {
  SlotRec* s = find_slot(ctx, slot);
  if (!s) return slot_error(ctx, slot);
  if (!ticket) return fail(ctx, JAXCUDA_EINVAL, "null ticket");
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "read inside a capture: reads synchronise the stream");
  if (start > s->bytes) return fail(ctx, JAXCUDA_EINVAL, "read start %zu beyond buffer of %zu bytes", start, s->bytes);
  if (count == SIZE_MAX) count = s->bytes - start;
  if (count > s->bytes - start) return fail(ctx, JAXCUDA_EINVAL, "read of %zu bytes at %zu beyond buffer of %zu bytes", count, start, s->bytes);
  if (count && !dst) return fail(ctx, JAXCUDA_EINVAL, "null destination");
  cudaSetDevice(ctx->device);
  if (int rc = jaxcuda_comm_join(ctx)) return rc;
  if (int rc = copy_streams(ctx)) return rc;
  CUDA_TRY(ctx, cudaEventRecord(ctx->copy_fork, ctx->stream));
  CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->down_stream, ctx->copy_fork, 0));
  if (count) CUDA_TRY(ctx, cudaMemcpyAsync(dst, (const char*)s->ptr + start, count, cudaMemcpyDeviceToHost, ctx->down_stream));
  uint64_t t;
  if (!ctx->free_tickets.empty()) {
    t = ctx->free_tickets.back();
    ctx->free_tickets.pop_back();
  } else {
    cudaEvent_t ev;
    CUDA_TRY(ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    ctx->tickets.push_back(ev);
    ctx->ticket_pending.push_back(0);
    t = ctx->tickets.size();
  }
  if (ctx->tc_dispatched) {  // a tensor-core kernel that gave up a bounded wait reports through this word
    CUDA_TRY(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->down_stream));
    ctx->tc_dispatched = false;
  }
  CUDA_TRY(ctx, cudaEventRecord(ctx->tickets[t - 1], ctx->down_stream));
  ctx->ticket_pending[t - 1] = 1;
  s->read_ticket = t;
  *ticket = t;
  return JAXCUDA_OK;
}

int jaxcuda_read_wait(jaxcuda_ctx* ctx, uint64_t ticket) {
  if (!ctx || ticket == 0 || ticket > ctx->tickets.size()) return JAXCUDA_EINVAL;
  for (uint64_t f : ctx->free_tickets) if (f == ticket) return fail(ctx, JAXCUDA_EINVAL, "ticket %llu is not pending", (unsigned long long)ticket);
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaEventSynchronize(ctx->tickets[ticket - 1]));
  ctx->ticket_pending[ticket - 1] = 0;
  ctx->free_tickets.push_back(ticket);
  return check_device_status(ctx);
}

int jaxcuda_read_event(jaxcuda_ctx* ctx, uint64_t ticket, void** event) {
  if (!ctx || !event || ticket == 0 || ticket > ctx->tickets.size()) return JAXCUDA_EINVAL;
  *event = (void*)ctx->tickets[ticket - 1];
  return JAXCUDA_OK;
}

int jaxcuda_event_block(void* event) {
  if (!event) return JAXCUDA_EINVAL;
  return cudaEventSynchronize((cudaEvent_t)event) == cudaSuccess ? JAXCUDA_OK : JAXCUDA_ECUDA;
}

uint64_t jaxcuda_order_waits(jaxcuda_ctx* ctx) { return ctx ? ctx->order_waits : 0; }

int jaxcuda_prepare_kernel(jaxcuda_ctx* ctx, const uint8_t* ir, size_t len, uint64_t hash, jaxcuda_exe** out) {
  if (!ctx || !out) return JAXCUDA_EINVAL;
  *out = nullptr;
  if (!ir) return fail(ctx, JAXCUDA_EINVAL, "null kernel image");
  if (hash == 0) hash = fnv1a(ir, len);
  auto it = ctx->kernels.find(hash);
  if (it != ctx->kernels.end()) {
    it->second->handles++;
    *out = it->second.get();
    return JAXCUDA_OK;
  }
  std::unique_ptr<jaxcuda_exe> exe(new jaxcuda_exe);
  exe->ctx = ctx;
  exe->hash = hash;
  std::string err = parse_kernel(ir, len, exe->ir);
  if (!err.empty()) return fail(ctx, JAXCUDA_EINVAL, "%s", err.c_str());
  if (exe->ir.nargs > (uint32_t)jaxcuda_max_args())
    return fail(ctx, JAXCUDA_EINVAL, "kernel takes %u arguments, at most %d are supported", exe->ir.nargs, jaxcuda_max_args());
  try {
    exe->plan = make_plan(exe->ir, ctx->opt);
  } catch (const std::exception& e) {
    return fail(ctx, JAXCUDA_EUNSUPPORTED, "%s", e.what());
  }
  exe->describe = exe->plan.describe;
  if (ctx->debug >= 4) fprintf(stderr, "[jaxcuda] %016llx %s\n", (unsigned long long)hash, exe->describe.c_str());
  if (ctx->debug >= 2) fprintf(stderr, "%s\n", exe->plan.source.c_str());
  cudaSetDevice(ctx->device);
  int rc = compile_plan(ctx, exe.get());
  if (rc != JAXCUDA_OK) { free_exe(ctx, exe.get()); return rc; }
  exe->handles = 1;
  *out = exe.get();
  ctx->kernels[hash] = std::move(exe);
  return JAXCUDA_OK;
}

int jaxcuda_check_kernel(const uint8_t* ir, size_t len, int sm_count, int force_skeleton, int compile,
                         char* describe, size_t describe_len, char* message, size_t message_len) {
  auto put = [](char* dst, size_t n, const std::string& s) {
    if (dst && n) { snprintf(dst, n, "%s", s.c_str()); }
  };
  KernelIR k;
  std::string err = parse_kernel(ir, len, k);
  if (!err.empty()) { put(message, message_len, err); return JAXCUDA_EINVAL; }
  Options opt;
  if (sm_count > 0) opt.sm_count = sm_count;
  opt.force_skeleton = force_skeleton;
  opt.allow_tc = env_int("JAXCUDA_NO_TC", 0) == 0;
  Plan plan;
  try {
    plan = make_plan(k, opt);
  } catch (const std::exception& e) {
    put(message, message_len, e.what());
    return JAXCUDA_EUNSUPPORTED;
  }
  put(describe, describe_len, plan.describe);
  if (compile) {
    std::vector<char> cubin;
    if (!nvrtc_compile(plan.source, cubin, err)) { put(message, message_len, err); return JAXCUDA_ECOMPILE; }
  } else {
    put(message, message_len, plan.source);
  }
  return JAXCUDA_OK;
}

// Minimal reader for the flat JSON object of `ScatterParams` (src/routine.ts:104-110).
static const char* json_value(const char* json, const char* key) {
  if (!json) return nullptr;
  std::string pat = std::string("\"") + key + "\"";
  const char* p = strstr(json, pat.c_str());
  if (!p) return nullptr;
  p = strchr(p + pat.size(), ':');
  if (!p) return nullptr;
  p++;
  while (*p == ' ' || *p == '\t' || *p == '\n') p++;
  return p;
}
static bool json_ints(const char* json, const char* key, std::vector<long long>& out) {
  const char* p = json_value(json, key);
  if (!p || *p != '[') return false;
  p++;
  while (*p && *p != ']') {
    char* end;
    long long v = strtoll(p, &end, 10);
    if (end == p) { p++; continue; }
    out.push_back(v);
    p = end;
  }
  return *p == ']';
}

static int prepare_scatter(jaxcuda_ctx* ctx, const jaxcuda_routine_type* type, const char* params, jaxcuda_exe** out) {
  std::vector<long long> shape, axis;
  const char* op = json_value(params, "op");
  const char* od = json_value(params, "outDim");
  const char* uq = json_value(params, "uniqueIndices");
  if (!op || !od || !json_ints(params, "shape", shape) || !json_ints(params, "axis", axis))
    return fail(ctx, JAXCUDA_EINVAL, "Scatter: params need op, shape, axis, outDim and uniqueIndices");
  if (type->n_inputs < 1 || type->n_inputs != 1 + (int)axis.size() || type->n_outputs != 1 || axis.size() > 8 || shape.size() > 8)
    return fail(ctx, JAXCUDA_EINVAL, "Scatter: one updates input plus one index input per indexed axis (at most 8 axes)");
  jaxcuda_scatter_desc d = {};
  d.dtype = type->input_dtypes[0];
  const bool add = !strncmp(op, "\"add\"", 5);
  d.unique = uq && !strncmp(uq, "true", 4);
  d.mode = (add && !d.unique) ? (d.dtype == JAXCUDA_BOOL ? 2 : 1) : 0;   // routine.ts:241
  d.out_dim = atoi(od);
  d.out_rank = (int)shape.size();
  d.out_size = 1;
  for (int i = d.out_rank - 1; i >= 0; i--) { d.out_shape[i] = shape[i]; d.out_stride[i] = d.out_size; d.out_size *= shape[i]; }
  // shapes: inputs are concatenated in type->input_shapes
  const int64_t* sh = type->input_shapes;
  d.upd_rank = type->input_ranks[0];
  if (d.upd_rank > 8) return fail(ctx, JAXCUDA_EINVAL, "Scatter: rank above 8");
  d.n_updates = 1;
  for (int i = d.upd_rank - 1; i >= 0; i--) { d.upd_shape[i] = sh[i]; d.upd_stride[i] = d.n_updates; d.n_updates *= sh[i]; }
  sh += d.upd_rank;
  d.n_index = (int)axis.size();
  d.index_rank = 0;
  for (int k = 0; k < d.n_index; k++) {
    const int r = type->input_ranks[1 + k];
    if (r > 8) return fail(ctx, JAXCUDA_EINVAL, "Scatter: rank above 8");
    if (type->input_dtypes[1 + k] != JAXCUDA_I32 && type->input_dtypes[1 + k] != JAXCUDA_U32)
      return fail(ctx, JAXCUDA_EINVAL, "Scatter: index inputs must be 32-bit integers");
    d.idx_rank[k] = r;
    long long st = 1;
    for (int j = r - 1; j >= 0; j--) { d.idx_shape[k][j] = sh[j]; d.idx_stride[k][j] = st; st *= sh[j]; }
    sh += r;
    d.index_rank = std::max(d.index_rank, r);
  }
  for (int ax = 0; ax < d.out_rank; ax++) {
    d.axis_to_index[ax] = -1;
    for (int k = 0; k < d.n_index; k++) if (axis[k] == ax) d.axis_to_index[ax] = k;
  }
  int nf = 0;
  for (int i = 0; i < d.upd_rank; i++)
    if (i < d.out_dim || i >= d.out_dim + d.index_rank) d.free_dims[nf++] = i;
  if (d.n_updates >= (1ll << 31) || d.out_size >= (1ll << 31)) return fail(ctx, JAXCUDA_EINVAL, "Scatter: array too large");
  std::unique_ptr<jaxcuda_exe> exe(new jaxcuda_exe);
  exe->ctx = ctx;
  exe->kind = 3;
  exe->scatter = d;
  exe->describe = std::string("Scatter ") + (d.mode == 0 ? (d.unique ? "update" : "update (last wins)") : d.mode == 1 ? "add" : "or") +
                  " updates=" + std::to_string(d.n_updates) + " out=" + std::to_string(d.out_size);
  exe->plan.describe = exe->describe;
  exe->plan.algo_bytes = (double)(d.n_updates + d.out_size) * dtype_bytes(d.dtype) + 4.0 * d.n_updates * d.n_index;
  exe->handles = 1;
  *out = exe.get();
  ctx->routines.push_back(std::move(exe));
  return JAXCUDA_OK;
}

// TriangularSolve / Cholesky / LU: shape rules and messages of src/routine.ts:298-381.
static int prepare_linalg(jaxcuda_ctx* ctx, const char* name, const jaxcuda_routine_type* type, const char* params,
                          jaxcuda_exe** out) {
  const int kind = !strcmp(name, "TriangularSolve") ? 4 : !strcmp(name, "Cholesky") ? 5 : !strcmp(name, "LU") ? 6 :
                   !strcmp(name, "JacobiEigh") ? 7 : 8;
  const int want_in = (kind == 4 || kind == 8) ? 2 : 1, want_out = kind == 6 ? 3 : (kind == 7 || kind == 8) ? 2 : 1;
  if (type->n_inputs != want_in || type->n_outputs != want_out)
    return fail(ctx, JAXCUDA_EINVAL, "%s: wrong number of inputs or outputs", name);
  const int dt = type->input_dtypes[0];
  if (dt != JAXCUDA_F32 && dt != JAXCUDA_F64)
    return fail(ctx, JAXCUDA_EUNSUPPORTED, "%s<%s> not supported in cuda backend", name, dtype_name(dt));
  const int ra = type->input_ranks[0];
  const int64_t* as = type->input_shapes;
  std::unique_ptr<jaxcuda_exe> exe(new jaxcuda_exe);
  exe->ctx = ctx;
  exe->kind = kind;
  exe->rt_dtype = dt;
  if (kind == 8) {  // src/routine.ts:549-560
    if (ra < 1) return fail(ctx, JAXCUDA_EINVAL, "fft: input must be at least 1D");
    if (type->input_dtypes[1] != dt) return fail(ctx, JAXCUDA_EINVAL, "fft: expected matching floating-point real/imag arrays");
    const int64_t n = as[ra - 1];
    if (n < 1) return fail(ctx, JAXCUDA_EINVAL, "fft: final axis must be non-empty, got %lld", (long long)n);
    exe->rt_n = n;
    exe->rt_batch = 1;
    for (int i = 0; i < ra - 1; i++) exe->rt_batch *= as[i];
    std::vector<long long> f;
    if (!params || !json_ints(params, "factors", f)) return fail(ctx, JAXCUDA_EINVAL, "fft: params need factors");
    long long prod = 1;
    for (long long v : f) { if (v < 1) return fail(ctx, JAXCUDA_EINVAL, "fft: bad factor"); prod *= v; exe->rt_factors.push_back((int)v); }
    if (prod != n || f.size() > 32) return fail(ctx, JAXCUDA_EINVAL, "fft: factors do not multiply to the axis length %lld", (long long)n);
    const char* inv = json_value(params, "inverse");
    exe->rt_flag = inv && !strncmp(inv, "true", 4);
    exe->describe = "Fft batch=" + std::to_string(exe->rt_batch) + " n=" + std::to_string(n) + (exe->rt_flag ? " inverse" : "");
    exe->plan.describe = exe->describe;
    exe->plan.algo_bytes = 4.0 * exe->rt_batch * n * dtype_bytes(dt);
    exe->handles = 1;
    *out = exe.get();
    ctx->routines.push_back(std::move(exe));
    return JAXCUDA_OK;
  }
  if (ra < 2)
    return fail(ctx, JAXCUDA_EINVAL, "%s: %s must be at least 2D",
                kind == 4 ? "triangular_solve" : kind == 5 ? "cholesky" : kind == 6 ? "lu" : "jacobi_eigh", kind == 4 ? "a" : "input");
  int64_t lead = 1;
  for (int i = 0; i < ra - 2; i++) lead *= as[i];
  const int64_t r0 = as[ra - 2], r1 = as[ra - 1];
  if (kind == 4) {
    const int rb = type->input_ranks[1];
    const int64_t* bs = type->input_shapes + ra;
    if (rb < 2) return fail(ctx, JAXCUDA_EINVAL, "triangular_solve: b must be at least 2D");
    if (r0 != r1 || r0 != bs[rb - 1]) return fail(ctx, JAXCUDA_EINVAL, "triangular_solve: incompatible shapes");
    if (type->input_dtypes[1] != dt) return fail(ctx, JAXCUDA_EINVAL, "triangular_solve: a and b differ in dtype");
    int64_t blead = 1;
    for (int i = 0; i < rb - 2; i++) blead *= bs[i];
    if (blead != lead) return fail(ctx, JAXCUDA_EINVAL, "triangular_solve: batch dimensions of a and b differ");
    exe->rt_batch = lead;
    exe->rt_n = r0;
    exe->rt_rows = bs[rb - 2];
    const char* u = params ? json_value(params, "unitDiagonal") : nullptr;
    exe->rt_flag = u && !strncmp(u, "true", 4);
  } else if (kind == 5) {
    if (r0 != r1) return fail(ctx, JAXCUDA_EINVAL, "cholesky: input must be square, got [%lld, %lld]", (long long)r0, (long long)r1);
    exe->rt_batch = lead;
    exe->rt_n = r0;
  } else if (kind == 7) {  // src/routine.ts:440-447
    if (r0 != r1) return fail(ctx, JAXCUDA_EINVAL, "jacobi_eigh: input must be square");
    exe->rt_batch = lead;
    exe->rt_n = r0;
    const char* ms = params ? json_value(params, "maxSweeps") : nullptr;
    const char* tol = params ? json_value(params, "tolerance") : nullptr;
    if (!ms || !tol) return fail(ctx, JAXCUDA_EINVAL, "jacobi_eigh: params need maxSweeps and tolerance");
    exe->rt_flag = atoi(ms);
    exe->rt_tolerance = strtod(tol, nullptr);
  } else {
    exe->rt_batch = lead;
    exe->rt_m = r0;
    exe->rt_n = r1;
  }
  if (exe->rt_n >= (1ll << 31) || exe->rt_m >= (1ll << 31)) return fail(ctx, JAXCUDA_EINVAL, "%s: matrix too large", name);
  // Size limits of the routine kernels, reported here and not at the first dispatch.
  if (kind == 4 && exe->rt_n > 25600)
    return fail(ctx, JAXCUDA_EUNSUPPORTED, "TriangularSolve: n = %lld exceeds 25600 (one right-hand side of doubles per warp in shared memory)", (long long)exe->rt_n);
  if (kind == 7 && exe->rt_n > 32768) return fail(ctx, JAXCUDA_EUNSUPPORTED, "JacobiEigh: n = %lld exceeds 32768", (long long)exe->rt_n);
  if (kind == 5 && exe->rt_n >= 256 && (exe->rt_batch > 65535 || exe->rt_n > 0x7fffffff / 2))
    return fail(ctx, JAXCUDA_EUNSUPPORTED, "Cholesky: matrices of 256 rows or more come in batches of at most 65535, n at most 2^30");
  if (exe->rt_batch > 0x7fffffff) return fail(ctx, JAXCUDA_EUNSUPPORTED, "%s: more than 2^31-1 matrices", name);
  exe->describe = std::string(name) + " batch=" + std::to_string(exe->rt_batch) +
                  (kind == 6 ? " m=" + std::to_string(exe->rt_m) : std::string()) + " n=" + std::to_string(exe->rt_n) +
                  (kind == 4 ? " rows=" + std::to_string(exe->rt_rows) + (exe->rt_flag ? " unit" : "") : std::string());
  exe->plan.describe = exe->describe;
  const double e = dtype_bytes(dt), n = (double)exe->rt_n, b = (double)exe->rt_batch;
  if (kind == 4) { exe->plan.algo_bytes = b * (n * n + 2.0 * exe->rt_rows * n) * e; exe->plan.algo_flops = b * exe->rt_rows * n * n; }
  if (kind == 5) { exe->plan.algo_bytes = 2.0 * b * n * n * e; exe->plan.algo_flops = b * n * n * n / 3.0; }
  if (kind == 7) exe->plan.algo_bytes = 3.0 * b * n * n * e;
  if (kind == 6) {
    const double m = (double)exe->rt_m, r = std::min(m, n);
    exe->plan.algo_bytes = 2.0 * b * m * n * e + 4.0 * b * (r + m);
    exe->plan.algo_flops = b * (2.0 * m * n * r - (m + n) * r * r + 2.0 * r * r * r / 3.0);
  }
  exe->handles = 1;
  *out = exe.get();
  ctx->routines.push_back(std::move(exe));
  return JAXCUDA_OK;
}

int jaxcuda_prepare_routine(jaxcuda_ctx* ctx, const char* name, const jaxcuda_routine_type* type,
                            const char* params_json, jaxcuda_exe** out) {
  if (!ctx || !out || !name || !type) return JAXCUDA_EINVAL;
  *out = nullptr;
  if (!strcmp(name, "Scatter")) return prepare_scatter(ctx, type, params_json, out);
  if (!strcmp(name, "TriangularSolve") || !strcmp(name, "Cholesky") || !strcmp(name, "LU") || !strcmp(name, "JacobiEigh") ||
      !strcmp(name, "Fft"))
    return prepare_linalg(ctx, name, type, params_json, out);
  const bool is_sort = !strcmp(name, "Sort"), is_argsort = !strcmp(name, "Argsort");
  if (!is_sort && !is_argsort)  // wording of UnsupportedRoutineError, src/backend.ts:236-240
    return fail(ctx, JAXCUDA_EUNSUPPORTED, "routine '%s' is not supported in cuda backend", name);
  if (type->n_inputs != 1 || type->n_outputs != (is_argsort ? 2 : 1))
    return fail(ctx, JAXCUDA_EINVAL, "%s: wrong number of inputs or outputs", name);
  const int rank = type->input_ranks[0];
  if (rank == 0) return fail(ctx, JAXCUDA_EINVAL, "%s: cannot sort a scalar", is_sort ? "sort" : "argsort");  // routine.ts:187, :197
  const int dt = type->input_dtypes[0];
  std::unique_ptr<jaxcuda_exe> exe(new jaxcuda_exe);
  exe->ctx = ctx;
  exe->kind = is_sort ? 1 : 2;
  exe->rt_dtype = dt;
  exe->rt_n = type->input_shapes[rank - 1];
  exe->rt_batch = 1;
  for (int i = 0; i < rank - 1; i++) exe->rt_batch *= type->input_shapes[i];
  if (exe->rt_n >= (1ll << 31)) return fail(ctx, JAXCUDA_EINVAL, "%s: axis too long", name);
  exe->describe = std::string(name) + " batch=" + std::to_string(exe->rt_batch) + " n=" + std::to_string(exe->rt_n);
  exe->plan.describe = exe->describe;
  exe->plan.algo_bytes = 2.0 * exe->rt_batch * exe->rt_n * dtype_bytes(dt) + (is_argsort ? 4.0 * exe->rt_batch * exe->rt_n : 0);
  exe->handles = 1;
  *out = exe.get();
  ctx->routines.push_back(std::move(exe));
  return JAXCUDA_OK;
}

static int dispatch_untraced(jaxcuda_ctx* ctx, jaxcuda_exe* exe, const jaxcuda_slot* inputs, int n_inputs,
                             const jaxcuda_slot* outputs, int n_outputs);

static const size_t kTraceLimit = 1 << 20;   // dispatches kept per trace; later ones run untimed

static int trace_event(jaxcuda_ctx* ctx, cudaEvent_t* out) {
  if (ctx->trace_events_used == ctx->trace_events.size()) {
    cudaEvent_t ev;
    CUDA_TRY(ctx, cudaEventCreate(&ev));
    ctx->trace_events.push_back(ev);
  }
  *out = ctx->trace_events[ctx->trace_events_used++];
  return JAXCUDA_OK;
}

int jaxcuda_dispatch(jaxcuda_ctx* ctx, jaxcuda_exe* exe, const jaxcuda_slot* inputs, int n_inputs,
                     const jaxcuda_slot* outputs, int n_outputs) {
  if (!ctx || !exe || exe->ctx != ctx) return JAXCUDA_EINVAL;
  // A captured list is timed as a whole by whoever replays it; its dispatches are deferred and fused.
  if (!ctx->tracing || ctx->alloc.capturing || ctx->trace.size() >= kTraceLimit)
    return dispatch_untraced(ctx, exe, inputs, n_inputs, outputs, n_outputs);
  cudaSetDevice(ctx->device);
  jaxcuda_ctx::TraceRec rec{exe, exe->describe, nullptr, nullptr};
  if (int rc = trace_event(ctx, &rec.begin)) return rc;
  if (int rc = trace_event(ctx, &rec.end)) return rc;
  CUDA_TRY(ctx, cudaEventRecord(rec.begin, ctx->stream));
  const int rc = dispatch_untraced(ctx, exe, inputs, n_inputs, outputs, n_outputs);
  CUDA_TRY(ctx, cudaEventRecord(rec.end, ctx->stream));
  if (rc == JAXCUDA_OK) ctx->trace.push_back(std::move(rec));
  return rc;
}

static int dispatch_untraced(jaxcuda_ctx* ctx, jaxcuda_exe* exe, const jaxcuda_slot* inputs, int n_inputs,
                             const jaxcuda_slot* outputs, int n_outputs) {
  cudaSetDevice(ctx->device);
  std::vector<SlotRec*> in(n_inputs), outv(n_outputs);
  for (int i = 0; i < n_inputs; i++) if (!(in[i] = find_slot(ctx, inputs[i]))) return slot_error(ctx, inputs[i]);
  for (int i = 0; i < n_outputs; i++) if (!(outv[i] = find_slot(ctx, outputs[i]))) return slot_error(ctx, outputs[i]);
  for (int i = 0; i < n_outputs; i++) if (int rc = order_after_users(ctx, outv[i])) return rc;
  for (int i = 0; i < n_inputs; i++) if (int rc = order_after_sum(ctx, in[i])) return rc;
  for (int i = 0; i < n_outputs; i++) drop_lo_plane(ctx, outv[i]->ptr);

  if (exe->kind != 0)
    if (int rc = flush_pending(ctx)) return rc;
  if (exe->kind == 3) {  // Scatter
    const jaxcuda_scatter_desc& d = exe->scatter;
    if (n_inputs != 1 + d.n_index || n_outputs != 1) return fail(ctx, JAXCUDA_EINVAL, "Scatter called with wrong slot counts");
    const size_t eb = dtype_bytes(d.dtype);
    if (in[0]->bytes < (size_t)d.n_updates * eb || outv[0]->bytes < (size_t)d.out_size * eb)
      return fail(ctx, JAXCUDA_EINVAL, "Scatter buffers are smaller than its declared shapes");
    const void* idx[8] = {};
    for (int k = 0; k < d.n_index; k++) idx[k] = in[1 + k]->ptr;
    const size_t wb = jaxcuda_scatter_work_bytes(&d);
    void* work = nullptr;
    if (wb) {
      cudaError_t e = ctx->alloc.get(wb, &work);
      if (e != cudaSuccess) return fail(ctx, JAXCUDA_ENOMEM, "scatter work space of %zu bytes: %s", wb, cudaGetErrorString(e));
    }
    int launches = 0;
    int rc = jaxcuda_scatter_launch(ctx->stream, &d, in[0]->ptr, idx, outv[0]->ptr, work, &launches);
    ctx->launches += launches;
    if (work) ctx->alloc.put(work, wb);
    if (rc) return fail(ctx, JAXCUDA_ECUDA, "scatter launch: %s", cudaGetErrorString((cudaError_t)rc));
    return JAXCUDA_OK;
  }
  if (exe->kind >= 4) {  // TriangularSolve / Cholesky / LU
    const size_t e = dtype_bytes(exe->rt_dtype);
    const size_t b = (size_t)exe->rt_batch, n = (size_t)exe->rt_n, m = (size_t)exe->rt_m, rows = (size_t)exe->rt_rows;
    int launches = 0, rc = 0;
    if (exe->kind == 4) {
      if (n_inputs != 2 || n_outputs != 1) return fail(ctx, JAXCUDA_EINVAL, "TriangularSolve called with wrong slot counts");
      if (in[0]->bytes < b * n * n * e || in[1]->bytes < b * rows * n * e || outv[0]->bytes < b * rows * n * e)
        return fail(ctx, JAXCUDA_EINVAL, "routine buffers are smaller than its declared shapes");
      rc = jaxcuda_triangular_solve_launch(ctx->stream, exe->rt_dtype, in[0]->ptr, in[1]->ptr, outv[0]->ptr, exe->rt_batch,
                                           exe->rt_rows, exe->rt_n, exe->rt_flag, &launches);
    } else if (exe->kind == 7) {
      if (n_inputs != 1 || n_outputs != 2) return fail(ctx, JAXCUDA_EINVAL, "JacobiEigh called with wrong slot counts");
      if (in[0]->bytes < b * n * n * e || outv[0]->bytes < b * n * n * e || outv[1]->bytes < b * n * n * e)
        return fail(ctx, JAXCUDA_EINVAL, "routine buffers are smaller than its declared shapes");
      rc = jaxcuda_jacobi_eigh_launch(ctx->stream, exe->rt_dtype, in[0]->ptr, outv[0]->ptr, outv[1]->ptr, exe->rt_batch, exe->rt_n,
                                      exe->rt_flag, exe->rt_tolerance, &launches);
    } else if (exe->kind == 8) {
      if (n_inputs != 2 || n_outputs != 2) return fail(ctx, JAXCUDA_EINVAL, "Fft called with wrong slot counts");
      for (int i = 0; i < 2; i++)
        if (in[i]->bytes < b * n * e || outv[i]->bytes < b * n * e)
          return fail(ctx, JAXCUDA_EINVAL, "routine buffers are smaller than its declared shapes");
      int max_radix = 1;
      for (int f : exe->rt_factors) max_radix = std::max(max_radix, f);
      const size_t wb = jaxcuda_fft_work_bytes(exe->rt_dtype, exe->rt_batch, exe->rt_n, max_radix);
      void* work = nullptr;
      if (wb) {
        cudaError_t ae = ctx->alloc.get(wb, &work);
        if (ae != cudaSuccess) return fail(ctx, JAXCUDA_ENOMEM, "fft work space of %zu bytes: %s", wb, cudaGetErrorString(ae));
      }
      rc = jaxcuda_fft_launch(ctx->stream, exe->rt_dtype, in[0]->ptr, in[1]->ptr, outv[0]->ptr, outv[1]->ptr, exe->rt_batch, exe->rt_n,
                              exe->rt_factors.data(), (int)exe->rt_factors.size(), exe->rt_flag, work, &launches);
      if (work) ctx->alloc.put(work, wb);  // stream order keeps it alive for the launches above
    } else if (exe->kind == 5) {
      if (n_inputs != 1 || n_outputs != 1) return fail(ctx, JAXCUDA_EINVAL, "Cholesky called with wrong slot counts");
      if (in[0]->bytes < b * n * n * e || outv[0]->bytes < b * n * n * e)
        return fail(ctx, JAXCUDA_EINVAL, "routine buffers are smaller than its declared shapes");
      const size_t wb = jaxcuda_cholesky_work_bytes(exe->rt_batch, exe->rt_n);
      void* work = nullptr;
      if (wb) {
        cudaError_t ae = ctx->alloc.get(wb, &work);
        if (ae != cudaSuccess) return fail(ctx, JAXCUDA_ENOMEM, "cholesky work space of %zu bytes: %s", wb, cudaGetErrorString(ae));
      }
      rc = jaxcuda_cholesky_launch(ctx->stream, exe->rt_dtype, in[0]->ptr, outv[0]->ptr, exe->rt_batch, exe->rt_n, work, &launches);
      if (work) ctx->alloc.put(work, wb);
    } else {
      if (n_inputs != 1 || n_outputs != 3) return fail(ctx, JAXCUDA_EINVAL, "LU called with wrong slot counts");
      const size_t r = std::min(m, n);
      if (in[0]->bytes < b * m * n * e || outv[0]->bytes < b * m * n * e || outv[1]->bytes < b * r * 4 || outv[2]->bytes < b * m * 4)
        return fail(ctx, JAXCUDA_EINVAL, "routine buffers are smaller than its declared shapes");
      rc = jaxcuda_lu_launch(ctx->stream, exe->rt_dtype, in[0]->ptr, outv[0]->ptr, (int32_t*)outv[1]->ptr, (int32_t*)outv[2]->ptr,
                             exe->rt_batch, exe->rt_m, exe->rt_n, &launches);
    }
    ctx->launches += launches;
    if (rc) return fail(ctx, JAXCUDA_ECUDA, "%s launch: %s", exe->describe.c_str(), cudaGetErrorString((cudaError_t)rc));
    return JAXCUDA_OK;
  }
  if (exe->kind != 0) {  // Sort / Argsort
    const bool arg = exe->kind == 2;
    if (n_inputs != 1 || n_outputs != (arg ? 2 : 1)) return fail(ctx, JAXCUDA_EINVAL, "routine called with wrong slot counts");
    const size_t need = (size_t)exe->rt_batch * exe->rt_n * dtype_bytes(exe->rt_dtype);
    if (in[0]->bytes < need || outv[0]->bytes < need || (arg && outv[1]->bytes < (size_t)exe->rt_batch * exe->rt_n * 4))
      return fail(ctx, JAXCUDA_EINVAL, "routine buffers are smaller than its declared shapes");
    const size_t wb = jaxcuda_sort_work_bytes(arg, exe->rt_dtype, exe->rt_batch, exe->rt_n);
    void* work = nullptr;
    if (wb) {
      cudaError_t e = ctx->alloc.get(wb, &work);
      if (e != cudaSuccess) return fail(ctx, JAXCUDA_ENOMEM, "sort work space of %zu bytes: %s", wb, cudaGetErrorString(e));
    }
    int launches = 0;
    int rc = jaxcuda_sort_launch(ctx->stream, arg, in[0]->ptr, outv[0]->ptr, arg ? (int32_t*)outv[1]->ptr : nullptr,
                                 exe->rt_dtype, exe->rt_batch, exe->rt_n, work, &launches);
    ctx->launches += launches;
    if (work) ctx->alloc.put(work, wb);  // stream order keeps it alive for the launches above
    if (rc) return fail(ctx, JAXCUDA_ECUDA, "sort launch: %s", cudaGetErrorString((cudaError_t)rc));
    return JAXCUDA_OK;
  }

  const KernelIR& k = exe->ir;
  if ((uint32_t)n_inputs != k.nargs || n_outputs != 1)
    return fail(ctx, JAXCUDA_EINVAL, "kernel takes %u inputs and 1 output, got %d and %d", k.nargs, n_inputs, n_outputs);
  const size_t out_bytes = (size_t)k.size * dtype_bytes(k.out_dtype());
  if (outv[0]->bytes < out_bytes)
    return fail(ctx, JAXCUDA_EINVAL, "output buffer of %zu bytes is smaller than the kernel's %zu", outv[0]->bytes, out_bytes);
  auto check_len = [&](const std::vector<Node>& nodes) -> int {
    for (const Node& nd : nodes)
      if (nd.op == JAXCUDA_OP_GLOBALINDEX && in[nd.arg0]->bytes < (size_t)nd.arg1 * dtype_bytes(nd.dtype))
        return fail(ctx, JAXCUDA_EINVAL, "input %llu holds %zu bytes, the kernel addresses %zu", (unsigned long long)nd.arg0,
                    in[nd.arg0]->bytes, (size_t)nd.arg1 * dtype_bytes(nd.dtype));
    return JAXCUDA_OK;
  };
  if (int rc = check_len(k.exp)) return rc;
  if (int rc = check_len(k.epi)) return rc;
  for (int i = 0; i < n_inputs; i++)
    if (in[i]->ptr && in[i]->ptr == outv[0]->ptr)
      return fail(ctx, JAXCUDA_EINVAL, "output slot %u is also input %d; kernels read inputs through the read-only path", outputs[0], i);
  if (k.size == 0) return JAXCUDA_OK;
  std::vector<void*> inptr(n_inputs);
  for (int i = 0; i < n_inputs; i++) inptr[i] = in[i]->ptr;
  if (ctx->alloc.capturing && ctx->fuse_rows) {
    if (exe->plan.scratch_bytes && exe->plan.scratch_persistent && !exe->persistent_scratch)
      return fail(ctx, JAXCUDA_EINVAL, "dispatch the program once before capturing it: a kernel still has to set up its arrival counters");
    PendingDispatch pd;
    pd.exe = exe;
    pd.in = inptr;
    for (int i = 0; i < n_inputs; i++) pd.in_bytes.push_back(in[i]->bytes);
    pd.out = outv[0]->ptr;
    pd.out_bytes = outv[0]->bytes;
    const Plan& pl = exe->plan;
    if (ctx->keep_lo_planes && pl.skeleton == SK_GEMM_TC && pl.tc_kind == 2 && !pl.tc_lo_in_kernel && !pl.gemm.b_gathered &&
        pl.tc_sk_counter_bytes == 0) {
      if (int rc = plane_ticket(ctx, inptr[pl.gemm.gidA], pl.gemm.lenA, pd.lo.a, pd.lo.compute_a)) return rc;
      if (int rc = plane_ticket(ctx, inptr[pl.gemm.gidB], pl.gemm.lenB, pd.lo.b, pd.lo.compute_b)) return rc;
    }
    ctx->pending.push_back(std::move(pd));
    return JAXCUDA_OK;
  }
  if (int rc = flush_pending(ctx)) return rc;
  return launch_kernel(ctx, exe, inptr, outv[0]->ptr);
}

}  // extern "C"

// Launches one prepared Kernel on the context's stream.
static int launch_kernel(jaxcuda_ctx* ctx, jaxcuda_exe* exe, const std::vector<void*>& inptr, void* outptr, const LoPlanes* lo) {
  const int n_inputs = (int)inptr.size();
  if (ctx->alloc.capturing) ctx->capture_bytes += exe->plan.algo_bytes;
  void* scratch = nullptr;
  if (exe->plan.scratch_bytes && exe->plan.scratch_persistent) {
    if (!exe->persistent_scratch && ctx->alloc.capturing)
      return fail(ctx, JAXCUDA_EINVAL, "dispatch the program once before capturing it: a kernel still has to set up its arrival counters");
    if (!exe->persistent_scratch) {
      cudaError_t e = ctx->alloc.get(exe->plan.scratch_bytes, &exe->persistent_scratch);
      if (e == cudaSuccess) e = cudaMemsetAsync(exe->persistent_scratch, 0, exe->plan.scratch_bytes, ctx->stream);
      if (e != cudaSuccess) return fail(ctx, JAXCUDA_ENOMEM, "scratch of %zu bytes: %s", exe->plan.scratch_bytes, cudaGetErrorString(e));
    }
    scratch = exe->persistent_scratch;
  } else if (exe->plan.scratch_bytes && !(lo && lo->a && lo->b)) {   // (kept remainder planes are all the scratch such a GEMM has)
    cudaError_t e = ctx->alloc.get(exe->plan.scratch_bytes, &scratch);
    if (e != cudaSuccess) return fail(ctx, JAXCUDA_ENOMEM, "scratch of %zu bytes: %s", exe->plan.scratch_bytes, cudaGetErrorString(e));
  }
  int rc = JAXCUDA_OK;
  if (exe->plan.skeleton == SK_GEMM_TC) {
    std::string err;
    int nl = launch_gemm_tc(ctx->drv.TensorMapEncodeTiled, (void*)ctx->drv.LaunchKernel, (void*)ctx->drv.LaunchKernelEx, exe->plan, exe->fns, inptr,
                            outptr, scratch, ctx->stream, ctx->status_dev, err,
                            // a persistent GEMM that holds every SM would keep a sum begun on the second
                            // stream waiting until it ends; leave that sum a few SMs while one is in flight
                            ctx->comm_pending && ctx->comm_sms > 0 ? std::max(1, ctx->opt.sm_count - ctx->comm_sms) : 0,
                            (lo && lo->a && lo->b) ? lo : nullptr);
    if (nl < 0) rc = fail(ctx, JAXCUDA_ECUDA, "%s", err.c_str());
    else { ctx->launches += nl; ctx->tc_dispatched = true; }
  } else {
    std::vector<void*> ptrs(n_inputs + 2);
    std::vector<void*> args(n_inputs + 3);
    int rev = 0;
    if (exe->plan.takes_rev) {
      rev = ctx->sweep_alternate ? ctx->sweep : 0;
      // only a kernel that streams more than a fraction of L2 changes what the cache holds
      if (exe->plan.algo_bytes >= 16.0 * 1024 * 1024) ctx->sweep ^= 1;
    }
    args[n_inputs + 2] = &rev;
    for (int i = 0; i < n_inputs; i++) ptrs[i] = inptr[i];
    ptrs[n_inputs] = outptr;
    ptrs[n_inputs + 1] = scratch;
    for (size_t i = 0; i < ptrs.size(); i++) args[i] = &ptrs[i];
    for (size_t s = 0; s < exe->plan.stages.size() && rc == JAXCUDA_OK; s++) {
      const Stage& st = exe->plan.stages[s];
      CUresult cr = ctx->drv.LaunchKernel(exe->fns[s], st.grid[0], st.grid[1], st.grid[2], st.block[0], st.block[1],
                                          st.block[2], st.smem, (CUstream)ctx->stream, args.data(), nullptr);
      if (cr != CUDA_SUCCESS) rc = drv_fail(ctx, "cuLaunchKernel", cr);
      else ctx->launches++;
    }
  }
  if (scratch && !exe->plan.scratch_persistent) ctx->alloc.put(scratch, exe->plan.scratch_bytes);
  return rc;
}

// The Kernels list[i..end) as stages of one row program over [R, C]: a buffer table with one entry
// per array instance (an address that is written again is a new instance), the stages, the address
// behind every buffer and a key that identifies the wiring.  False where the group must not be
// fused as it stands (a stage would overwrite an array the group reads).
struct RowGroup {
  std::vector<FuseBuffer> bufs;
  std::vector<void*> ptr_of;
  std::vector<FuseStage> stages;
  std::string key;
};

static bool build_row_group(const std::vector<PendingDispatch>& list, size_t i, size_t end, int64_t R, int64_t C, RowGroup& g) {
  // An output that the list releases needs no store only if nothing behind the group reads it before
  // the release.
  auto dies_inside = [&](const PendingDispatch& pd) {
    if (!pd.out_freed) return false;
    for (size_t r = end; r < list.size() && r < pd.freed_at; r++)
      for (void* p : list[r].in) if (p == pd.out) return false;
    return true;
  };
  std::unordered_map<void*, int> cur;
  std::map<std::string, int> seen;  // Kernel + inputs -> output buffer, for repeated Kernels
  std::ostringstream key;
  key << R << "x" << C;
  for (size_t s = i; s < end; s++) {
    const PendingDispatch& pd = list[s];
    FuseStage st;
    st.ir = &pd.exe->ir;
    std::ostringstream sk;
    sk << std::hex << pd.exe->hash << ":";
    for (size_t a = 0; a < pd.in.size(); a++) {
      auto it = cur.find(pd.in[a]);
      int b;
      if (it != cur.end()) b = it->second;
      else {
        FuseBuffer fb;
        fb.external = true;
        fb.bytes = pd.in_bytes[a];
        b = (int)g.bufs.size();
        g.bufs.push_back(fb);
        g.ptr_of.push_back(pd.in[a]);
        cur[pd.in[a]] = b;
      }
      st.in_buf.push_back(b);
      sk << b << ",";
    }
    auto oit = cur.find(pd.out);
    if (oit != cur.end() && g.bufs[oit->second].external) return false;
    auto dup = seen.find(sk.str());
    if (dup != seen.end() && dies_inside(pd)) {  // the same Kernel on the same arrays again: reuse its result
      cur[pd.out] = dup->second;
      key << "|=" << dup->second;
      continue;
    }
    FuseBuffer ob;
    ob.store = !dies_inside(pd);
    ob.bytes = pd.out_bytes;
    st.out_buf = (int)g.bufs.size();
    g.bufs.push_back(ob);
    g.ptr_of.push_back(pd.out);
    cur[pd.out] = st.out_buf;
    seen[sk.str()] = st.out_buf;
    key << "|" << sk.str() << ">" << st.out_buf << (ob.store ? "s" : "");
    g.stages.push_back(st);
  }
  g.key = key.str();
  return !g.stages.empty();
}

// The longest run of row stages that starts at list[i] (a row reduction); 0 if there is none.
static size_t row_group_extent(const std::vector<PendingDispatch>& list, size_t i, int64_t& R, int64_t& C) {
  const KernelIR& seed = list[i].exe->ir;
  if (list[i].exe->kind != 0 || !seed.has_red) return 0;
  R = (int64_t)seed.size;
  C = (int64_t)seed.red_size;
  if (C % 4 || row_stage_type(seed, R, C) != RS_REDUCE) return 0;
  size_t end = i;
  while (end < list.size() && list[end].exe->kind == 0 && row_stage_type(list[end].exe->ir, R, C) != RS_NONE) end++;
  return end - i >= 2 ? end : 0;
}

// Tries to replace the Kernels pending[i..] by one row program; returns the index after the last
// Kernel it covered, or i if it launched nothing.
static size_t launch_row_group(jaxcuda_ctx* ctx, std::vector<PendingDispatch>& list, size_t i) {
  int64_t R = 0, C = 0;
  size_t end = row_group_extent(list, i, R, C);
  for (; end >= i + 2; end--) {
    RowGroup g;
    if (!build_row_group(list, i, end, R, C, g)) continue;
    jaxcuda_exe* fx = nullptr;
    auto hit = ctx->fused.find(g.key);
    if (hit != ctx->fused.end()) fx = hit->second.get();
    else {
      std::unique_ptr<jaxcuda_exe> exe(new jaxcuda_exe);
      exe->ctx = ctx;
      std::string why;
      bool planned = false;
      try {
        planned = plan_row_fusion(g.stages, g.bufs, R, C, ctx->opt, exe->plan, exe->fuse_params, why);
      } catch (const std::exception& e) { why = e.what(); }
      if (!planned) {
        if (ctx->debug >= 4) fprintf(stderr, "[jaxcuda] no row program for %zu kernels: %s\n", end - i, why.c_str());
        ctx->fused[g.key] = nullptr;   // remember the refusal
        continue;
      }
      exe->describe = exe->plan.describe;
      if (ctx->debug >= 4) fprintf(stderr, "[jaxcuda] %s\n", exe->describe.c_str());
      if (ctx->debug >= 2) fprintf(stderr, "%s\n", exe->plan.source.c_str());
      if (compile_plan(ctx, exe.get()) != JAXCUDA_OK) {
        if (ctx->debug >= 1) fprintf(stderr, "[jaxcuda] row program failed to compile: %s\n", ctx->last_error.c_str());
        free_exe(ctx, exe.get());
        ctx->fused[g.key] = nullptr;
        continue;
      }
      fx = exe.get();
      ctx->fused[g.key] = std::move(exe);
    }
    if (!fx) continue;
    std::vector<void*> ptrs(fx->fuse_params.size());
    std::vector<void*> args(ptrs.size());
    for (size_t a = 0; a < ptrs.size(); a++) { ptrs[a] = g.ptr_of[fx->fuse_params[a]]; args[a] = &ptrs[a]; }
    const Stage& st = fx->plan.stages[0];
    CUresult cr = ctx->drv.LaunchKernel(fx->fns[0], st.grid[0], st.grid[1], st.grid[2], st.block[0], st.block[1], st.block[2],
                                        st.smem, (CUstream)ctx->stream, args.data(), nullptr);
    if (cr != CUDA_SUCCESS) { drv_fail(ctx, "cuLaunchKernel (row program)", cr); return i; }
    ctx->launches++;
    ctx->capture_bytes += fx->plan.algo_bytes;
    ctx->capture_groups++;
    return end;
  }
  return i;
}

// Kernel list[i] (elementwise, a reduction of size 1 included) feeds only list[i + 1], which is
// elementwise, and its output is released afterwards: the consumer with the producer's expression
// in place of its load (emit.hpp: compose_elementwise).  Returns the argument of the consumer that
// is replaced, or -1.
static int composable_pair(const std::vector<PendingDispatch>& list, size_t i, KernelIR& composed, bool& epilogue) {
  if (i + 1 >= list.size()) return -1;
  const PendingDispatch& a = list[i];
  const PendingDispatch& b = list[i + 1];
  if (a.exe->kind != 0 || b.exe->kind != 0 || !a.out_freed || a.freed_at < i + 2) return -1;
  int b_arg = -1;
  for (size_t k = 0; k < b.in.size(); k++)
    if (b.in[k] == a.out) { if (b_arg >= 0) return -1; b_arg = (int)k; }
  if (b_arg < 0) return -1;
  for (size_t r = i + 2; r < list.size() && r < a.freed_at; r++)   // another reader of the same array
    for (void* p : list[r].in) if (p == a.out) return -1;
  for (void* p : a.in) if (p == b.out) return -1;                  // the consumer's output replaces one of the producer's inputs
  std::string why;
  if (compose_elementwise(a.exe->ir, b.exe->ir, (uint32_t)b_arg, composed, why)) { epilogue = false; return b_arg; }
  // a GEMM-shaped Kernel takes an elementwise consumer of its own outputs into its epilogue
  if ((a.exe->plan.skeleton == SK_GEMM_TC || a.exe->plan.skeleton == SK_GEMM_FFMA) &&
      compose_epilogue(a.exe->ir, b.exe->ir, (uint32_t)b_arg, composed, why)) {
    epilogue = true;
    return b_arg;
  }
  return -1;
}

// arguments of the composed Kernel: the consumer's without the replaced one, then the producer's
// (the other way round when the consumer went into the producer's epilogue)
static std::vector<void*> composed_inputs(const PendingDispatch& a, const PendingDispatch& b, int b_arg, bool epilogue) {
  std::vector<void*> in;
  if (epilogue) for (void* p : a.in) in.push_back(p);
  for (size_t k = 0; k < b.in.size(); k++) if ((int)k != b_arg) in.push_back(b.in[k]);
  if (!epilogue) for (void* p : a.in) in.push_back(p);
  return in;
}

// Launches list[i] and list[i + 1] as one Kernel where that is possible; returns i + 2 then, else i.
static size_t launch_composed_pair(jaxcuda_ctx* ctx, std::vector<PendingDispatch>& list, size_t i) {
  KernelIR composed;
  bool epilogue = false;
  const int b_arg = composable_pair(list, i, composed, epilogue);
  if (b_arg < 0) return i;
  std::ostringstream key;
  key << "compose:" << std::hex << list[i].exe->hash << ">" << list[i + 1].exe->hash << "@" << b_arg;
  jaxcuda_exe* fx = nullptr;
  auto hit = ctx->fused.find(key.str());
  if (hit != ctx->fused.end()) fx = hit->second.get();
  else {
    std::unique_ptr<jaxcuda_exe> exe(new jaxcuda_exe);
    exe->ctx = ctx;
    exe->ir = composed;
    bool ok = false;
    try {
      exe->plan = make_plan(exe->ir, ctx->opt);
      // the longer epilogue must not cost the producer its skeleton
      auto family = [](const std::string& d) { return d.substr(0, d.find(' ')); };
      ok = !epilogue || (exe->plan.skeleton == list[i].exe->plan.skeleton && family(exe->plan.describe) == family(list[i].exe->plan.describe));
    } catch (const std::exception&) {}
    if (ok) {
      exe->describe = exe->plan.describe + (epilogue ? " (consumer in the epilogue)" : " (producer substituted)");
      if (ctx->debug >= 4) fprintf(stderr, "[jaxcuda] %s\n", exe->describe.c_str());
      if (ctx->debug >= 2) fprintf(stderr, "%s\n", exe->plan.source.c_str());
      if (compile_plan(ctx, exe.get()) != JAXCUDA_OK) { free_exe(ctx, exe.get()); ok = false; }
    }
    if (!ok) { ctx->fused[key.str()] = nullptr; return i; }
    fx = exe.get();
    ctx->fused[key.str()] = std::move(exe);
  }
  if (!fx) return i;
  // (a GEMM that took its consumer into the epilogue has the GEMM's operands first: its planes apply)
  if (launch_kernel(ctx, fx, composed_inputs(list[i], list[i + 1], b_arg, epilogue), list[i + 1].out, epilogue ? &list[i].lo : nullptr) != JAXCUDA_OK) return i;
  ctx->capture_groups++;
  return i + 2;
}

// ---- runs of small Kernels as one launch (emit.hpp: plan_small_batch) ---------------------------
static bool is_small_kernel(const PendingDispatch& pd) {
  if (pd.exe->kind != 0) return false;
  const KernelIR& k = pd.exe->ir;
  if (k.size == 0 || (double)k.size * (k.has_red ? std::max<uint32_t>(1, k.red_size) : 1) > small_kernel_work() || k.nargs > 16) return false;
  // A reduction joins only if its own kernel also adds up one output's terms in order in one thread
  // (the batch does): then a replay keeps the bits of the Kernels one by one.
  if (k.has_red && k.red_size > 1) {
    const std::string& d = pd.exe->plan.describe;
    if (pd.exe->plan.skeleton != SK_REDUCE_COL || d.find(" TY=1 splits=1") == std::string::npos) return false;
  }
  return true;
}

struct SmallBatch {
  std::vector<BatchStage> stages;
  std::vector<void*> params;
  std::string key;
};

static size_t small_batch_extent(const std::vector<PendingDispatch>& list, size_t i) {
  size_t end = i;
  while (end < list.size() && end - i < 24 && is_small_kernel(list[end])) end++;
  return end - i >= 3 ? end : 0;
}

static void build_small_batch(const std::vector<PendingDispatch>& list, size_t i, size_t end, SmallBatch& b) {
  std::unordered_map<void*, int> at;
  auto param = [&](void* p) {
    auto it = at.find(p);
    if (it != at.end()) return it->second;
    const int n = (int)b.params.size();
    b.params.push_back(p);
    at[p] = n;
    return n;
  };
  std::ostringstream key;
  key << "batch";
  for (size_t s = i; s < end; s++) {
    BatchStage st;
    st.ir = &list[s].exe->ir;
    key << "|" << std::hex << list[s].exe->hash << ":";
    for (void* p : list[s].in) { st.in_param.push_back(param(p)); key << st.in_param.back() << ","; }
    st.out_param = param(list[s].out);
    key << ">" << st.out_param;
    b.stages.push_back(st);
  }
  b.key = key.str();
}

static size_t launch_small_batch(jaxcuda_ctx* ctx, std::vector<PendingDispatch>& list, size_t i) {
  const size_t end = small_batch_extent(list, i);
  if (!end) return i;
  SmallBatch b;
  build_small_batch(list, i, end, b);
  jaxcuda_exe* fx = nullptr;
  auto hit = ctx->fused.find(b.key);
  if (hit != ctx->fused.end()) fx = hit->second.get();
  else {
    std::unique_ptr<jaxcuda_exe> exe(new jaxcuda_exe);
    exe->ctx = ctx;
    std::string why;
    bool ok = false;
    try { ok = plan_small_batch(b.stages, (int)b.params.size(), ctx->opt, exe->plan, why); } catch (const std::exception&) {}
    if (ok) {
      exe->describe = exe->plan.describe;
      if (ctx->debug >= 4) fprintf(stderr, "[jaxcuda] %s\n", exe->describe.c_str());
      if (ctx->debug >= 2) fprintf(stderr, "%s\n", exe->plan.source.c_str());
      if (compile_plan(ctx, exe.get()) != JAXCUDA_OK) { free_exe(ctx, exe.get()); ok = false; }
    }
    if (!ok) { ctx->fused[b.key] = nullptr; return i; }
    fx = exe.get();
    ctx->fused[b.key] = std::move(exe);
  }
  if (!fx) return i;
  std::vector<void*> args(b.params.size());
  for (size_t a = 0; a < args.size(); a++) args[a] = &b.params[a];
  const Stage& st = fx->plan.stages[0];
  CUresult cr = ctx->drv.LaunchKernel(fx->fns[0], 1, 1, 1, st.block[0], 1, 1, 0, (CUstream)ctx->stream, args.data(), nullptr);
  if (cr != CUDA_SUCCESS) { drv_fail(ctx, "cuLaunchKernel (small batch)", cr); return i; }
  ctx->launches++;
  ctx->capture_bytes += fx->plan.algo_bytes;
  ctx->capture_groups++;
  return end;
}

// Launches everything dispatched so far inside the capture, in order.
static int flush_pending(jaxcuda_ctx* ctx) {
  if (ctx->pending.empty()) return JAXCUDA_OK;
  std::vector<PendingDispatch> list = std::move(ctx->pending);
  ctx->pending.clear();
  for (size_t i = 0; i < list.size();) {
    size_t next = launch_row_group(ctx, list, i);
    if (next > i) { i = next; continue; }
    next = launch_composed_pair(ctx, list, i);
    if (next > i) { i = next; continue; }
    next = launch_small_batch(ctx, list, i);
    if (next > i) { i = next; continue; }
    if (int rc = launch_kernel(ctx, list[i].exe, list[i].in, list[i].out, &list[i].lo)) return rc;
    i++;
  }
  return JAXCUDA_OK;
}

extern "C" {

int jaxcuda_check_step_list(int n, const uint8_t* const* irs, const size_t* lens, const int* n_inputs, const int* inputs,
                            const int* outputs, const uint8_t* output_freed, int compile, char* report, size_t report_len,
                            char* message, size_t message_len) {
  auto put = [](char* dst, size_t cap, const std::string& s) {
    if (dst && cap) { snprintf(dst, cap, "%s", s.c_str()); }
  };
  if (n < 0 || (n > 0 && (!irs || !lens || !n_inputs || !inputs || !outputs))) return JAXCUDA_EINVAL;
  std::vector<std::unique_ptr<jaxcuda_exe>> exes;
  std::vector<PendingDispatch> list;
  Options opt;
  opt.allow_tc = env_int("JAXCUDA_NO_TC", 0) == 0;
  size_t at = 0;
  for (int i = 0; i < n; i++) {
    std::unique_ptr<jaxcuda_exe> exe(new jaxcuda_exe);
    std::string err = parse_kernel(irs[i], lens[i], exe->ir);
    if (!err.empty()) { put(message, message_len, err); return JAXCUDA_EINVAL; }
    exe->hash = fnv1a(irs[i], lens[i]);
    try { exe->plan = make_plan(exe->ir, opt); } catch (const std::exception&) {}   // reported (or refused) per Kernel below
    PendingDispatch pd;
    pd.exe = exe.get();
    // the diagnostic has no buffers: array ids stand in for addresses, sizes are taken as sufficient
    for (int a = 0; a < n_inputs[i]; a++) { pd.in.push_back((void*)(uintptr_t)(inputs[at + a] + 1)); pd.in_bytes.push_back((size_t)1 << 40); }
    at += n_inputs[i];
    pd.out = (void*)(uintptr_t)(outputs[i] + 1);
    pd.out_bytes = (size_t)1 << 40;
    pd.out_freed = output_freed && output_freed[i];
    list.push_back(std::move(pd));
    exes.push_back(std::move(exe));
  }
  std::ostringstream rep, src;
  for (size_t i = 0; i < list.size();) {
    int64_t R = 0, C = 0;
    size_t end = row_group_extent(list, i, R, C), done = 0;
    for (; end >= i + 2 && !done; end--) {
      RowGroup g;
      if (!build_row_group(list, i, end, R, C, g)) continue;
      Plan plan;
      std::vector<int> params;
      std::string why;
      try {
        if (!plan_row_fusion(g.stages, g.bufs, R, C, opt, plan, params, why)) continue;
      } catch (const std::exception& e) { continue; }
      if (compile) {
        std::vector<char> cubin;
        std::string err;
        if (!nvrtc_compile(plan.source, cubin, err)) { put(message, message_len, err); return JAXCUDA_ECOMPILE; }
      }
      rep << i << "-" << end - 1 << ": " << plan.describe << " bytes=" << (long long)plan.algo_bytes << "\n";
      src << plan.source << "\n";
      done = end;
    }
    if (done) { i = done; continue; }
    {
      KernelIR composed;
      bool epilogue = false;
      if (composable_pair(list, i, composed, epilogue) >= 0) {
        try {
          Plan plan = make_plan(composed, opt);
          if (epilogue && (plan.skeleton != list[i].exe->plan.skeleton ||
                           plan.describe.substr(0, plan.describe.find(' ')) != list[i].exe->plan.describe.substr(0, list[i].exe->plan.describe.find(' '))))
            throw std::runtime_error("skeleton lost");
          if (compile) {
            std::vector<char> cubin;
            std::string err;
            if (!nvrtc_compile(plan.source, cubin, err)) { put(message, message_len, err); return JAXCUDA_ECOMPILE; }
          }
          rep << i << "-" << i + 1 << ": " << plan.describe << (epilogue ? " (consumer in the epilogue)" : " (producer substituted)") << " bytes=" << (long long)plan.algo_bytes << "\n";
          src << plan.source << "\n";
          i += 2;
          continue;
        } catch (const std::exception&) {}
      }
    }
    if (const size_t bend = small_batch_extent(list, i)) {
      SmallBatch b;
      build_small_batch(list, i, bend, b);
      Plan plan;
      std::string why;
      bool ok = false;
      try { ok = plan_small_batch(b.stages, (int)b.params.size(), opt, plan, why); } catch (const std::exception&) {}
      if (ok && compile) {
        std::vector<char> cubin;
        std::string err;
        if (!nvrtc_compile(plan.source, cubin, err)) { put(message, message_len, err); return JAXCUDA_ECOMPILE; }
      }
      if (ok) {
        rep << i << "-" << bend - 1 << ": " << plan.describe << " bytes=" << (long long)plan.algo_bytes << "\n";
        src << plan.source << "\n";
        i = bend;
        continue;
      }
    }
    try {
      Plan plan = make_plan(list[i].exe->ir, opt);
      rep << i << ": " << plan.describe << " bytes=" << (long long)plan.algo_bytes << "\n";
    } catch (const std::exception& e) {
      put(message, message_len, e.what());
      return JAXCUDA_EUNSUPPORTED;
    }
    i++;
  }
  put(report, report_len, rep.str());
  if (!compile) put(message, message_len, src.str());
  return JAXCUDA_OK;
}

int jaxcuda_exe_release(jaxcuda_exe* exe) {
  if (exe && exe->handles > 0) exe->handles--;
  return JAXCUDA_OK;
}

const char* jaxcuda_exe_describe(jaxcuda_exe* exe) { return exe ? exe->describe.c_str() : ""; }
const char* jaxcuda_exe_source(jaxcuda_exe* exe) { return exe ? exe->plan.source.c_str() : ""; }
int jaxcuda_exe_cost(jaxcuda_exe* exe, double* algo_bytes, double* algo_flops, int* n_launches) {
  if (!exe) return JAXCUDA_EINVAL;
  if (algo_bytes) *algo_bytes = exe->plan.algo_bytes;
  if (algo_flops) *algo_flops = exe->plan.algo_flops;
  if (n_launches) *n_launches = exe->kind ? 1 : (int)exe->plan.stages.size();
  return JAXCUDA_OK;
}

int jaxcuda_host_alloc(jaxcuda_ctx* ctx, size_t bytes, void** out) {
  if (!ctx || !out) return JAXCUDA_EINVAL;
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
  return JAXCUDA_OK;
}
int jaxcuda_host_free(jaxcuda_ctx* ctx, void* ptr) {
  if (!ctx) return JAXCUDA_EINVAL;
  if (ptr) CUDA_TRY(ctx, cudaFreeHost(ptr));
  return JAXCUDA_OK;
}

int jaxcuda_sync(jaxcuda_ctx* ctx) {
  if (!ctx) return JAXCUDA_EINVAL;
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "sync inside a capture");
  cudaSetDevice(ctx->device);
  if (int rc = jaxcuda_comm_join(ctx)) return rc;
  if (ctx->tc_dispatched) {  // only contexts that ran the tensor-core skeleton have anything to report
    CUDA_TRY(ctx, cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    ctx->tc_dispatched = false;
  }
  CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  return check_device_status(ctx);
}

int jaxcuda_event_record(jaxcuda_ctx* ctx, int index) {
  if (!ctx || index < 0 || index >= 65536) return JAXCUDA_EINVAL;
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "event_record inside a capture");
  cudaSetDevice(ctx->device);
  if ((size_t)index >= ctx->events.size()) ctx->events.resize(index + 1, nullptr);
  if (!ctx->events[index]) CUDA_TRY(ctx, cudaEventCreate(&ctx->events[index]));
  if (int rc = jaxcuda_comm_join(ctx)) return rc;  // an interval covers the sums begun inside it
  CUDA_TRY(ctx, cudaEventRecord(ctx->events[index], ctx->stream));
  return JAXCUDA_OK;
}
int jaxcuda_event_elapsed_ms(jaxcuda_ctx* ctx, int a, int b, float* ms) {
  const int n = ctx ? (int)ctx->events.size() : 0;
  if (!ctx || a < 0 || a >= n || b < 0 || b >= n || !ctx->events[a] || !ctx->events[b] || !ms) return JAXCUDA_EINVAL;
  CUDA_TRY(ctx, cudaEventSynchronize(ctx->events[b]));
  CUDA_TRY(ctx, cudaEventElapsedTime(ms, ctx->events[a], ctx->events[b]));
  return JAXCUDA_OK;
}
uint64_t jaxcuda_launch_count(jaxcuda_ctx* ctx) { return ctx ? ctx->launches : 0; }

// ---- checked build --------------------------------------------------------------------------
int jaxcuda_checked_counts(jaxcuda_ctx* ctx, uint64_t* allowed_outside, uint64_t* proven_outside) {
  if (!ctx) return JAXCUDA_EINVAL;
  if (!ctx->oob_dev) return fail(ctx, JAXCUDA_EINVAL, "not a checked build: create the context with JAXCUDA_CHECKED=1 in the environment");
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "checked_counts inside a capture");
  cudaSetDevice(ctx->device);
  if (int rc = jaxcuda_sync(ctx)) return rc;
  unsigned words[2] = {0, 0};
  CUDA_TRY(ctx, cudaMemcpy(words, ctx->oob_dev, sizeof words, cudaMemcpyDeviceToHost));
  CUDA_TRY(ctx, cudaMemset(ctx->oob_dev, 0, sizeof words));
  if (allowed_outside) *allowed_outside = words[0];
  if (proven_outside) *proven_outside = words[1];
  return JAXCUDA_OK;
}

// ---- tracing ------------------------------------------------------------------------------
int jaxcuda_trace_start(jaxcuda_ctx* ctx) {
  if (!ctx) return JAXCUDA_EINVAL;
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "trace_start inside a capture");
  cudaSetDevice(ctx->device);
  if (!ctx->trace_origin) CUDA_TRY(ctx, cudaEventCreate(&ctx->trace_origin));
  ctx->trace.clear();
  ctx->trace_events_used = 0;
  CUDA_TRY(ctx, cudaEventRecord(ctx->trace_origin, ctx->stream));
  ctx->tracing = true;
  return JAXCUDA_OK;
}
int jaxcuda_trace_stop(jaxcuda_ctx* ctx, int* n_records) {
  if (!ctx) return JAXCUDA_EINVAL;
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "trace_stop inside a capture");
  ctx->tracing = false;
  cudaSetDevice(ctx->device);
  if (!ctx->trace.empty()) CUDA_TRY(ctx, cudaEventSynchronize(ctx->trace.back().end));
  if (n_records) *n_records = (int)ctx->trace.size();
  return JAXCUDA_OK;
}
int jaxcuda_trace_record(jaxcuda_ctx* ctx, int index, jaxcuda_exe** exe, double* start_ms, double* duration_ms,
                         char* name, size_t name_len) {
  if (!ctx || index < 0 || (size_t)index >= ctx->trace.size() || ctx->tracing) return JAXCUDA_EINVAL;
  const jaxcuda_ctx::TraceRec& r = ctx->trace[index];
  cudaSetDevice(ctx->device);
  float t0 = 0, dt = 0;
  CUDA_TRY(ctx, cudaEventSynchronize(r.end));
  CUDA_TRY(ctx, cudaEventElapsedTime(&t0, ctx->trace_origin, r.begin));
  CUDA_TRY(ctx, cudaEventElapsedTime(&dt, r.begin, r.end));
  if (exe) *exe = r.exe;
  if (start_ms) *start_ms = t0;
  if (duration_ms) *duration_ms = dt;
  if (name && name_len) snprintf(name, name_len, "%s", r.name.c_str());
  return JAXCUDA_OK;
}

// ---- captured step lists ------------------------------------------------------------------
int jaxcuda_copy(jaxcuda_ctx* ctx, jaxcuda_slot dst, jaxcuda_slot src) {
  SlotRec* d = find_slot(ctx, dst);
  if (!d) return slot_error(ctx, dst);
  SlotRec* s = find_slot(ctx, src);
  if (!s) return slot_error(ctx, src);
  if (d->bytes != s->bytes) return fail(ctx, JAXCUDA_EINVAL, "copy between slots of %zu and %zu bytes", s->bytes, d->bytes);
  cudaSetDevice(ctx->device);
  if (int rc = flush_pending(ctx)) return rc;
  if (int rc = order_after_users(ctx, d)) return rc;
  drop_lo_plane(ctx, d->ptr);
  if (d->bytes && d->ptr != s->ptr)
    CUDA_TRY(ctx, cudaMemcpyAsync(d->ptr, s->ptr, d->bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return JAXCUDA_OK;
}

int jaxcuda_capture_begin(jaxcuda_ctx* ctx) {
  if (!ctx) return JAXCUDA_EINVAL;
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "a capture is already open");
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  // relaxed mode: the allocator may still call cudaMalloc for a size it has never seen
  CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  ctx->alloc.capturing = ctx->next_graph_id++;
  ctx->capture_launches0 = ctx->launches;
  ctx->capture_bytes = 0;
  ctx->capture_groups = 0;
  ctx->pending.clear();
  return JAXCUDA_OK;
}

int jaxcuda_capture_end(jaxcuda_ctx* ctx, jaxcuda_graph** out) {
  if (!ctx || !out) return JAXCUDA_EINVAL;
  *out = nullptr;
  if (!ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "no capture is open");
  const int flush_rc = flush_pending(ctx);
  drop_all_lo_planes(ctx);   // (graph-owned blocks: they return to the graph's own pool)
  jaxcuda_comm_join(ctx);  // a forked stream must rejoin before the capture closes
  const int id = ctx->alloc.capturing;
  ctx->alloc.capturing = 0;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
  if (e != cudaSuccess || !graph) {
    ctx->alloc.release_graph(id);
    return fail(ctx, JAXCUDA_ECUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
  }
  if (flush_rc) {
    cudaGraphDestroy(graph);
    ctx->alloc.release_graph(id);
    return flush_rc;
  }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(graph);
    ctx->alloc.release_graph(id);
    return fail(ctx, JAXCUDA_ECUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  }
  jaxcuda_graph* g = new jaxcuda_graph;
  g->ctx = ctx; g->id = id; g->graph = graph; g->exec = exec;
  g->kernels = ctx->launches - ctx->capture_launches0;
  g->algo_bytes = ctx->capture_bytes;
  g->fused_groups = ctx->capture_groups;
  ctx->launches = ctx->capture_launches0;  // nothing has run yet: launches count when the graph does
  *out = g;
  return JAXCUDA_OK;
}

int jaxcuda_graph_launch(jaxcuda_ctx* ctx, jaxcuda_graph* g) {
  if (!ctx || !g || g->ctx != ctx) return JAXCUDA_EINVAL;
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "graph launch inside a capture");
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launches += g->kernels;
  ctx->tc_dispatched = true;
  return JAXCUDA_OK;
}

int jaxcuda_graph_cost(jaxcuda_graph* g, uint64_t* launches, double* algo_bytes, int* fused_groups) {
  if (!g) return JAXCUDA_EINVAL;
  if (launches) *launches = g->kernels;
  if (algo_bytes) *algo_bytes = g->algo_bytes;
  if (fused_groups) *fused_groups = g->fused_groups;
  return JAXCUDA_OK;
}

int jaxcuda_graph_destroy(jaxcuda_ctx* ctx, jaxcuda_graph* g) {
  if (!ctx || !g || g->ctx != ctx) return JAXCUDA_EINVAL;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  ctx->alloc.release_graph(g->id);
  delete g;
  return JAXCUDA_OK;
}

int jaxcuda_slot_ptr(jaxcuda_ctx* ctx, jaxcuda_slot slot, uint64_t* device_ptr) {
  SlotRec* s = find_slot(ctx, slot);
  if (!s) return slot_error(ctx, slot);
  *device_ptr = (uint64_t)(uintptr_t)s->ptr;
  return JAXCUDA_OK;
}
uint64_t jaxcuda_stream(jaxcuda_ctx* ctx) { return ctx ? (uint64_t)(uintptr_t)ctx->stream : 0; }

// ---- NCCL ------------------------------------------------------------------------------
// Minimal prototypes of the NCCL C API (nccl.h), bound at run time.
typedef struct { char internal[128]; } jx_nccl_uid;
typedef int (*nccl_get_uid_t)(jx_nccl_uid*);
typedef int (*nccl_init_rank_t)(void**, int, jx_nccl_uid, int);
typedef int (*nccl_allreduce_t)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*nccl_destroy_t)(void*);
typedef int (*nccl_group_t)(void);
typedef const char* (*nccl_errstr_t)(int);
typedef int (*nccl_async_err_t)(void*, int*);

static void* nccl_handle(jaxcuda_ctx* ctx) {
  static void* h = nullptr;
  if (!h) {
    const char* override_ = getenv("JAXCUDA_NCCL_LIB");
    if (override_) h = dlopen(override_, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  }
  if (!h && ctx) ctx->last_error = std::string("NCCL library not found: ") + dlerror();
  return h;
}

int jaxcuda_comm_unique_id(void* id128) {
  void* h = nccl_handle(nullptr);
  if (!h || !id128) return JAXCUDA_ECUDA;
  auto fn = (nccl_get_uid_t)dlsym(h, "ncclGetUniqueId");
  if (!fn) return JAXCUDA_ECUDA;
  return fn((jx_nccl_uid*)id128) == 0 ? JAXCUDA_OK : JAXCUDA_ECUDA;
}

int jaxcuda_comm_init(jaxcuda_ctx* ctx, int rank, int nranks, const void* id128) {
  if (!ctx || !id128 || nranks < 1 || rank < 0 || rank >= nranks) return JAXCUDA_EINVAL;
  void* h = nccl_handle(ctx);
  if (!h) return JAXCUDA_ECUDA;
  auto init = (nccl_init_rank_t)dlsym(h, "ncclCommInitRank");
  auto errstr = (nccl_errstr_t)dlsym(h, "ncclGetErrorString");
  if (!init) return fail(ctx, JAXCUDA_ECUDA, "ncclCommInitRank not found");
  cudaSetDevice(ctx->device);
  jx_nccl_uid uid;
  memcpy(&uid, id128, sizeof uid);
  int r = init(&ctx->comm, nranks, uid, rank);
  if (r != 0) return fail(ctx, JAXCUDA_ECUDA, "ncclCommInitRank: %s", errstr ? errstr(r) : "error");
  ctx->nccl_lib = h;
  ctx->nranks = nranks;
  return JAXCUDA_OK;
}

static int allreduce_on(jaxcuda_ctx* ctx, const jaxcuda_slot* slots, int n, cudaStream_t stream);

int jaxcuda_allreduce_sum_f32(jaxcuda_ctx* ctx, const jaxcuda_slot* slots, int n) {
  if (!ctx || (n > 0 && !slots)) return JAXCUDA_EINVAL;
  if (!ctx->comm) {
    if (ctx->nranks == 1) return JAXCUDA_OK;  // a single rank: the sum is the input
    return fail(ctx, JAXCUDA_EINVAL, "communicator not initialised");
  }
  if (int rc = flush_pending(ctx)) return rc;
  if (int rc = jaxcuda_comm_join(ctx)) return rc;  // keep NCCL calls of this rank in one order
  return allreduce_on(ctx, slots, n, ctx->stream);
}

// The same sum issued on a second stream, so that it runs under the kernels dispatched after it
// (a gradient leaf is summed while the layers below it are still being differentiated).  The sum
// starts after everything dispatched so far; nothing dispatched later waits for it until
// jaxcuda_comm_join, which the caller issues before the first use of the summed slots.  The slots
// must stay alive until then.
int jaxcuda_allreduce_sum_f32_async(jaxcuda_ctx* ctx, const jaxcuda_slot* slots, int n) {
  if (!ctx || (n > 0 && !slots)) return JAXCUDA_EINVAL;
  if (!ctx->comm) {
    if (ctx->nranks == 1) return JAXCUDA_OK;
    return fail(ctx, JAXCUDA_EINVAL, "communicator not initialised");
  }
  cudaSetDevice(ctx->device);
  if (!ctx->comm_stream) {
    int least = 0, greatest = 0;  // the sum's CTAs go first when SMs free up: it is the longer pole
    CUDA_TRY(ctx, cudaDeviceGetStreamPriorityRange(&least, &greatest));
    CUDA_TRY(ctx, cudaStreamCreateWithPriority(&ctx->comm_stream, cudaStreamNonBlocking,
                                               env_int("JAXCUDA_COMM_PRIORITY", 1) ? greatest : least));
    CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->comm_fork, cudaEventDisableTiming));
    CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->comm_done, cudaEventDisableTiming));
  }
  if (int rc = flush_pending(ctx)) return rc;
  CUDA_TRY(ctx, cudaEventRecord(ctx->comm_fork, ctx->stream));
  CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->comm_stream, ctx->comm_fork, 0));
  ctx->comm_pending = true;
  for (int i = 0; i < n; i++)
    if (SlotRec* r = find_slot(ctx, slots[i])) ctx->comm_ptrs.insert(r->ptr);
  if (int rc = allreduce_on(ctx, slots, n, ctx->comm_stream)) return rc;
  if (ctx->comm_events_used == ctx->comm_events.size()) {
    cudaEvent_t ev;
    CUDA_TRY(ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    ctx->comm_events.push_back(ev);
  }
  cudaEvent_t done = ctx->comm_events[ctx->comm_events_used++];
  CUDA_TRY(ctx, cudaEventRecord(done, ctx->comm_stream));
  for (int i = 0; i < n; i++)
    if (SlotRec* r = find_slot(ctx, slots[i])) ctx->comm_ptr_event[r->ptr] = done;
  return JAXCUDA_OK;
}

int jaxcuda_comm_join(jaxcuda_ctx* ctx) {
  if (!ctx) return JAXCUDA_EINVAL;
  if (!ctx->comm_pending) return JAXCUDA_OK;
  cudaSetDevice(ctx->device);
  if (int rc = flush_pending(ctx)) return rc;
  CUDA_TRY(ctx, cudaEventRecord(ctx->comm_done, ctx->comm_stream));
  CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->comm_done, 0));
  ctx->comm_pending = false;
  ctx->comm_ptrs.clear();
  ctx->comm_ptr_event.clear();
  ctx->comm_events_used = 0;
  return JAXCUDA_OK;
}

static int allreduce_on(jaxcuda_ctx* ctx, const jaxcuda_slot* slots, int n, cudaStream_t stream) {
  auto allreduce = (nccl_allreduce_t)dlsym(ctx->nccl_lib, "ncclAllReduce");
  auto gstart = (nccl_group_t)dlsym(ctx->nccl_lib, "ncclGroupStart");
  auto gend = (nccl_group_t)dlsym(ctx->nccl_lib, "ncclGroupEnd");
  auto errstr = (nccl_errstr_t)dlsym(ctx->nccl_lib, "ncclGetErrorString");
  if (!allreduce || !gstart || !gend) return fail(ctx, JAXCUDA_ECUDA, "NCCL symbols missing");
  cudaSetDevice(ctx->device);
  for (int i = 0; i < n; i++) if (!find_slot(ctx, slots[i])) return slot_error(ctx, slots[i]);
  for (int i = 0; i < n; i++) drop_lo_plane(ctx, find_slot(ctx, slots[i])->ptr);   // summed in place
  gstart();
  int r = 0;
  for (int i = 0; i < n && r == 0; i++) {
    SlotRec* s = find_slot(ctx, slots[i]);
    if (s->bytes) r = allreduce(s->ptr, s->ptr, s->bytes / 4, /*ncclFloat32*/ 7, /*ncclSum*/ 0, ctx->comm, stream);
  }
  int r2 = gend();
  if (r == 0) r = r2;
  if (r != 0) return fail(ctx, JAXCUDA_ECUDA, "ncclAllReduce: %s", errstr ? errstr(r) : "error");
  return JAXCUDA_OK;
}

// Asynchronous error state of the communicator (ncclCommGetAsyncError).  A communicator that reports
// an error is aborted (ncclCommAbort returns without waiting for the peers, and ends the NCCL kernels
// of this rank that still wait for them) and the context goes back to "no communicator".
static int poll_comm(jaxcuda_ctx* ctx) {
  if (!ctx->comm) return JAXCUDA_OK;
  auto async_err = (nccl_async_err_t)dlsym(ctx->nccl_lib, "ncclCommGetAsyncError");
  if (!async_err) return JAXCUDA_OK;
  int state = 0;
  int r = async_err(ctx->comm, &state);
  if (r == 0 && (state == 0 || state == /*ncclInProgress*/ 7)) return JAXCUDA_OK;
  auto errstr = (nccl_errstr_t)dlsym(ctx->nccl_lib, "ncclGetErrorString");
  const int code = r != 0 ? r : state;
  std::string what = errstr ? errstr(code) : "error";
  jaxcuda_comm_abort(ctx);
  return fail(ctx, JAXCUDA_ECUDA, "NCCL communicator failed (%s) and was aborted", what.c_str());
}

int jaxcuda_comm_abort(jaxcuda_ctx* ctx) {
  if (!ctx) return JAXCUDA_EINVAL;
  if (!ctx->comm) return JAXCUDA_OK;
  auto abort_ = (nccl_destroy_t)dlsym(ctx->nccl_lib, "ncclCommAbort");
  if (abort_) abort_(ctx->comm);
  ctx->comm = nullptr;
  ctx->nranks = 0;   // sums now fail with "communicator not initialised" instead of passing as one rank
  return JAXCUDA_OK;
}

int jaxcuda_comm_wait(jaxcuda_ctx* ctx, int timeout_ms) {
  if (!ctx || timeout_ms < 0) return JAXCUDA_EINVAL;
  if (ctx->alloc.capturing) return fail(ctx, JAXCUDA_EINVAL, "comm_wait inside a capture");
  cudaSetDevice(ctx->device);
  if (int rc = flush_pending(ctx)) return rc;
  if (!ctx->wait_compute) {
    CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->wait_compute, cudaEventDisableTiming));
    CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->wait_comm, cudaEventDisableTiming));
  }
  CUDA_TRY(ctx, cudaEventRecord(ctx->wait_compute, ctx->stream));
  if (ctx->comm_stream) CUDA_TRY(ctx, cudaEventRecord(ctx->wait_comm, ctx->comm_stream));
  const auto t0 = std::chrono::steady_clock::now();
  for (int spins = 0;; spins++) {
    cudaError_t a = cudaEventQuery(ctx->wait_compute);
    cudaError_t b = ctx->comm_stream ? cudaEventQuery(ctx->wait_comm) : cudaSuccess;
    if (a != cudaSuccess && a != cudaErrorNotReady) return fail(ctx, JAXCUDA_ECUDA, "comm_wait: %s", cudaGetErrorString(a));
    if (b != cudaSuccess && b != cudaErrorNotReady) return fail(ctx, JAXCUDA_ECUDA, "comm_wait: %s", cudaGetErrorString(b));
    if (int rc = poll_comm(ctx)) return rc;
    if (a == cudaSuccess && b == cudaSuccess) return JAXCUDA_OK;
    const auto waited = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
    if (waited >= (long long)timeout_ms * 1000)
      return fail(ctx, JAXCUDA_ETIMEOUT, "work issued before comm_wait has not finished after %d ms", timeout_ms);
    if (spins > 200) std::this_thread::sleep_for(std::chrono::microseconds(100));
  }
}

int jaxcuda_comm_destroy(jaxcuda_ctx* ctx) {
  if (!ctx || !ctx->comm) return JAXCUDA_OK;
  auto destroy = (nccl_destroy_t)dlsym(ctx->nccl_lib, "ncclCommDestroy");
  if (destroy) destroy(ctx->comm);
  ctx->comm = nullptr;
  return JAXCUDA_OK;
}

}  // extern "C"

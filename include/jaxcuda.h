/*
 * C ABI of libjaxcuda.so: the B200 `cuda` device backend for jax-js.
 *
 * Each entry point stands behind one method of the reference's `Backend` interface
 * (src/backend.ts:158-211); the TypeScript class that implements that interface calls
 * these through a Node addon (jax_js_b200/ts/addon.cc).  Plain pointers and sizes only.
 *
 * Every call returns a jaxcuda_status; on failure jaxcuda_last_error(ctx) holds a
 * message (NVRTC logs and the generated source included for compile errors, as the
 * reference surfaces shader compile errors, src/backend/webgpu.ts:778-792).
 *
 * Threading: one host thread drives a context at a time (the reference's backends are
 * driven from the single JS thread).  All device work of a context is ordered on one
 * stream: dispatch order is execution order (src/backend.ts:203-210).
 */
#ifndef JAXCUDA_H
#define JAXCUDA_H

#include <stddef.h>
#include <stdint.h>

#include "jaxcuda_ir.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  JAXCUDA_OK = 0,
  JAXCUDA_ESLOT = 1,        /* SlotError: slot invalid or already freed (src/backend.ts:222-226) */
  JAXCUDA_EUNSUPPORTED = 2, /* UnsupportedOpError / UnsupportedRoutineError (src/backend.ts:228-240) */
  JAXCUDA_EINVAL = 3,       /* plain Error: size mismatch, bad image, bad range (src/backend/cpu.ts:21-24) */
  JAXCUDA_ECOMPILE = 4,     /* NVRTC rejected generated source */
  JAXCUDA_ECUDA = 5,        /* a CUDA or NCCL call failed */
  JAXCUDA_ENOMEM = 6,
  JAXCUDA_ETIMEOUT = 7      /* jaxcuda_comm_wait: the work is still running; nothing was cancelled */
} jaxcuda_status;

typedef struct jaxcuda_ctx jaxcuda_ctx;
typedef struct jaxcuda_exe jaxcuda_exe;
typedef struct jaxcuda_graph jaxcuda_graph;
typedef uint32_t jaxcuda_slot; /* `Slot`, src/backend.ts:155 */

/* createBackend("cuda") arm (src/backend.ts:72-142): binds a context to one GPU and creates
 * its stream.  Fails with JAXCUDA_ECUDA when no usable GPU or driver is present: there is no
 * CPU fallback. */
int jaxcuda_create(int device, jaxcuda_ctx** out);
int jaxcuda_destroy(jaxcuda_ctx* ctx);
const char* jaxcuda_last_error(jaxcuda_ctx* ctx); /* ctx may be NULL: error of the last failed create */

/* Backend.maxArgs (src/backend.ts:163; the Wasm backend's value, src/backend/wasm.ts:38). */
int jaxcuda_max_args(void);

/* Backend.malloc (src/backend.ts:166-171): new slot with reference count 1.  `init` may be NULL;
 * otherwise `init_bytes` must equal `bytes` (JAXCUDA_EINVAL, as src/backend/cpu.ts:21-24).
 * bytes == 0 is legal (src/backend/webgpu.ts:84-86). */
int jaxcuda_malloc(jaxcuda_ctx* ctx, size_t bytes, const void* init, size_t init_bytes, jaxcuda_slot* out);
/* Backend.incRef / decRef (src/backend.ts:173-180).  decRef of a dead slot is JAXCUDA_ESLOT. */
int jaxcuda_incref(jaxcuda_ctx* ctx, jaxcuda_slot slot);
int jaxcuda_decref(jaxcuda_ctx* ctx, jaxcuda_slot slot);
/* Backend.read / readSync (src/backend.ts:182-190): copies bytes [start, start+count) to dst after
 * all dispatched work has finished.  count == SIZE_MAX means "to the end"; count == 0 is a pure
 * barrier (src/frontend/array.ts:827). */
int jaxcuda_read(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t start, size_t count, void* dst);
/* Upload into an existing slot (the H2D half of malloc(initialData), for callers that reuse
 * slots between steps instead of reallocating; the Wasm backend writes through its memory view,
 * src/backend/wasm.ts:57-75). */
int jaxcuda_write(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t start, size_t count, const void* src);
/* Backend.read as the reference declares it, returning a Promise (src/backend.ts:182-186): the copy
 * of bytes [start, start+count) to dst is enqueued on a copy stream of its own, after everything
 * dispatched so far, and the call returns.  jaxcuda_read_wait(ticket) is where the Promise resolves.
 * dst must be pinned memory (jaxcuda_host_alloc).  The slot may be released, written or dispatched
 * into before the wait returns: the runtime orders whatever touches its memory next behind the copy.
 * Uploads, kernels and downloads of consecutive steps then overlap.  read_wait also reports a
 * tensor-core kernel that abandoned a bounded wait, as jaxcuda_read and jaxcuda_sync do. */
int jaxcuda_read_async(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t start, size_t count, void* dst, uint64_t* ticket);
int jaxcuda_read_wait(jaxcuda_ctx* ctx, uint64_t ticket);
/* For callers that wait on another thread (the Promise of a Node-API addon): one host thread drives
 * a context at a time, so a worker thread must not enter the calls above.  jaxcuda_read_event gives,
 * on the driving thread, the event behind a ticket; jaxcuda_event_block waits for it from any thread
 * and touches no context state; jaxcuda_read_wait on the driving thread then returns at once and
 * retires the ticket. */
int jaxcuda_read_event(jaxcuda_ctx* ctx, uint64_t ticket, void** event);
int jaxcuda_event_block(void* event);
/* How often the compute stream had to be ordered behind a download or a sum that still used a slot
 * which was being released, written or dispatched into (diagnostic). */
uint64_t jaxcuda_order_waits(jaxcuda_ctx* ctx);
/* jaxcuda_write on a copy stream: starts after everything dispatched so far (earlier kernels may
 * still read the slot); everything dispatched afterwards waits for it.  src must be pinned and
 * unchanged until a later read_wait or sync has returned. */
int jaxcuda_write_async(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t start, size_t count, const void* src);
int jaxcuda_slot_size(jaxcuda_ctx* ctx, jaxcuda_slot slot, size_t* bytes);

/* Backend.prepareKernel[Sync] (src/backend.ts:192-196).  `ir` is the lowered Kernel image of
 * jaxcuda_ir.h; `hash` is the caller's cache key (FpHash of the Kernel, src/backend/wasm.ts:126),
 * 0 to let the library hash the image.  Compiles with NVRTC on a cache miss. */
int jaxcuda_prepare_kernel(jaxcuda_ctx* ctx, const uint8_t* ir, size_t len, uint64_t hash, jaxcuda_exe** out);

/* Diagnostic that needs no GPU: parse, choose the skeleton and (compile != 0) run NVRTC for
 * sm_100a.  Writes the plan description to `describe`; `message` receives the error text, or,
 * when compile == 0, the generated CUDA C.  force_skeleton < 0 lets the planner choose.
 * Used by CPU-side tests of the code generator; no counterpart in the reference. */
int jaxcuda_check_kernel(const uint8_t* ir, size_t len, int sm_count, int force_skeleton, int compile,
                         char* describe, size_t describe_len, char* message, size_t message_len);

/* `RoutineType` (src/routine.ts:112-123) flattened: shapes are concatenated, ranks give the split. */
typedef struct {
  int n_inputs, n_outputs;
  const int32_t* input_dtypes;  /* jaxcuda_dtype per input */
  const int32_t* input_ranks;
  const int64_t* input_shapes;  /* all input shapes, concatenated */
  const int32_t* output_dtypes;
  const int32_t* output_ranks;
  const int64_t* output_shapes;
} jaxcuda_routine_type;

/* Backend.prepareRoutine[Sync] (src/backend.ts:198-202).  name is a `Routines` member
 * (src/routine.ts:32-102): every member is implemented ("Sort", "Argsort", "Scatter", "TriangularSolve",
 * "Cholesky", "LU", "JacobiEigh", "Fft"); any other name returns JAXCUDA_EUNSUPPORTED
 * (UnsupportedRoutineError).  params_json is the routine's `params` object as JSON (Scatter:
 * `ScatterParams`, src/routine.ts:104-110; TriangularSolve: {"unitDiagonal": bool}; JacobiEigh:
 * {"maxSweeps": int, "tolerance": number}; Fft: {"factors": [int...], "inverse": bool}).  Shapes the reference rejects
 * (src/routine.ts:305-313, :341-346) return JAXCUDA_EINVAL with its message.
 * Size limits, checked here (JAXCUDA_EUNSUPPORTED with the limit in the message), never at
 * dispatch: the sorted axis and every matrix dimension below 2^31; TriangularSolve n <= 25600;
 * JacobiEigh n <= 32768; Cholesky of n >= 256 in batches of at most 65535 matrices, n <= 2^30;
 * at most 2^31-1 matrices per call.  Sort/Argsort, Scatter and Fft have no limit besides memory
 * (work space comes from the allocator at dispatch: JAXCUDA_ENOMEM). */
int jaxcuda_prepare_routine(jaxcuda_ctx* ctx, const char* name, const jaxcuda_routine_type* type,
                            const char* params_json, jaxcuda_exe** out);

/* Backend.dispatch (src/backend.ts:204-211): enqueue only; runs in dispatch order. */
int jaxcuda_dispatch(jaxcuda_ctx* ctx, jaxcuda_exe* exe, const jaxcuda_slot* inputs, int n_inputs,
                     const jaxcuda_slot* outputs, int n_outputs);
/* Executables are owned by the context's cache; release drops the caller's handle. */
int jaxcuda_exe_release(jaxcuda_exe* exe);

/* What the backend decided for an executable (setDebug(4) prints the same for WebGPU tuning,
 * src/tuner.ts:250): skeleton name and launch shape, generated CUDA C, algorithmic bytes/flops. */
const char* jaxcuda_exe_describe(jaxcuda_exe* exe);
const char* jaxcuda_exe_source(jaxcuda_exe* exe);
int jaxcuda_exe_cost(jaxcuda_exe* exe, double* algo_bytes, double* algo_flops, int* n_launches);

/* Pinned host staging memory for callers that time host<->device transfers. */
int jaxcuda_host_alloc(jaxcuda_ctx* ctx, size_t bytes, void** out);
int jaxcuda_host_free(jaxcuda_ctx* ctx, void* ptr);

/* Barrier: wait for everything dispatched so far (read(slot, 0, 0) without a slot). */
int jaxcuda_sync(jaxcuda_ctx* ctx);

/* Device timing of a dispatch sequence on the context's stream (the cuda counterpart of the
 * WebGPU timestamp queries, src/backend/webgpu/tracing.ts:11-164): records an event now. */
int jaxcuda_event_record(jaxcuda_ctx* ctx, int index); /* index in [0, 65536) */
int jaxcuda_event_elapsed_ms(jaxcuda_ctx* ctx, int start_index, int stop_index, float* ms);

/* Checked build (the pool's memory checker cannot be run on these kernels, so the library checks
 * itself).  With JAXCUDA_CHECKED=1 in the environment when the process first creates a context,
 * every scalar load of the generated kernels tests its index, also where the planner has proven
 * the range and the normal build tests nothing, and counts the indices outside the buffer.
 * jaxcuda_checked_counts waits for the stream, returns and resets the two counters:
 * allowed_outside, loads that the Kernel lets fall outside and that read element 0 as the
 * reference's Wasm backend does (src/backend/wasm/translation.ts:221-228); proven_outside, loads
 * that were proven in range and were not: any non-zero value is a bug of the planner.  Vector
 * loads and TMA are not instrumented (the planner takes them only for proven, contiguous ranges).  JAXCUDA_EINVAL in a
 * normal build. */
int jaxcuda_checked_counts(jaxcuda_ctx* ctx, uint64_t* allowed_outside, uint64_t* proven_outside);

/* Per-dispatch tracing: profiler.startTrace / stopTrace flip a flag (src/tracing.ts:15-33) and a
 * backend that sees it times every dispatch and reports it through emitTrace (src/tracing.ts:89-106;
 * the wasm backend around dispatch, src/backend/wasm.ts:172-173 and 266-269; the webgpu backend with
 * a timestamp pair per pass, src/backend/webgpu/tracing.ts:11-164).  Here: between trace_start and
 * trace_stop every eager jaxcuda_dispatch is bracketed by a pair of CUDA events on the context's
 * stream (at most 2^20 dispatches per trace; dispatches inside a capture are not timed one by one,
 * a replay is timed by its caller).  trace_stop waits for the last traced dispatch and returns
 * the number of records; trace_record gives record `index`: the executable, its start relative
 * to trace_start and its duration on the device, in milliseconds, and its plan (the text of
 * jaxcuda_exe_describe, valid even if the executable has been released since).  The records
 * stay until the next trace_start. */
int jaxcuda_trace_start(jaxcuda_ctx* ctx);
int jaxcuda_trace_stop(jaxcuda_ctx* ctx, int* n_records);
int jaxcuda_trace_record(jaxcuda_ctx* ctx, int index, jaxcuda_exe** exe, double* start_ms, double* duration_ms,
                         char* name, size_t name_len);
/* Number of kernels this context has launched so far (its own kernels only). */
uint64_t jaxcuda_launch_count(jaxcuda_ctx* ctx);

/* Replay of a static step list as one CUDA graph: the counterpart of `JitProgram.execute`
 * (src/frontend/jit.ts:111-162), which replays the same malloc / execute / free steps on every call.
 * Between capture_begin and capture_end the usual calls (malloc without initialData, dispatch,
 * incref/decref, copy, allreduce) are recorded instead of run; every buffer touched in between
 * belongs to the graph until it is destroyed, so slots that are still alive at capture_end (the
 * step's outputs) keep their addresses and are rewritten in place by every launch.  Dispatch each
 * program eagerly at least once before capturing it.  read / sync / event_record are refused
 * inside a capture.
 *
 * Because a captured list is in hand as a whole, runs of consecutive Kernels that walk the rows of
 * one [rows, cols] array (row reductions, elementwise Kernels over rows*cols and per-row Kernels,
 * the shape in which softmax, logsumexp and argmax arrive: src/library/nn.ts:291-345,
 * src/library/numpy.ts:533-556) are replaced by one row-resident kernel that reads every outside
 * array once and writes only the slots still alive when the run ends; a Kernel repeated on the same
 * arrays is computed once.  Results are those of the separate Kernels up to the summation order
 * of the row reductions.  Likewise an elementwise Kernel (a reduction of size 1 included) whose
 * output only the next Kernel reads, elementwise too, before the list releases it, is substituted
 * into that Kernel: the consumer evaluates the producer's expression at the index of its load and
 * the intermediate array is never written (a vmapped gradient's per-example products, which
 * arrive batch-last followed by the Kernel that moves the batch axis first,
 * src/frontend/vmap.ts:297-303); and an elementwise Kernel that reads a tensor-core GEMM's output at
 * gidx, as its only reader, runs as the tail of that GEMM's epilogue; and a run of three or more
 * Kernels of at most 16384 element evaluations each is recorded as one single-CTA kernel that
 * evaluates them in turn.  Same operations on the same values in the same order: same bits.
 * JAXCUDA_FUSE=0 in the environment turns both replacements off. */
int jaxcuda_capture_begin(jaxcuda_ctx* ctx);
int jaxcuda_capture_end(jaxcuda_ctx* ctx, jaxcuda_graph** out);
int jaxcuda_graph_launch(jaxcuda_ctx* ctx, jaxcuda_graph* graph);
int jaxcuda_graph_destroy(jaxcuda_ctx* ctx, jaxcuda_graph* graph);
/* What one launch of the graph does: kernels launched, their algorithmic bytes (distinct bytes each
 * kernel reads plus bytes it writes; a fused kernel counts its own), and how many runs were fused.
 * Any pointer may be null.  Plays the part of `JitProgram.toString()` (src/frontend/jit.ts:466). */
int jaxcuda_graph_cost(jaxcuda_graph* graph, uint64_t* launches, double* algo_bytes, int* fused_groups);
/* Device-to-device copy between two slots of equal size, in stream order (capturable). */
int jaxcuda_copy(jaxcuda_ctx* ctx, jaxcuda_slot dst, jaxcuda_slot src);

/* Diagnostic that needs no GPU: what a capture would launch for a list of n Kernels.  Kernel i has
 * n_inputs[i] entries of `inputs` (array ids, consecutive over the list) and writes array outputs[i];
 * output_freed[i] != 0 says that this output's slot is released before the capture ends (an
 * intermediate of the step list).  `report` receives one line per launch: the positions it covers
 * and its plan; `message` the error text or, when compile == 0, the CUDA C of the fused kernels.
 * Used by CPU-side tests; no counterpart in the reference. */
int jaxcuda_check_step_list(int n, const uint8_t* const* irs, const size_t* lens, const int* n_inputs, const int* inputs,
                            const int* outputs, const uint8_t* output_freed, int compile, char* report, size_t report_len,
                            char* message, size_t message_len);

/* Interop for host code that shares the CUDA primary context (torch): raw pointer of a slot and
 * the stream handle (cudaStream_t) as integers.  No counterpart in the reference. */
int jaxcuda_slot_ptr(jaxcuda_ctx* ctx, jaxcuda_slot slot, uint64_t* device_ptr);
uint64_t jaxcuda_stream(jaxcuda_ctx* ctx);

/* Data-parallel gradient sum.  No counterpart in the reference, which has no multi-device
 * support: one context per GPU and process, an NCCL communicator over them, and an in-place
 * f32 sum over the listed slots on the context's stream, ordered after prior dispatches. */
int jaxcuda_comm_unique_id(void* id128); /* fills 128 bytes (ncclUniqueId) on rank 0 */
int jaxcuda_comm_init(jaxcuda_ctx* ctx, int rank, int nranks, const void* id128);
int jaxcuda_allreduce_sum_f32(jaxcuda_ctx* ctx, const jaxcuda_slot* slots, int n);
/* The same sum on a second stream: it starts after everything dispatched so far and runs under
 * what is dispatched next.  jaxcuda_comm_join makes later dispatches wait for every sum begun
 * this way; read, sync, event_record and capture_end join by themselves, and so does releasing,
 * writing or dispatching into one of the slots (the runtime joins first, so the sum is never
 * overtaken).  A Kernel that only reads one of the slots before the join sees unsummed or
 * partly summed data: that ordering is the caller's. */
int jaxcuda_allreduce_sum_f32_async(jaxcuda_ctx* ctx, const jaxcuda_slot* slots, int n);
int jaxcuda_comm_join(jaxcuda_ctx* ctx);
int jaxcuda_comm_destroy(jaxcuda_ctx* ctx);
/* Failure detection for the sums.  A sum whose peer is late or gone never finishes, and a plain
 * read or sync behind it would block for ever.  jaxcuda_comm_wait blocks the host until
 * everything issued so far on the context's stream and on the sums' stream has finished, for at
 * most timeout_ms, and polls the communicator's asynchronous error state (ncclCommGetAsyncError)
 * meanwhile.  JAXCUDA_OK: all done.  JAXCUDA_ETIMEOUT: still running; nothing was cancelled, the
 * call may be repeated, or the caller gives up with jaxcuda_comm_abort.  JAXCUDA_ECUDA: NCCL
 * reported an error; the communicator has been aborted and later sums fail until
 * jaxcuda_comm_init is called again.  Not allowed inside a capture.
 * jaxcuda_comm_abort (ncclCommAbort) ends this rank's part of the communicator without waiting
 * for the peers: NCCL kernels of this rank that still wait for a peer return, so the context's
 * streams drain and the context stays usable. */
int jaxcuda_comm_wait(jaxcuda_ctx* ctx, int timeout_ms);
int jaxcuda_comm_abort(jaxcuda_ctx* ctx);

/* Sort along the last axis of a contiguous [batch, n] device array without allocating anything.
 * No counterpart in the reference.  It is for embedders that cannot let the library call
 * cudaMalloc (all device memory already belongs to their own pool, or the device-wide
 * synchronisation of an allocation is unacceptable inside a serving loop): the work buffer that
 * jaxcuda_dispatch would take from the allocator is a fixed 16 MiB array inside the library image.
 * x and y are device pointers (jaxcuda_slot_ptr), stream a cudaStream_t (jaxcuda_stream); the owning
 * device must be current.  Limit: batch * next_pow2(n) <= 4 Mi keys (rows up to 32768 keys never
 * touch the buffer); beyond it JAXCUDA_EINVAL with the reason in err.  The first call on a device
 * looks the buffer up and belongs outside any stream capture; all calls share the buffer, so calls
 * that overlap on the GPU race. */
int jaxcuda_sort_no_alloc(void* stream, int dtype, const void* x, void* y, int64_t batch, int64_t n,
                          char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* JAXCUDA_H */

// Skeleton choice and CUDA C generation for one lowered Kernel.
//
// A Kernel (src/alu.ts:1479) reaches the backend as an untagged expression DAG; this file
// decides which hand-written sm_100a skeleton it runs in and splices the DAG into it.
// It takes the place of `tuneWebgpu` + `pipelineSource` (src/tuner.ts:243-478,
// src/backend/webgpu.ts:285-530) and of the Wasm tile planner
// (src/backend/wasm/tilePlan.ts:278-334), re-derived for Blackwell.
#pragma once
#include <cstdlib>

#include <string>
#include <vector>

#include "ir.hpp"

namespace jaxcuda {

enum Skeleton {
  SK_ELEMENTWISE = 0,  // 128-bit vectorised streaming kernel
  SK_REDUCE_ROW = 1,   // lanes of a warp/CTA stride over ridx, shuffle + shared-memory tree
  SK_REDUCE_COL = 2,   // one thread per (vector of) outputs loops over ridx; optional split over ridx
  SK_GEMM_FFMA = 3,    // shared-memory tiled FFMA GEMM with spliced epilogue (any strides)
  SK_GEMM_TC = 4,      // TMA + tcgen05/TMEM GEMM (f16 operands, or f32 as 3xTF32)
};

// Strides are in elements.  C[b, m, n] = sum_k A[offA + b*sAb + m*sAm + k*sAk] * B[offB + b*sBb + n*sBn + k*sBk]
struct GemmDesc {
  bool valid = false;
  uint32_t gidA = 0, gidB = 0, dtA = 0, dtB = 0;
  uint64_t lenA = 0, lenB = 0;
  int64_t M = 0, N = 0, K = 0, batch = 1;
  int64_t offA = 0, sAm = 0, sAk = 0, sAb = 0;
  int64_t offB = 0, sBn = 0, sBk = 0, sBb = 0;
  bool round_product_f16 = false;  // body is Cast<f32>(Mul<f16>(a, b))
  // Convolutions: the B operand is not an argument but a [batch][K][b_pitch] array that a gather
  // stage of the same plan writes into the plan's scratch (with its 3xTF32 remainder plane behind
  // it); then gidB is unused, sBn = 1, sBk = b_pitch, sBb = K * b_pitch, offB = 0.
  bool b_gathered = false;
  int64_t b_pitch = 0;
  // ... or, with b_implicit as well, no array at all: warps of the GEMM kernel evaluate the patch
  // expression straight into the shared-memory stages (gemm_tc.cpp, B_GATHER).
  bool b_implicit = false;
};

struct Stage {
  std::string entry;
  unsigned grid[3] = {1, 1, 1};
  unsigned block[3] = {1, 1, 1};
  unsigned smem = 0;
  unsigned cluster = 1;   // CTAs per thread-block cluster along x (the paired tensor-core GEMM launches with 2)
};

struct Plan {
  int skeleton = SK_ELEMENTWISE;
  std::string source;        // complete CUDA C translation unit for NVRTC
  std::vector<Stage> stages;  // launched in order on the backend's stream
  size_t scratch_bytes = 0;   // global scratch shared by the stages (split reductions, TF32 planes)
  // The kernel takes a trailing `int jx_rev`: non-zero walks the grid from the last block to the
  // first.  Consecutive streaming kernels alternate, so that each starts on the part of the
  // previous kernel's data that is still in L2.
  bool takes_rev = false;
  bool scratch_persistent = false;  // scratch belongs to the executable and starts zeroed (arrival counters)
  std::string describe;       // one line: skeleton and launch shape
  GemmDesc gemm;
  double algo_bytes = 0;      // distinct input bytes addressed + output bytes
  double algo_flops = 0;      // 2*M*N*K for GEMM-shaped kernels, else size * K
  // tensor-core GEMM launch parameters (SK_GEMM_TC), filled by gemm_tc.cpp
  int tc_kind = 0;            // 1 f16, 2 3xTF32
  int tc_bm = 0, tc_bn = 0, tc_bk = 0, tc_stages = 0;
  bool tc_pair = false;          // CTA pairs (tcgen05 cta_group::2) on 256 x BN tiles
  bool tc_lo_in_kernel = false;  // 3xTF32 remainder tiles are made inside the GEMM kernel: no split stage, no planes in scratch
  size_t tc_sk_offset = 0, tc_sk_counter_bytes = 0;  // stream-K arrival counters inside the scratch (cleared per launch)
};

struct Options {
  int sm_count = 148;
  int ew_ilp = 2;             // independent 128-bit accesses in flight per thread (elementwise)
  int ew_blocks_per_sm = 4096;  // grid cap; at the default the grid covers the array in one pass
  int gemm_min_dim = 32;      // below this M or N a GEMM-shaped kernel stays on the reduce skeletons
  bool allow_tc = true;       // tcgen05 path allowed (JAXCUDA_NO_TC=1 clears it)
  int tc_bn = 0;              // force the tensor-core tile width (64, 128, 192, 256); 0 = planner's choice (JAXCUDA_TC_BN)
  int tc_streamk = 1;         // 0: whole tiles only; 1: an output with at most half as many tiles as SMs and a long K is cut along K; 2: so is any last wave that is at most half full (JAXCUDA_TC_STREAMK)
  int tc_pair = 1;            // CTA pairs on 256-row tiles (cta_group::2): 0 never, 1 f16 GEMMs, 2 3xTF32 as well (JAXCUDA_TC_PAIR)
  int tc_half_last = 1;       // CTA pairs: a last wave that is at most half full runs as half-width tiles: 0 never, 1 3xTF32, 2 f16 as well (JAXCUDA_TC_HALF_LAST)
  int tc_spin_limit = 20000000;  // polls of a tensor-core pipeline wait before it gives up (JAXCUDA_TC_SPIN_LIMIT)
  int tc_lo_in_kernel = 1;    // 3xTF32 remainder tiles derived in shared memory by warps of the GEMM kernel instead of a split pass through global memory: 0 never, 1 for outputs of at most one wave of tiles, 2 always (JAXCUDA_TC_LO_IN_KERNEL)
  int tc_fault = 0;           // tests of the wind-down only: 1 = one CTA's producer announces a stage and never loads it (JAXCUDA_TC_FAULT)
  int force_skeleton = -1;    // tests: force SK_REDUCE_ROW / SK_REDUCE_COL / SK_GEMM_FFMA
  int exact_math = -1;        // 1: bit-faithful exp everywhere, 0: fast everywhere, -1: exact below exact_math_work
  double exact_math_work = 1 << 20;  // element evaluations (size x K) under which a kernel is latency-bound anyway
  int ld_hint = -1;           // 1: 128-bit loads use ld.global.nc.L1::no_allocate.L2::256B; 0: plain loads; -1: per skeleton (column reduce only)
  int row_tpr = 0;            // threads per output row in the row-reduce skeleton (0: chosen from K)
  int row_unroll = 0;         // vector loads in flight per thread in the row-reduce loop (0: trip count, at most 4)
  int col_threads = 128;      // CTA size of the column-reduce skeleton
  int col_ctas_per_sm = 4;    // spread ridx over threads and CTAs until the grid holds this many 256-thread CTAs per SM
  int col_ty = 0;             // threads sharing one output vector inside a CTA (0: chosen)
  int col_unroll = 4;         // independent loads in flight per thread in the column-reduce loop
  int conv_implicit = 1;      // convolutions: 1 = the patch operand is gathered inside the GEMM kernel, 0 = by a stage of its own through global memory (JAXCUDA_CONV_IMPLICIT)
  int fuse_chunks = 0;        // 128-bit pieces of a row per thread in a row program (1, 2 or 4; 0: chosen)
  int fuse_min_ctas = 0;      // CTAs per SM the row program's register allocation is held to (0: compiler's choice)
};

// Throws std::runtime_error with the reference's UnsupportedOpError wording
// ("Op<dtype> not supported in cuda backend") for combinations that cannot be emitted.
Plan make_plan(const KernelIR& k, const Options& opt);

// ---- several Kernels of one step list as one row-resident kernel ---------------------------------
//
// `jit` hands over softmax, logsumexp or argmax over the last axis as chains of Kernels that all
// walk the same [rows, cols] array: row reductions (size rows, reduction size cols), elementwise
// Kernels over rows*cols elements and per-row Kernels over rows elements (src/library/nn.ts:291-345,
// src/frontend/jit.ts:833-885 for why the frontend cannot fuse them).  A captured step list is in
// hand as a whole, so a run of such Kernels is replaced by one kernel: a CTA per row keeps the row
// and every intermediate in registers, reads each outside array once and writes only what lives on.
enum RowStageType { RS_NONE = 0, RS_REDUCE = 1, RS_ELEMENTWISE = 2, RS_PER_ROW = 3 };

// Can this Kernel be a stage of a row program over [rows, cols]?
RowStageType row_stage_type(const KernelIR& k, int64_t rows, int64_t cols);

struct FuseStage {
  const KernelIR* ir = nullptr;
  std::vector<int> in_buf;  // per Kernel argument: index into the buffer table
  int out_buf = -1;
};
struct FuseBuffer {
  bool external = false;  // holds data before the first stage: read from global memory
  bool store = false;     // lives on after the last stage: written to global memory
  size_t bytes = 0;
};

// Builds the fused kernel.  `params` lists the buffers that become pointer parameters, in order.
// Returns false (with a reason) where the stages do not fit the row program.
bool plan_row_fusion(const std::vector<FuseStage>& stages, const std::vector<FuseBuffer>& bufs, int64_t rows, int64_t cols,
                     const Options& opt, Plan& plan, std::vector<int>& params, std::string& why);

// ---- a producer substituted into its only consumer ---------------------------------------------
//
// `vmap` of a gradient hands over a per-example outer product as a Dot with the batch axis last
// followed by the Kernel that moves the batch axis first (src/frontend/vmap.ts:297-303 and the
// moveaxis of the outputs): the 205 MB result is written, read and written again.  Where a captured
// step list shows that Kernel B is the only reader of Kernel A's output (which the list then frees),
// A elementwise (a reduction of size 1 counts) and B elementwise with one load of that output at an
// index proven in range, B runs with A's expression in place of the load, evaluated at B's index:
// what `jit` itself does for views of elementwise producers, across the Kernel boundary the
// reduction put there.  Arguments of the result: B's without `b_arg`, then A's.
bool compose_elementwise(const KernelIR& a, const KernelIR& b, uint32_t b_arg, KernelIR& out, std::string& why);

// The mirror case: A reduces (a Dot), B is elementwise over the same index space and loads A's
// output at gidx itself; then B's expression becomes the tail of A's epilogue (the back-propagated
// cotangent t = dz W^T masked by the ReLU gate: the GEMM writes the masked product and t is never
// stored).  Arguments of the result: A's, then B's without `b_arg`.
bool compose_epilogue(const KernelIR& a, const KernelIR& b, uint32_t b_arg, KernelIR& out, std::string& why);

// ---- a run of small Kernels as one launch ------------------------------------------------------
//
// A jitted step ends up with many Kernels over a few hundred or thousand elements (the softmax of a
// [64, 10] logit array is six of them, an Adam step of a bias two): inside a graph each costs its
// node-to-node latency, about 2 us, whatever it computes.  A run of such Kernels becomes one kernel
// of a single CTA that evaluates them one after the other, `__syncthreads()` between them, arrays
// passing through global memory exactly as before (so any Kernel qualifies: reductions are looped
// per output).  `in_param` / `out_param` index the kernel's pointer parameters.
struct BatchStage {
  const KernelIR* ir = nullptr;
  std::vector<int> in_param;
  int out_param = -1;
};
// work (outputs x reduction length) up to which a Kernel counts as small
inline double small_kernel_work() { return 16384; }

// JAXCUDA_CHECKED=1 (read once per process): the emitter routes every scalar load through jx_ix,
// which counts indices outside the buffer, and the runtime compiles with JX_CHECKED defined.
inline bool emit_checked() {
  static const bool on = [] { const char* v = getenv("JAXCUDA_CHECKED"); return v && *v && atoi(v) != 0; }();
  return on;
}
bool plan_small_batch(const std::vector<BatchStage>& stages, int n_params, const Options& opt, Plan& plan, std::string& why);

// Implemented in gemm_tc.cpp: rewrites `plan` to the tcgen05 skeleton when `g` qualifies.
// `gather_source` (with g.b_gathered) is the CUDA C of the kernel `jx_gather_b` that fills the B
// operand; it is compiled with the GEMM and launched first.
bool plan_gemm_tc(const KernelIR& k, const GemmDesc& g, const Options& opt, Plan& plan,
                  const std::string& epilogue_body, const std::string& params_decl,
                  const std::string& epilogue_preload = std::string(), const std::string& gather_source = std::string());

}  // namespace jaxcuda

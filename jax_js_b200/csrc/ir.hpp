// Kernel image parsing and index analysis for the cuda backend.
//
// The image is the lowered Kernel of include/jaxcuda_ir.h.  `analyze()` puts every
// int32 index expression it can into the form
//
//     c0 + sum_j  c_j * ((v_j / d_j) % m_j)        v_j in {gidx, ridx}
//
// which is what the skeleton choice and the 128-bit load classification read.  The
// reference does the same job for its Wasm tile plans with `coefficientOfSymbol` and
// `analyzeStride` (src/backend/wasm/tilePlan.ts:74-96, :191-236) and, for WebGPU, by
// looking for stride-0 axes in `tuneWebgpu` (src/tuner.ts:290-323).
#pragma once

#include <cstdint>
#include <optional>
#include <string>
#include <vector>

#include "../../include/jaxcuda_ir.h"

namespace jaxcuda {

struct Node {
  uint32_t op = 0, dtype = 0, nsrc = 0, src[4] = {0, 0, 0, 0};
  uint64_t arg0 = 0;
  uint32_t arg1 = 0;
};

struct KernelIR {
  uint32_t nargs = 0;
  uint64_t size = 0;
  bool has_red = false;
  uint32_t red_dtype = 0, red_op = 0, red_size = 0;
  std::vector<Node> exp, epi;
  uint32_t out_dtype() const { return has_red ? epi.back().dtype : exp.back().dtype; }
};

// Returns an empty string on success, else a message.
std::string parse_kernel(const uint8_t* ir, size_t len, KernelIR& out);

inline int dtype_bytes(uint32_t dt) { return dt == JAXCUDA_F16 ? 2 : dt == JAXCUDA_F64 ? 8 : 4; }
inline bool dtype_is_float(uint32_t dt) { return dt == JAXCUDA_F32 || dt == JAXCUDA_F16 || dt == JAXCUDA_F64; }
const char* dtype_name(uint32_t dt);
const char* op_name(uint32_t op);

// One digit of gidx or ridx: coef * ((v / div) % mod); mod == 0 means "no modulus".
struct Term {
  int var;  // 0 gidx, 1 ridx
  int64_t div, mod, coef;
};

struct Affine {
  int64_t c0 = 0;
  std::vector<Term> terms;
  int64_t lo = 0, hi = 0;  // inclusive value range over the whole index space

  int64_t coef_of(int var, int64_t div) const;        // coefficient of the digit with this divisor (0 if absent)
  bool depends_on(int var) const;
  bool only_plain(int var) const;                      // var appears at most as the plain term v (div 1, no mod)
};

struct Analysis {
  // Per node of one DAG: affine form if the node is an int32 index expression in that form.
  std::vector<std::optional<Affine>> affine;
  std::vector<bool> dep_g, dep_r;  // value depends on gidx / ridx
};

Analysis analyze(const std::vector<Node>& nodes, uint64_t gsize, uint64_t rsize);

}  // namespace jaxcuda

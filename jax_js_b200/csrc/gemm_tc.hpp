// TMA + tcgen05/TMEM GEMM skeleton: planning (source generation) and launch.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "emit.hpp"

namespace jaxcuda {

// Launches the stages of a SK_GEMM_TC plan.  Returns the number of kernels launched, or -1
// with `err` set.  `status_dev` is a device-visible word the kernel writes a code to when a
// pipeline wait times out (0 = healthy).  `max_ctas` > 0 caps the persistent grid (the tile loop strides by
// the grid size, so any grid is correct): used to leave SMs to a collective running beside the GEMM.  `encode_fn` is cuTensorMapEncodeTiled, `launch_fn` cuLaunchKernel, `launch_ex_fn` cuLaunchKernelEx (cluster launch of the paired kernel).
// Remainder planes (3xTF32) kept by the caller instead of the scratch: a null pointer means "in the
// scratch", compute_x false means the plane already holds x - tf32(x) of this operand.
struct LoPlanes {
  float* a = nullptr;
  float* b = nullptr;
  bool compute_a = true, compute_b = true;
};

int launch_gemm_tc(void* encode_fn, void* launch_fn, void* launch_ex_fn, const Plan& plan, const std::vector<CUfunction>& fns,
                   const std::vector<void*>& inputs, void* out, void* scratch, cudaStream_t stream,
                   int* status_dev, std::string& err, int max_ctas = 0, const LoPlanes* lo = nullptr);

}  // namespace jaxcuda

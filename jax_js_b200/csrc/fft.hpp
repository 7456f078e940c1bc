// Fft routine of src/routine.ts (:96-101, CPU reference :543-624).  Plain C entry point over device
// pointers; compiled by nvcc for sm_100a.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// real, imag, out_real, out_imag: [batch, n] of JAXCUDA_F32 or JAXCUDA_F64; `factors` multiply to n
// (the order is the order of the stages).  Rows that do not fit in shared memory are transformed
// stage by stage through global memory and need `work` (jaxcuda_fft_work_bytes bytes, else null).
// Returns a cudaError_t value; cudaErrorInvalidValue when the factors do not multiply to n.
size_t jaxcuda_fft_work_bytes(int dtype, int64_t batch, int64_t n, int max_radix);
int jaxcuda_fft_launch(cudaStream_t stream, int dtype, const void* real, const void* imag, void* out_real, void* out_imag,
                       int64_t batch, int64_t n, const int* factors, int n_factors, int inverse, void* work, int* launches);

#ifdef __cplusplus
}
#endif

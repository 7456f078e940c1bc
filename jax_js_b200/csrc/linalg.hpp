// Dense linear-algebra routines of src/routine.ts: TriangularSolve (:298-338), Cholesky (:340-366),
// LU (:368-432) and JacobiEigh (:434-541).  Plain C entry points over device pointers; compiled by nvcc for sm_100a.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// dtype: JAXCUDA_F32 or JAXCUDA_F64.  Each returns a cudaError_t value (0 = launched).

// y[b] = lower-triangular L with x[b] = L L^T, upper triangle zero-filled; x, y: [batch, n, n].
// Matrices of 256 rows or more are factored block column by block column over many CTAs and need
// `work` (jaxcuda_cholesky_work_bytes bytes; null below that size).
size_t jaxcuda_cholesky_work_bytes(int64_t batch, int64_t n);
int jaxcuda_cholesky_launch(cudaStream_t stream, int dtype, const void* x, void* y, int64_t batch, int64_t n, void* work,
                            int* launches);

// a: [mats, n, n] upper triangular, b and x: [mats, rows, n]; each row solves a x = b.
int jaxcuda_triangular_solve_launch(cudaStream_t stream, int dtype, const void* a, const void* b, void* x, int64_t mats,
                                    int64_t rows, int64_t n, int unit_diagonal, int* launches);

// a, lu: [batch, m, n]; pivots: int32 [batch, min(m, n)]; perm: int32 [batch, m].  Partial pivoting.
int jaxcuda_lu_launch(cudaStream_t stream, int dtype, const void* a, void* lu, int32_t* pivots, int32_t* perm,
                      int64_t batch, int64_t m, int64_t n, int* launches);

// x: [batch, n, n] symmetric (lower triangle read); diagonalized, vectors: [batch, n, n].  Cyclic Jacobi
// sweeps until the largest off-diagonal magnitude is at most tolerance * max(1, max|x|) or max_sweeps.
int jaxcuda_jacobi_eigh_launch(cudaStream_t stream, int dtype, const void* x, void* diagonalized, void* vectors,
                               int64_t batch, int64_t n, int max_sweeps, double tolerance, int* launches);

#ifdef __cplusplus
}
#endif

// TriangularSolve, Cholesky and LU routines (CPU reference: src/routine.ts:298-432).
//
// The reference runs these on typed arrays with JavaScript numbers: every intermediate is a double
// and a value is rounded to the array's element type only when it is stored.  The kernels keep
// that arithmetic (double accumulators and quotients, one rounding per store), so float32 results
// agree with the reference to the last bit except where a sum's order of addition (here: split
// over the lanes of a warp) changes a double's last bit exactly at a float32 rounding boundary.
//
// Parallelism: independent matrices (and right-hand sides) go to different CTAs (warps); inside a
// matrix the algorithms are the reference's, column by column, with the work of one column spread
// over the CTA.  A matrix stays in L2/L1 while its CTA works on it.  Cholesky of matrices with 256
// rows or more runs blocked over many CTAs (below); LU and the triangular solve do not.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jaxcuda_ir.h"
#include "linalg.hpp"

namespace {

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- Cholesky-Banachiewicz, one CTA per matrix -------------------------------------------------
// Column j: the diagonal first (warp 0), then L[i, j] for i > j, one warp per row, lanes over k.
template <class T>
__global__ void __launch_bounds__(1024) cholesky_kernel(const T* __restrict__ x, T* __restrict__ y, int n) {
  extern __shared__ double rowj[];  // row j of L, columns < j; rowj[n] = the stored diagonal
  const T* A = x + (size_t)blockIdx.x * n * n;
  T* L = y + (size_t)blockIdx.x * n * n;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (size_t i = threadIdx.x; i < (size_t)n * n; i += blockDim.x) L[i] = (T)0;
  __syncthreads();
  for (int j = 0; j < n; j++) {
    for (int k = threadIdx.x; k < j; k += blockDim.x) rowj[k] = (double)L[(size_t)j * n + k];
    __syncthreads();
    if (warp == 0) {
      double s = 0.0;
      for (int k = lane; k < j; k += 32) s = fma(rowj[k], rowj[k], s);
      s = warp_sum(s);
      if (lane == 0) {
        const T d = (T)sqrt((double)A[(size_t)j * n + j] - s);
        L[(size_t)j * n + j] = d;
        rowj[n] = (double)d;
      }
    }
    __syncthreads();
    const double d = rowj[n];
    for (int i = j + 1 + warp; i < n; i += nw) {
      const T* Li = L + (size_t)i * n;
      double s = 0.0;
      for (int k = lane; k < j; k += 32) s = fma((double)Li[k], rowj[k], s);
      s = warp_sum(s);
      if (lane == 0) L[(size_t)i * n + j] = (T)(((double)A[(size_t)i * n + j] - s) / d);
    }
    __syncthreads();
  }
}

// ---- blocked Cholesky over many CTAs, for matrices of 256 rows and more ---------------------------
// The reference switches to a blocked multi-pass variant on its GPU backend for large matrices
// (src/backend/webgpu/routines.ts:630-634).  Here the matrix is cut into block columns of NB = 64.
// L[i, j] = (A[i, j] - sum_{k<j} L[i, k] L[j, k]) / L[j, j] keeps the reference's arithmetic: the sum
// is a double from k = 0 to j - 1 and the only rounding is the store.  For the block column that
// starts at column J0 the sum is split at J0:
//   chol_update   S[i, c] = sum_{k < J0} L[i, k] L[J0 + c, k]       every row i >= J0, many CTAs, double
//   chol_diag     the NB x NB diagonal block, column by column, from S  one CTA
//   chol_rows     rows below the block, each on its own (a row needs  a warp per row, many CTAs
//                 only itself and the diagonal block)
// S stays in double in a work buffer, so no value is rounded before its store.
constexpr int kCholNB = 64;

template <class T>
__global__ void __launch_bounds__(256) chol_update(const T* __restrict__ y, double* __restrict__ S, int n, int J0) {
  // CTA: 64 rows x 64 block columns; thread: 4 x 4 outputs; K in slices of 16 through shared memory
  __shared__ double As[16][64 + 1], Bs[16][64 + 1];
  const T* L = y + (size_t)blockIdx.y * n * n;
  double* Sm = S + (size_t)blockIdx.y * n * kCholNB;
  const int r0 = J0 + blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  double acc[4][4] = {};
  for (int k0 = 0; k0 < J0; k0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int rr = e >> 4, kk = e & 15;
      const int i = r0 + rr, c = J0 + rr;
      As[kk][rr] = (i < n) ? (double)L[(size_t)i * n + k0 + kk] : 0.0;
      Bs[kk][rr] = (c < n) ? (double)L[(size_t)c * n + k0 + kk] : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; kk++) {
      double a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; u++) { a[u] = As[kk][ty * 4 + u]; b[u] = Bs[kk][tx * 4 + u]; }
#pragma unroll
      for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) acc[u][v] = fma(a[u], b[v], acc[u][v]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; u++) {
    const int i = r0 + ty * 4 + u;
    if (i >= n) continue;
#pragma unroll
    for (int v = 0; v < 4; v++) Sm[(size_t)i * kCholNB + tx * 4 + v] = acc[u][v];
  }
}

template <class T>
__global__ void __launch_bounds__(256) chol_diag(const T* __restrict__ x, T* __restrict__ y, const double* __restrict__ S, int n, int J0) {
  __shared__ double Lb[kCholNB][kCholNB + 1];   // the block's entries as stored
  const T* A = x + (size_t)blockIdx.x * n * n;
  T* L = y + (size_t)blockIdx.x * n * n;
  const double* Sm = S + (size_t)blockIdx.x * n * kCholNB;
  const int nb = min(kCholNB, n - J0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int c = 0; c < nb; c++) {
    const int j = J0 + c;
    if (warp == 0) {
      double s = 0.0;
      for (int k = lane; k < c; k += 32) s = fma(Lb[c][k], Lb[c][k], s);
      s = warp_sum(s);
      if (lane == 0) {
        const T d = (T)sqrt((double)A[(size_t)j * n + j] - (Sm[(size_t)j * kCholNB + c] + s));
        L[(size_t)j * n + j] = d;
        Lb[c][c] = (double)d;
      }
    }
    __syncthreads();
    const double d = Lb[c][c];
    for (int r = c + 1 + warp; r < nb; r += nw) {
      double s = 0.0;
      for (int k = lane; k < c; k += 32) s = fma(Lb[r][k], Lb[c][k], s);
      s = warp_sum(s);
      if (lane == 0) {
        const int i = J0 + r;
        const T v = (T)(((double)A[(size_t)i * n + j] - (Sm[(size_t)i * kCholNB + c] + s)) / d);
        L[(size_t)i * n + j] = v;
        Lb[r][c] = (double)v;
      }
    }
    __syncthreads();
  }
}

template <class T>
__global__ void __launch_bounds__(256) chol_rows(const T* __restrict__ x, T* __restrict__ y, const double* __restrict__ S, int n, int J0) {
  __shared__ double Lb[kCholNB][kCholNB + 1];
  __shared__ double rowv[8][kCholNB];
  const T* A = x + (size_t)blockIdx.y * n * n;
  T* L = y + (size_t)blockIdx.y * n * n;
  const double* Sm = S + (size_t)blockIdx.y * n * kCholNB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < kCholNB * kCholNB; e += 256) {
    const int r = e / kCholNB, c = e % kCholNB;
    Lb[r][c] = (c <= r && J0 + r < n) ? (double)L[(size_t)(J0 + r) * n + J0 + c] : 0.0;
  }
  __syncthreads();
  const int i = J0 + kCholNB + blockIdx.x * 8 + warp;
  if (i >= n) return;
  double* rv = rowv[warp];
  for (int c = 0; c < kCholNB; c++) {
    double s = 0.0;
    for (int k = lane; k < c; k += 32) s = fma(rv[k], Lb[c][k], s);
    s = warp_sum(s);
    if (lane == 0) {
      const int j = J0 + c;
      const T v = (T)(((double)A[(size_t)i * n + j] - (Sm[(size_t)i * kCholNB + c] + s)) / Lb[c][c]);
      L[(size_t)i * n + j] = v;
      rv[c] = (double)v;
    }
    __syncwarp();
  }
}

template <class T>
cudaError_t cholesky_blocked(cudaStream_t stream, const T* x, T* y, double* work, int64_t batch, int n, int* launches) {
  cudaError_t e = cudaMemsetAsync(y, 0, (size_t)batch * n * n * sizeof(T), stream);
  if (e != cudaSuccess) return e;
  for (int J0 = 0; J0 < n; J0 += kCholNB) {
    const int rows = n - J0;
    if (J0 > 0) {
      chol_update<T><<<dim3((rows + 63) / 64, (unsigned)batch), 256, 0, stream>>>(y, work, n, J0);
    } else {
      e = cudaMemsetAsync(work, 0, (size_t)batch * n * kCholNB * sizeof(double), stream);
      if (e != cudaSuccess) return e;
    }
    chol_diag<T><<<(unsigned)batch, 256, 0, stream>>>(x, y, work, n, J0);
    const int below = rows - kCholNB;
    if (below > 0) chol_rows<T><<<dim3((below + 7) / 8, (unsigned)batch), 256, 0, stream>>>(x, y, work, n, J0);
    if (launches) *launches += 3;
  }
  return cudaGetLastError();
}

// ---- back substitution, one warp per right-hand side ----------------------------------------------
template <class T>
__global__ void __launch_bounds__(256) trisolve_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ x,
                                                       int n, long long rows, long long total, int unit) {
  extern __shared__ double xs_all[];  // [warps][n]: the solved entries, as stored
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const long long rhs = (long long)blockIdx.x * nw + warp;
  if (rhs >= total) return;
  const T* A = a + (size_t)(rhs / rows) * n * n;
  const T* bv = b + (size_t)rhs * n;
  T* xv = x + (size_t)rhs * n;
  double* xs = xs_all + (size_t)warp * n;
  for (int i = n - 1; i >= 0; i--) {
    const T* Ai = A + (size_t)i * n;
    double s = 0.0;
    for (int j = i + 1 + lane; j < n; j += 32) s = fma((double)Ai[j], xs[j], s);
    s = warp_sum(s);
    if (lane == 0) {
      double v = (double)bv[i] - s;
      if (!unit) v = v / (double)Ai[i];
      const T r = (T)v;
      xv[i] = r;
      xs[i] = (double)r;
    }
    __syncwarp();
  }
}

// ---- LU with partial pivoting, one CTA per matrix ---------------------------------------------------
template <class T>
__global__ void __launch_bounds__(1024) lu_kernel(const T* __restrict__ a, T* __restrict__ lu_all, int32_t* __restrict__ pivots,
                                                  int32_t* __restrict__ perm_all, int m, int n) {
  __shared__ double best_v[32];
  __shared__ int best_r[32];
  __shared__ int pivot_row;
  const int r = m < n ? m : n;
  const T* A = a + (size_t)blockIdx.x * m * n;
  T* lu = lu_all + (size_t)blockIdx.x * m * n;
  int32_t* piv = pivots + (size_t)blockIdx.x * r;
  int32_t* perm = perm_all + (size_t)blockIdx.x * m;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  for (size_t i = tid; i < (size_t)m * n; i += blockDim.x) lu[i] = A[i];
  for (int i = tid; i < m; i += blockDim.x) perm[i] = i;
  __syncthreads();
  for (int j = 0; j < r; j++) {
    // Pivot: the reference scans rows j+1.. and moves on a strictly greater |value| (a NaN never
    // compares greater; a NaN in row j stays the pivot): the first row attaining the maximum.
    double bv = -1.0;
    int br = 0x7fffffff;
    for (int i = j + 1 + tid; i < m; i += blockDim.x) {
      const double v = fabs((double)lu[(size_t)i * n + j]);
      if (v > bv) { bv = v; br = i; }      // ascending i per thread: keeps the first of equals
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int orow = __shfl_xor_sync(0xffffffffu, br, o);
      if (ov > bv || (ov == bv && orow < br)) { bv = ov; br = orow; }
    }
    if (lane == 0) { best_v[warp] = bv; best_r[warp] = br; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < nw ? best_v[lane] : -1.0;
      br = lane < nw ? best_r[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const double ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int orow = __shfl_xor_sync(0xffffffffu, br, o);
        if (ov > bv || (ov == bv && orow < br)) { bv = ov; br = orow; }
      }
      if (lane == 0) {
        const double own = fabs((double)lu[(size_t)j * n + j]);
        const int row = (bv > own) ? br : j;   // own = NaN: every comparison is false, row j stays
        pivot_row = row;
        piv[j] = row;
        if (row != j) { const int t = perm[j]; perm[j] = perm[row]; perm[row] = t; }
      }
    }
    __syncthreads();
    const int row = pivot_row;
    if (row != j) {
      for (int c = tid; c < n; c += blockDim.x) {
        const T t = lu[(size_t)j * n + c];
        lu[(size_t)j * n + c] = lu[(size_t)row * n + c];
        lu[(size_t)row * n + c] = t;
      }
      __syncthreads();
    }
    const double diag = (double)lu[(size_t)j * n + j];
    if (diag != 0.0) {
      // trailing update with the unrounded factor, as the reference keeps it in a local
      for (int i = j + 1 + warp; i < m; i += nw) {
        const double f = (double)lu[(size_t)i * n + j] / diag;
        T* row_i = lu + (size_t)i * n;
        const T* row_j = lu + (size_t)j * n;
        for (int c = j + 1 + lane; c < n; c += 32)
          row_i[c] = (T)__dsub_rn((double)row_i[c], __dmul_rn(f, (double)row_j[c]));
      }
      __syncthreads();
      for (int i = j + 1 + tid; i < m; i += blockDim.x)
        lu[(size_t)i * n + j] = (T)((double)lu[(size_t)i * n + j] / diag);
    }
    __syncthreads();
  }
}

// ---- cyclic Jacobi eigendecomposition, one CTA per matrix (src/routine.ts:434-541) -------------------
// The rotations run in the reference's order (p ascending, q ascending inside), one after the
// other; the n-element row/column updates of one rotation are spread over the CTA.  Every formula
// is evaluated with the reference's grouping in unfused double arithmetic, so convergence tests and
// results follow the reference step by step.  `a` keeps only its lower triangle (symIndex).
__device__ __forceinline__ double jmul(double a, double b) { return __dmul_rn(a, b); }

template <class T>
__device__ __forceinline__ double block_max(double v, double* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = red[0];
  for (int w = 1; w < nw; w++) v = fmax(v, red[w]);
  return v;
}

template <class T>
__global__ void __launch_bounds__(1024) jacobi_kernel(const T* __restrict__ in, T* __restrict__ a_all, T* __restrict__ v_all,
                                                      int n, int max_sweeps, double tolerance, int in_smem) {
  extern __shared__ __align__(16) unsigned char jac_smem[];
  __shared__ double red[32];
  const size_t nn = (size_t)n * n;
  const T* x = in + blockIdx.x * nn;
  T* ag = a_all + blockIdx.x * nn;
  T* vg = v_all + blockIdx.x * nn;
  T* a = in_smem ? reinterpret_cast<T*>(jac_smem) : ag;
  T* v = in_smem ? reinterpret_cast<T*>(jac_smem) + nn : vg;
  for (size_t idx = threadIdx.x; idx < nn; idx += blockDim.x) {
    const int i = (int)(idx / n), j = (int)(idx - (size_t)i * n);
    a[idx] = j <= i ? x[idx] : (T)0;
    v[idx] = i == j ? (T)1 : (T)0;
  }
  __syncthreads();
  auto off_diagonal_max = [&](bool with_diagonal, double start) {
    double m = start;
    for (size_t idx = threadIdx.x; idx < nn; idx += blockDim.x) {
      const int i = (int)(idx / n), j = (int)(idx - (size_t)i * n);
      if (j < i || (with_diagonal && j == i)) {
        const double val = fabs((double)a[idx]);
        if (val > m) m = val;                 // Math.max would propagate a NaN; a NaN input is outside the contract
      }
    }
    return block_max<T>(m, red);
  };
  const double threshold = jmul(tolerance, off_diagonal_max(true, 1.0));
  double off = off_diagonal_max(false, 0.0);
  for (int sweep = 0; sweep < max_sweeps && off > threshold; sweep++) {
    for (int p = 0; p < n - 1; p++) {
      for (int q = p + 1; q < n; q++) {
        const size_t pp = (size_t)p * n + p, qq = (size_t)q * n + q, pq = (size_t)q * n + p;  // q > p: symIndex(p, q)
        const double app = (double)a[pp], aqq = (double)a[qq], apq = (double)a[pq];
        __syncthreads();                      // everyone has read the three before anyone writes them
        if (apq == 0.0) continue;
        const double tau = __ddiv_rn(__dsub_rn(aqq, app), jmul(2.0, apq));
        const double sign = tau >= 0.0 ? 1.0 : -1.0;
        const double t = __ddiv_rn(sign, __dadd_rn(fabs(tau), __dsqrt_rn(__dadd_rn(jmul(tau, tau), 1.0))));
        const double c = __ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(jmul(t, t), 1.0)));
        const double s = jmul(t, c);
        for (int k = threadIdx.x; k < n; k += blockDim.x) {
          if (k != p && k != q) {
            const size_t kp = k >= p ? (size_t)k * n + p : (size_t)p * n + k;
            const size_t kq = k >= q ? (size_t)k * n + q : (size_t)q * n + k;
            const double akp = (double)a[kp], akq = (double)a[kq];
            a[kp] = (T)__dsub_rn(jmul(c, akp), jmul(s, akq));
            a[kq] = (T)__dadd_rn(jmul(s, akp), jmul(c, akq));
          }
          const size_t vp = (size_t)k * n + p, vq = (size_t)k * n + q;
          const double vkp = (double)v[vp], vkq = (double)v[vq];
          v[vp] = (T)__dsub_rn(jmul(c, vkp), jmul(s, vkq));
          v[vq] = (T)__dadd_rn(jmul(s, vkp), jmul(c, vkq));
        }
        if (threadIdx.x == 0) {
          const double sc2 = jmul(jmul(jmul(2.0, s), c), apq);
          a[pp] = (T)__dadd_rn(__dsub_rn(jmul(jmul(c, c), app), sc2), jmul(jmul(s, s), aqq));
          a[qq] = (T)__dadd_rn(__dadd_rn(jmul(jmul(s, s), app), sc2), jmul(jmul(c, c), aqq));
          a[pq] = (T)0;
        }
        __syncthreads();
      }
    }
    off = off_diagonal_max(false, 0.0);
  }
  if (in_smem) {
    __syncthreads();
    for (size_t idx = threadIdx.x; idx < nn; idx += blockDim.x) { ag[idx] = a[idx]; vg[idx] = v[idx]; }
  }
}

template <class K>
cudaError_t allow_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

extern "C" {

size_t jaxcuda_cholesky_work_bytes(int64_t batch, int64_t n) {
  return n >= 256 ? (size_t)batch * (size_t)n * kCholNB * sizeof(double) : 0;
}

int jaxcuda_cholesky_launch(cudaStream_t stream, int dtype, const void* x, void* y, int64_t batch, int64_t n, void* work,
                            int* launches) {
  if (launches) *launches = 0;
  if (batch <= 0 || n <= 0) return cudaSuccess;
  if (n >= 256) {
    if (!work || batch > 65535 || n > 0x7fffffff / 2) return cudaErrorInvalidValue;
    if (dtype == JAXCUDA_F32) return cholesky_blocked<float>(stream, (const float*)x, (float*)y, (double*)work, batch, (int)n, launches);
    return cholesky_blocked<double>(stream, (const double*)x, (double*)y, (double*)work, batch, (int)n, launches);
  }
  const size_t smem = (size_t)(n + 1) * sizeof(double);
  if (smem > 200 * 1024 || batch > 0x7fffffff) return cudaErrorInvalidValue;
  const int threads = n >= 256 ? 1024 : n >= 64 ? 256 : 64;
  cudaError_t e;
  if (dtype == JAXCUDA_F32) {
    if ((e = allow_smem(cholesky_kernel<float>, smem)) != cudaSuccess) return e;
    cholesky_kernel<float><<<(unsigned)batch, threads, smem, stream>>>((const float*)x, (float*)y, (int)n);
  } else {
    if ((e = allow_smem(cholesky_kernel<double>, smem)) != cudaSuccess) return e;
    cholesky_kernel<double><<<(unsigned)batch, threads, smem, stream>>>((const double*)x, (double*)y, (int)n);
  }
  if (launches) *launches = 1;
  return cudaGetLastError();
}

int jaxcuda_triangular_solve_launch(cudaStream_t stream, int dtype, const void* a, const void* b, void* x, int64_t mats,
                                    int64_t rows, int64_t n, int unit_diagonal, int* launches) {
  if (launches) *launches = 0;
  const int64_t total = mats * rows;
  if (total <= 0 || n <= 0) return cudaSuccess;
  int warps = 8;
  while (warps > 1 && (size_t)warps * n * sizeof(double) > 160 * 1024) warps >>= 1;
  const size_t smem = (size_t)warps * n * sizeof(double);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  const int64_t blocks = (total + warps - 1) / warps;
  if (blocks > 0x7fffffff) return cudaErrorInvalidValue;
  cudaError_t e;
  if (dtype == JAXCUDA_F32) {
    if ((e = allow_smem(trisolve_kernel<float>, smem)) != cudaSuccess) return e;
    trisolve_kernel<float><<<(unsigned)blocks, warps * 32, smem, stream>>>((const float*)a, (const float*)b, (float*)x, (int)n,
                                                                           rows, total, unit_diagonal);
  } else {
    if ((e = allow_smem(trisolve_kernel<double>, smem)) != cudaSuccess) return e;
    trisolve_kernel<double><<<(unsigned)blocks, warps * 32, smem, stream>>>((const double*)a, (const double*)b, (double*)x, (int)n,
                                                                            rows, total, unit_diagonal);
  }
  if (launches) *launches = 1;
  return cudaGetLastError();
}

int jaxcuda_lu_launch(cudaStream_t stream, int dtype, const void* a, void* lu, int32_t* pivots, int32_t* perm,
                      int64_t batch, int64_t m, int64_t n, int* launches) {
  if (launches) *launches = 0;
  if (batch <= 0 || m <= 0 || n <= 0) return cudaSuccess;
  if (batch > 0x7fffffff || m > 0x7fffffff || n > 0x7fffffff) return cudaErrorInvalidValue;
  const int threads = m * n >= 65536 ? 1024 : m * n >= 4096 ? 256 : 64;
  if (dtype == JAXCUDA_F32)
    lu_kernel<float><<<(unsigned)batch, threads, 0, stream>>>((const float*)a, (float*)lu, pivots, perm, (int)m, (int)n);
  else
    lu_kernel<double><<<(unsigned)batch, threads, 0, stream>>>((const double*)a, (double*)lu, pivots, perm, (int)m, (int)n);
  if (launches) *launches = 1;
  return cudaGetLastError();
}

int jaxcuda_jacobi_eigh_launch(cudaStream_t stream, int dtype, const void* x, void* diagonalized, void* vectors,
                               int64_t batch, int64_t n, int max_sweeps, double tolerance, int* launches) {
  if (launches) *launches = 0;
  if (batch <= 0 || n <= 0) return cudaSuccess;
  if (batch > 0x7fffffff || n > 32768) return cudaErrorInvalidValue;
  const size_t e = dtype == JAXCUDA_F32 ? 4 : 8;
  const size_t want = 2 * (size_t)n * n * e;
  const int in_smem = want <= 200 * 1024;
  const size_t smem = in_smem ? want : 0;
  int threads = 32;
  while (threads < n && threads < 1024) threads <<= 1;
  cudaError_t err;
  if (dtype == JAXCUDA_F32) {
    if ((err = allow_smem(jacobi_kernel<float>, smem)) != cudaSuccess) return err;
    jacobi_kernel<float><<<(unsigned)batch, threads, smem, stream>>>((const float*)x, (float*)diagonalized, (float*)vectors,
                                                                     (int)n, max_sweeps, tolerance, in_smem);
  } else {
    if ((err = allow_smem(jacobi_kernel<double>, smem)) != cudaSuccess) return err;
    jacobi_kernel<double><<<(unsigned)batch, threads, smem, stream>>>((const double*)x, (double*)diagonalized, (double*)vectors,
                                                                      (int)n, max_sweeps, tolerance, in_smem);
  }
  if (launches) *launches = 1;
  return cudaGetLastError();
}

}  // extern "C"

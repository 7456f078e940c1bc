// Fft routine (src/routine.ts:96-101, CPU reference runFft :543-624): complex FFT along the last axis
// of a real/imaginary pair, for the factorisation of the length the frontend passes in.
//
// The reference is a mixed-radix decimation-in-time transform: a digit-reversal permutation, then
// one stage per factor; a stage multiplies each input of a butterfly by its twiddle and takes a
// radix-point DFT, all in double arithmetic, and stores the stage's result in the output arrays
// (so float32 data is rounded once per stage).  The kernel keeps that structure and rounding.  One
// CTA per row; the row lives in shared memory in the element type; a thread computes one output
// point of one butterfly per step (radix inputs, twiddled on the fly); a stage's two twiddle tables
// (cos/sin of 2 pi t / span and of 2 pi t / radix) are built in shared memory first, so the
// transcendental work is O(span + radix) per stage instead of O(n radix).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jaxcuda_ir.h"
#include "fft.hpp"

namespace {

constexpr int kMaxFactors = 32;
struct FftPlan {
  int n, n_factors, inverse;
  int factors[kMaxFactors];
};

template <class T>
__global__ void __launch_bounds__(256) fft_kernel(const T* __restrict__ real, const T* __restrict__ imag, T* __restrict__ out_real,
                                                  T* __restrict__ out_imag, FftPlan plan, int max_radix) {
  extern __shared__ __align__(16) unsigned char fft_smem[];
  const int n = plan.n;
  double* tw = reinterpret_cast<double*>(fft_smem);          // [2 * n]: cos, sin of angleScale * t / span
  double* tr = tw + 2 * (size_t)n;                           // [2 * max_radix]: the same over the radix
  T* buf = reinterpret_cast<T*>(tr + 2 * (size_t)max_radix); // [2][2 * n]: real then imaginary, ping-pong
  const size_t row = (size_t)blockIdx.x * n;
  const double angle_scale = (plan.inverse ? 2.0 : -2.0) * 3.141592653589793;
  // digit reversal (:549-563)
  for (int index = threadIdx.x; index < n; index += blockDim.x) {
    int remaining = index, stride = 1, reversed = 0;
    for (int f = 0; f < plan.n_factors; f++) {
      const int factor = plan.factors[f];
      const int digit = remaining % factor;
      remaining /= factor;
      stride *= factor;
      reversed += digit * (n / stride);
    }
    buf[index] = real[row + reversed];
    buf[n + index] = imag[row + reversed];
  }
  int cur = 0, prev = 1;
  for (int stage = 0; stage < plan.n_factors; stage++) {
    const int radix = plan.factors[stage];
    const int span = prev * radix;
    const double stage_scale = (plan.inverse && stage == plan.n_factors - 1) ? 1.0 / n : 1.0;
    __syncthreads();
    for (int t = threadIdx.x; t < span; t += blockDim.x) {
      const double angle = angle_scale * t / span;
      tw[2 * t] = cos(angle);
      tw[2 * t + 1] = sin(angle);
    }
    for (int t = threadIdx.x; t < radix; t += blockDim.x) {
      const double angle = angle_scale * t / radix;
      tr[2 * t] = cos(angle);
      tr[2 * t + 1] = sin(angle);
    }
    __syncthreads();
    const T* src = buf + (size_t)cur * 2 * n;
    T* dst = buf + (size_t)(cur ^ 1) * 2 * n;
    for (int o = threadIdx.x; o < n; o += blockDim.x) {
      const int group = o / span * span, within = o - group;
      const int p = within / prev, j = within - p * prev;
      double sum_real = 0.0, sum_imag = 0.0;
      for (int q = 0; q < radix; q++) {
        const int idx = group + j + q * prev;
        const double xr0 = (double)src[idx], xi0 = (double)src[n + idx];
        const int t1 = q * j;                                 // < span
        const double c1 = tw[2 * t1], s1 = tw[2 * t1 + 1];
        const double xr = __dsub_rn(__dmul_rn(xr0, c1), __dmul_rn(xi0, s1));
        const double xi = __dadd_rn(__dmul_rn(xr0, s1), __dmul_rn(xi0, c1));
        const int t2 = (int)(((long long)q * p) % radix);
        const double c2 = tr[2 * t2], s2 = tr[2 * t2 + 1];
        sum_real = __dadd_rn(sum_real, __dsub_rn(__dmul_rn(xr, c2), __dmul_rn(xi, s2)));
        sum_imag = __dadd_rn(sum_imag, __dadd_rn(__dmul_rn(xr, s2), __dmul_rn(xi, c2)));
      }
      dst[o] = (T)__dmul_rn(sum_real, stage_scale);
      dst[n + o] = (T)__dmul_rn(sum_imag, stage_scale);
    }
    cur ^= 1;
    prev = span;
  }
  __syncthreads();
  const T* fin = buf + (size_t)cur * 2 * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    out_real[row + i] = fin[i];
    out_imag[row + i] = fin[n + i];
  }
}

// Rows too long for shared memory: the same permutation and stages as separate kernels over global
// memory, ping-ponging between the output arrays and a work buffer of the same size.  A thread
// still computes one output point of one butterfly; its twiddles are evaluated on the fly with the
// same double-precision expressions that fill the shared-memory tables above, so both paths give
// the same numbers.
template <class T>
__global__ void __launch_bounds__(256) fft_reverse_kernel(const T* __restrict__ real, const T* __restrict__ imag, T* __restrict__ dst_real,
                                                          T* __restrict__ dst_imag, FftPlan plan, long long total) {
  const int n = plan.n;
  for (long long t = (long long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long long)gridDim.x * 256) {
    const long long row = t / n * n;
    int remaining = (int)(t - row), stride = 1, reversed = 0;
    for (int f = 0; f < plan.n_factors; f++) {
      const int factor = plan.factors[f];
      const int digit = remaining % factor;
      remaining /= factor;
      stride *= factor;
      reversed += digit * (n / stride);
    }
    dst_real[t] = real[row + reversed];
    dst_imag[t] = imag[row + reversed];
  }
}

template <class T>
__global__ void __launch_bounds__(256) fft_stage_kernel(const T* __restrict__ src_real, const T* __restrict__ src_imag, T* __restrict__ dst_real,
                                                        T* __restrict__ dst_imag, int n, int radix, int prev, double angle_scale,
                                                        double stage_scale, long long total) {
  const int span = prev * radix;
  for (long long t = (long long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long long)gridDim.x * 256) {
    const long long row = t / n * n;
    const int o = (int)(t - row);
    const int group = o / span * span, within = o - group;
    const int p = within / prev, j = within - p * prev;
    double sum_real = 0.0, sum_imag = 0.0;
    for (int q = 0; q < radix; q++) {
      const long long idx = row + group + j + q * prev;
      const double xr0 = (double)src_real[idx], xi0 = (double)src_imag[idx];
      const double a1 = angle_scale * (q * j) / span;
      const double c1 = cos(a1), s1 = sin(a1);
      const double xr = __dsub_rn(__dmul_rn(xr0, c1), __dmul_rn(xi0, s1));
      const double xi = __dadd_rn(__dmul_rn(xr0, s1), __dmul_rn(xi0, c1));
      const double a2 = angle_scale * (int)(((long long)q * p) % radix) / radix;
      const double c2 = cos(a2), s2 = sin(a2);
      sum_real = __dadd_rn(sum_real, __dsub_rn(__dmul_rn(xr, c2), __dmul_rn(xi, s2)));
      sum_imag = __dadd_rn(sum_imag, __dadd_rn(__dmul_rn(xr, s2), __dmul_rn(xi, c2)));
    }
    dst_real[t] = (T)__dmul_rn(sum_real, stage_scale);
    dst_imag[t] = (T)__dmul_rn(sum_imag, stage_scale);
  }
}

template <class T>
cudaError_t fft_global(cudaStream_t stream, const T* real, const T* imag, T* out_real, T* out_imag, T* work, const FftPlan& plan,
                       long long batch, int* launches) {
  const long long total = batch * plan.n;
  const unsigned grid = (unsigned)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  T* buf_real[2] = {out_real, work};
  T* buf_imag[2] = {out_imag, work + total};
  int cur = plan.n_factors & 1;   // after n_factors hops the data must sit in the output arrays
  fft_reverse_kernel<T><<<grid, 256, 0, stream>>>(real, imag, buf_real[cur], buf_imag[cur], plan, total);
  if (launches) (*launches)++;
  const double angle_scale = (plan.inverse ? 2.0 : -2.0) * 3.141592653589793;
  int prev = 1;
  for (int stage = 0; stage < plan.n_factors; stage++) {
    const int radix = plan.factors[stage];
    const double stage_scale = (plan.inverse && stage == plan.n_factors - 1) ? 1.0 / plan.n : 1.0;
    fft_stage_kernel<T><<<grid, 256, 0, stream>>>(buf_real[cur], buf_imag[cur], buf_real[cur ^ 1], buf_imag[cur ^ 1], plan.n, radix, prev,
                                                  angle_scale, stage_scale, total);
    if (launches) (*launches)++;
    cur ^= 1;
    prev *= radix;
  }
  return cudaGetLastError();
}

size_t fft_smem_bytes(int dtype, int64_t n, int max_radix) {
  const size_t e = dtype == JAXCUDA_F32 ? 4 : 8;
  return (2 * (size_t)n + 2 * (size_t)max_radix) * sizeof(double) + 4 * (size_t)n * e;
}
constexpr size_t kFftSmemLimit = 220 * 1024;   // rows up to 6.8 K points (float32) / 4.5 K (float64) stay in shared memory

}  // namespace

// Bytes of global work space the transform needs: none while a row fits in shared memory.
extern "C" size_t jaxcuda_fft_work_bytes(int dtype, int64_t batch, int64_t n, int max_radix) {
  if (fft_smem_bytes(dtype, n, max_radix) <= kFftSmemLimit) return 0;
  return 2 * (size_t)batch * (size_t)n * (dtype == JAXCUDA_F32 ? 4 : 8);
}

extern "C" int jaxcuda_fft_launch(cudaStream_t stream, int dtype, const void* real, const void* imag, void* out_real,
                                  void* out_imag, int64_t batch, int64_t n, const int* factors, int n_factors, int inverse,
                                  void* work, int* launches) {
  if (launches) *launches = 0;
  if (batch <= 0) return cudaSuccess;
  if (n < 1 || n_factors < 0 || n_factors > kMaxFactors || batch > 0x7fffffff) return cudaErrorInvalidValue;
  FftPlan plan;
  plan.n = (int)n;
  plan.n_factors = n_factors;
  plan.inverse = inverse;
  int max_radix = 1;
  long long prod = 1;
  for (int i = 0; i < n_factors; i++) {
    if (factors[i] < 1) return cudaErrorInvalidValue;
    plan.factors[i] = factors[i];
    max_radix = factors[i] > max_radix ? factors[i] : max_radix;
    prod *= factors[i];
  }
  if (prod != n) return cudaErrorInvalidValue;
  const size_t smem = fft_smem_bytes(dtype, n, max_radix);
  if (smem > kFftSmemLimit) {
    if (!work || (long long)batch * n >= (1ll << 40)) return cudaErrorInvalidValue;
    if (dtype == JAXCUDA_F32)
      return fft_global<float>(stream, (const float*)real, (const float*)imag, (float*)out_real, (float*)out_imag, (float*)work, plan, batch, launches);
    return fft_global<double>(stream, (const double*)real, (const double*)imag, (double*)out_real, (double*)out_imag, (double*)work, plan, batch, launches);
  }
  cudaError_t err = cudaSuccess;
  if (dtype == JAXCUDA_F32) {
    if (smem > 48 * 1024) err = cudaFuncSetAttribute(fft_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    fft_kernel<float><<<(unsigned)batch, 256, smem, stream>>>((const float*)real, (const float*)imag, (float*)out_real,
                                                              (float*)out_imag, plan, max_radix);
  } else {
    if (smem > 48 * 1024) err = cudaFuncSetAttribute(fft_kernel<double>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    fft_kernel<double><<<(unsigned)batch, 256, smem, stream>>>((const double*)real, (const double*)imag, (double*)out_real,
                                                               (double*)out_imag, plan, max_radix);
  }
  if (launches) *launches = 1;
  return cudaGetLastError();
}

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

}  // namespace

extern "C" int jaxcuda_fft_launch(cudaStream_t stream, int dtype, const void* real, const void* imag, void* out_real,
                                  void* out_imag, int64_t batch, int64_t n, const int* factors, int n_factors, int inverse,
                                  int* launches) {
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
  const size_t e = dtype == JAXCUDA_F32 ? 4 : 8;
  const size_t smem = (2 * (size_t)n + 2 * (size_t)max_radix) * sizeof(double) + 4 * (size_t)n * e;
  if (smem > 220 * 1024) return cudaErrorInvalidValue;    // n up to 6.8 K (float32) / 4.5 K (float64) per row
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

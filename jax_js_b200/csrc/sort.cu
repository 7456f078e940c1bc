// Sort / Argsort routines (src/routine.ts:32-42): sort along the last axis of a
// contiguous [batch, n] array.
//
//   Sort     numeric order of TypedArray.prototype.sort (src/routine.ts:185-193):
//            -0 before +0, NaN last.
//   Argsort  stable; NaNs equal to each other and last, -0 == +0, ties by index
//            (src/routine.ts:195-214); outputs the gathered values and int32 indices.
//
// Both are compare-only, so results are bit-exact.  Values are mapped to order-preserving
// uint32 keys and sorted with a bitonic network: one CTA per row in shared memory while the
// padded row fits (the reference's WGSL routine has the same shape,
// src/backend/webgpu/routines.ts:57-261), otherwise chunk sorts in shared memory joined by
// global compare-exchange passes.  Argsort sorts (key, index) pairs as one 64-bit composite,
// which makes the network's result the stable order.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/jaxcuda_ir.h"

namespace jaxcuda_sort {

__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
  return f;
}
__device__ __forceinline__ uint16_t float_to_half_bits(float f) {
  uint16_t h;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
  return h;
}

// Order-preserving key of element `i` of a row.  canon: Argsort's equalities.
__device__ __forceinline__ uint32_t make_key(const void* row, int dtype, int64_t i, bool canon) {
  uint32_t bits;
  if (dtype == JAXCUDA_F16) bits = __float_as_uint(half_bits_to_float(((const uint16_t*)row)[i]));
  else bits = ((const uint32_t*)row)[i];
  if (dtype == JAXCUDA_U32) return bits;
  if (dtype == JAXCUDA_I32 || dtype == JAXCUDA_BOOL) return bits ^ 0x80000000u;
  const bool nan = (bits & 0x7fffffffu) > 0x7f800000u;
  if (nan) return canon ? 0xffffffffu : (0xffc00000u | (bits & 0x003fffffu));
  if (canon && bits == 0x80000000u) bits = 0;  // -0 == +0
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ void store_from_key(void* row, int dtype, int64_t i, uint32_t key) {
  uint32_t bits;
  if (dtype == JAXCUDA_U32) bits = key;
  else if (dtype == JAXCUDA_I32 || dtype == JAXCUDA_BOOL) bits = key ^ 0x80000000u;
  else bits = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
  if (dtype == JAXCUDA_F16) ((uint16_t*)row)[i] = float_to_half_bits(__uint_as_float(bits));
  else ((uint32_t*)row)[i] = bits;
}

__device__ __forceinline__ void copy_elem(void* dst, const void* src, int dtype, int64_t di, int64_t si) {
  if (dtype == JAXCUDA_F16) ((uint16_t*)dst)[di] = ((const uint16_t*)src)[si];
  else ((uint32_t*)dst)[di] = ((const uint32_t*)src)[si];
}

template <bool ARG> struct Item;
template <> struct Item<false> { typedef uint32_t T; };
template <> struct Item<true> { typedef unsigned long long T; };

template <bool ARG>
__device__ __forceinline__ typename Item<ARG>::T load_item(const void* row, int dtype, int64_t n, int64_t i) {
  if (ARG) {
    uint32_t key = i < n ? make_key(row, dtype, i, true) : 0xffffffffu;
    return (typename Item<ARG>::T)(((unsigned long long)key << 32) | (uint32_t)i);
  }
  return (typename Item<ARG>::T)(i < n ? make_key(row, dtype, i, false) : 0xffffffffu);
}

template <class T>
__device__ __forceinline__ void cmpx(T& a, T& b, bool up) {
  if ((a > b) == up) { T t = a; a = b; b = t; }
}

// All compare-exchange steps (k, j) with j < span, for k from k_lo to k_hi, on `cnt` items in
// shared memory whose first item has global position `base` in the padded row.
template <class T>
__device__ __forceinline__ void bitonic_smem(T* s, int cnt, int64_t base, int64_t k_lo, int64_t k_hi) {
  for (int64_t k = k_lo; k <= k_hi; k <<= 1) {
    for (int64_t j = (k >> 1) < cnt ? (k >> 1) : (cnt >> 1); j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < cnt / 2; t += blockDim.x) {
        const int lo = (int)(((int64_t)t / j) * 2 * j + (t % j));
        const bool up = (((base + lo) & k) == 0);
        cmpx(s[lo], s[lo + j], up);
      }
      __syncthreads();
    }
  }
}

// Whole padded row (P items) fits in shared memory: one CTA per row.
template <bool ARG>
__global__ void sort_rows_smem(const void* x, void* y, int32_t* yi, int dtype, int64_t n, int P) {
  typedef typename Item<ARG>::T T;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* s = (T*)smem_raw;
  const int eb = dtype == JAXCUDA_F16 ? 2 : 4;
  const unsigned char* xr = (const unsigned char*)x + (size_t)blockIdx.x * n * eb;
  unsigned char* yr = (unsigned char*)y + (size_t)blockIdx.x * n * eb;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s[i] = load_item<ARG>(xr, dtype, n, i);
  __syncthreads();
  bitonic_smem(s, P, 0, 2, P);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    if (ARG) {
      const uint32_t src = (uint32_t)s[i];
      yi[(size_t)blockIdx.x * n + i] = (int32_t)src;
      copy_elem(yr, xr, dtype, i, src);
    } else {
      store_from_key(yr, dtype, i, (uint32_t)s[i]);
    }
  }
}

// Large rows: items live in a global work buffer of batch * P items.
template <bool ARG>
__global__ void sort_fill(const void* x, typename Item<ARG>::T* work, int dtype, int64_t n, int64_t P, int64_t total) {
  const int eb = dtype == JAXCUDA_F16 ? 2 : 4;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = t / P, i = t % P;
    work[t] = load_item<ARG>((const unsigned char*)x + (size_t)row * n * eb, dtype, n, i);
  }
}

// Chunk of C items per CTA: steps with j < C for every k in [k_lo, k_hi].
template <class T>
__global__ void sort_chunks(T* work, int C, int64_t P, int64_t k_lo, int64_t k_hi) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* s = (T*)smem_raw;
  const int64_t start = (int64_t)blockIdx.x * C;
  for (int i = threadIdx.x; i < C; i += blockDim.x) s[i] = work[start + i];
  __syncthreads();
  bitonic_smem(s, C, start % P, k_lo, k_hi);
  for (int i = threadIdx.x; i < C; i += blockDim.x) work[start + i] = s[i];
}

template <class T>
__global__ void sort_global_step(T* work, int64_t P, int64_t k, int64_t j, int64_t pairs) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < pairs; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t lo = (t / j) * 2 * j + (t % j);
    const bool up = (((lo % P) & k) == 0);
    T a = work[lo], b = work[lo + j];
    if ((a > b) == up) { work[lo] = b; work[lo + j] = a; }
  }
}

template <bool ARG>
__global__ void sort_drain(const typename Item<ARG>::T* work, const void* x, void* y, int32_t* yi, int dtype,
                           int64_t n, int64_t P, int64_t total) {
  const int eb = dtype == JAXCUDA_F16 ? 2 : 4;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = t / n, i = t % n;
    const typename Item<ARG>::T it = work[row * P + i];
    unsigned char* yr = (unsigned char*)y + (size_t)row * n * eb;
    if (ARG) {
      const uint32_t src = (uint32_t)it;
      yi[t] = (int32_t)src;
      copy_elem(yr, (const unsigned char*)x + (size_t)row * n * eb, dtype, i, src);
    } else {
      store_from_key(yr, dtype, i, (uint32_t)it);
    }
  }
}

template <bool ARG>
cudaError_t run(cudaStream_t st, const void* x, void* y, int32_t* yi, int dtype, int64_t batch, int64_t n,
                void* work, int* launches) {
  typedef typename Item<ARG>::T T;
  int64_t P = 2;
  while (P < n) P <<= 1;
  const int64_t smem_items = ARG ? 16384 : 32768;  // 128 KiB of items
  if (P <= smem_items) {
    const int threads = (int)(P / 2 < 32 ? 32 : P / 2 > 1024 ? 1024 : P / 2);
    const size_t smem = (size_t)P * sizeof(T);
    cudaError_t e = cudaFuncSetAttribute(sort_rows_smem<ARG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return e;
    sort_rows_smem<ARG><<<(unsigned)batch, threads, smem, st>>>(x, y, yi, dtype, n, (int)P);
    (*launches)++;
    return cudaGetLastError();
  }
  T* w = (T*)work;
  const int C = (int)smem_items / 2;  // chunk items (64 KiB of shared memory)
  const int64_t total = batch * P;
  const unsigned wide = (unsigned)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256);
  cudaError_t e = cudaFuncSetAttribute(sort_chunks<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  if (e != cudaSuccess) return e;
  sort_fill<ARG><<<wide, 256, 0, st>>>(x, w, dtype, n, P, total);
  sort_chunks<T><<<(unsigned)(total / C), 1024, (size_t)C * sizeof(T), st>>>(w, C, P, 2, C);
  *launches += 2;
  for (int64_t k = (int64_t)C * 2; k <= P; k <<= 1) {
    for (int64_t j = k >> 1; j >= C; j >>= 1) {
      sort_global_step<T><<<wide, 256, 0, st>>>(w, P, k, j, total / 2);
      (*launches)++;
    }
    sort_chunks<T><<<(unsigned)(total / C), 1024, (size_t)C * sizeof(T), st>>>(w, C, P, k, k);
    (*launches)++;
  }
  const int64_t out_total = batch * n;
  sort_drain<ARG><<<(unsigned)((out_total + 255) / 256 > 148 * 32 ? 148 * 32 : (out_total + 255) / 256), 256, 0, st>>>(
      w, x, y, yi, dtype, n, P, out_total);
  (*launches)++;
  return cudaGetLastError();
}

}  // namespace jaxcuda_sort

// Bytes of global work space a sort of rows of n items needs (0 when rows fit in shared memory).
extern "C" size_t jaxcuda_sort_work_bytes(int argsort, int64_t batch, int64_t n) {
  int64_t P = 2;
  while (P < n) P <<= 1;
  const int64_t smem_items = argsort ? 16384 : 32768;
  if (P <= smem_items) return 0;
  return (size_t)batch * P * (argsort ? 8 : 4);
}

extern "C" int jaxcuda_sort_launch(void* stream, int argsort, const void* x, void* y, int32_t* yi, int dtype,
                                   int64_t batch, int64_t n, void* work, int* launches) {
  cudaStream_t st = (cudaStream_t)stream;
  if (batch == 0 || n == 0) return 0;
  return (int)(argsort ? jaxcuda_sort::run<true>(st, x, y, yi, dtype, batch, n, work, launches)
                       : jaxcuda_sort::run<false>(st, x, y, yi, dtype, batch, n, work, launches));
}

// ---- Sort without any allocation --------------------------------------------------------------
//
// jaxcuda_dispatch takes the work buffer of a large-row sort from the context's allocator, which
// may call cudaMalloc.  Some embedders cannot afford that call: a process that has handed all of
// the GPU's memory to its own pool (cudaMalloc then fails, or eats into a reserve), and serving
// loops in which the implicit device-wide synchronisation of cudaMalloc is a latency spike.  For
// them the same sort is offered over a work buffer that is part of the library image itself: a
// fixed array in device global memory.  Every GPU that loads the library holds these 16 MiB until
// the process exits, whether or not the entry point is ever called.
#define JX_SORT_STATIC_ITEMS (4 * 1024 * 1024) /* padded keys: batch * next_pow2(n) may not exceed this */
static __device__ __align__(256) uint32_t jx_sort_static_work[JX_SORT_STATIC_ITEMS];

// In host code the array's name is only a handle for the runtime, not an address a kernel could
// use; the device address is looked up once per device and cached here.
static void* g_static_work_addr[64] = {};

// Sorts each row of a contiguous [batch, n] array along the last axis (same order as the Sort
// routine: numeric, -0 before +0, NaN last) from device pointer x to device pointer y, on `stream`,
// without allocating host or device memory.  The device that owns x, y and the stream must be
// current.  dtype is a jaxcuda_dtype other than float64.
//
// Limits and rules:
//   * batch * P <= 4 Mi keys, P = n rounded up to a power of two (rows of up to 32768 keys are
//     sorted in shared memory and do not touch the static buffer at all); larger inputs are
//     rejected with JAXCUDA_EINVAL and a message in `err`.
//   * The first call on a device resolves the buffer's device address (cudaGetSymbolAddress); make
//     that first call outside any stream capture.
//   * All calls share the one buffer and it keeps whatever the previous call left there.  Nothing in
//     it has to start at zero: each call overwrites every key slot it later reads.  Two calls that
//     overlap on the GPU (different streams) race on it; keep them on one stream or order them.
extern "C" int jaxcuda_sort_no_alloc(void* stream, int dtype, const void* x, void* y, int64_t batch, int64_t n,
                                     char* err, size_t err_len) {
  auto fail = [&](int status, const char* msg) {
    if (err && err_len) snprintf(err, err_len, "%s", msg);
    return status;
  };
  if (err && err_len) err[0] = '\0';
  if (batch < 0 || n < 0 || (batch > 0 && n > 0 && (!x || !y))) return fail(3, "sort_no_alloc: null buffer or negative size");
  if (dtype < 0 || dtype > JAXCUDA_F16) return fail(2, "sort_no_alloc: dtype not supported (float64 has no 32-bit key)");
  if (batch == 0 || n == 0) return 0;
  if (n >= ((int64_t)1 << 31)) return fail(3, "sort_no_alloc: axis too long");
  int64_t P = 2;
  while (P < n) P <<= 1;
  if (P > 32768 && (batch > JX_SORT_STATIC_ITEMS / P)) {
    char msg[200];
    snprintf(msg, sizeof msg, "sort_no_alloc: %lld rows of %lld keys pad to %lld keys, the static work buffer holds %d",
             (long long)batch, (long long)n, (long long)(batch * P), JX_SORT_STATIC_ITEMS);
    return fail(3, msg);
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(5, "sort_no_alloc: no current CUDA device");
  if (!g_static_work_addr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, jx_sort_static_work);
    if (e != cudaSuccess || !p) return fail(5, cudaGetErrorString(e));
    g_static_work_addr[dev] = p;
  }
  int launches = 0;
  cudaError_t e = jaxcuda_sort::run<false>((cudaStream_t)stream, x, y, nullptr, dtype, batch, n, g_static_work_addr[dev], &launches);
  if (e != cudaSuccess) return fail(5, cudaGetErrorString(e));
  return 0;
}

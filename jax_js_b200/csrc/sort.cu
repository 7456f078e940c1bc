// Sort / Argsort routines (src/routine.ts:32-42): sort along the last axis of a
// contiguous [batch, n] array.
//
//   Sort     numeric order of TypedArray.prototype.sort (src/routine.ts:185-193):
//            -0 before +0, NaN last.
//   Argsort  stable; NaNs equal to each other and last, -0 == +0, ties by index
//            (src/routine.ts:195-214); outputs the gathered values and int32 indices.
//
// Both are compare-only, so results are bit-exact.  Values are mapped to order-preserving
// unsigned keys (32 bits; 64 bits for float64) and sorted with a bitonic network: one CTA per row in shared memory while the
// padded row fits (the reference's WGSL routine has the same shape,
// src/backend/webgpu/routines.ts:57-261), otherwise chunk sorts in shared memory joined by
// global compare-exchange passes.  Argsort sorts (key, index) pairs as one 64-bit composite,
// which makes the network's result the stable order.
#include <atomic>
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

// float64: the same mapping on 64 bits.
__device__ __forceinline__ unsigned long long make_key64(const void* row, int64_t i, bool canon) {
  unsigned long long bits = ((const unsigned long long*)row)[i];
  const bool nan = (bits & 0x7fffffffffffffffull) > 0x7ff0000000000000ull;
  if (nan) return canon ? ~0ull : (0xfff8000000000000ull | (bits & 0x0007ffffffffffffull));
  if (canon && bits == 0x8000000000000000ull) bits = 0;
  return (bits & 0x8000000000000000ull) ? ~bits : (bits | 0x8000000000000000ull);
}
__device__ __forceinline__ unsigned long long bits_from_key64(unsigned long long key) {
  return (key & 0x8000000000000000ull) ? (key & 0x7fffffffffffffffull) : ~key;
}

// A 64-bit key with the element's index: Argsort of float64.
struct KeyIndex {
  unsigned long long key;
  unsigned long long idx;
  __device__ __forceinline__ bool operator>(const KeyIndex& o) const { return key > o.key || (key == o.key && idx > o.idx); }
};

// ARG: Argsort (items carry the index); WIDE: float64 (64-bit keys).
template <bool ARG, bool WIDE> struct Item;
template <> struct Item<false, false> { typedef uint32_t T; };
template <> struct Item<true, false> { typedef unsigned long long T; };
template <> struct Item<false, true> { typedef unsigned long long T; };
template <> struct Item<true, true> { typedef KeyIndex T; };

__device__ __forceinline__ uint32_t item_index(unsigned long long it) { return (uint32_t)it; }
__device__ __forceinline__ uint32_t item_index(const KeyIndex& it) { return (uint32_t)it.idx; }
__device__ __forceinline__ uint32_t item_index(uint32_t) { return 0; }

template <bool ARG, bool WIDE>
__device__ __forceinline__ typename Item<ARG, WIDE>::T load_item(const void* row, int dtype, int64_t n, int64_t i) {
  typedef typename Item<ARG, WIDE>::T T;
  if constexpr (WIDE && ARG) {
    KeyIndex it;
    it.key = i < n ? make_key64(row, i, true) : ~0ull;
    it.idx = (unsigned long long)i;
    return it;
  } else if constexpr (WIDE) {
    return (T)(i < n ? make_key64(row, i, false) : ~0ull);
  } else if constexpr (ARG) {
    uint32_t key = i < n ? make_key(row, dtype, i, true) : 0xffffffffu;
    return (T)(((unsigned long long)key << 32) | (uint32_t)i);
  } else {
    return (T)(i < n ? make_key(row, dtype, i, false) : 0xffffffffu);
  }
}

// Writes output element i of a row from its sorted item (Sort: the key mapped back; Argsort: the
// index and the value gathered from the input row).
template <bool ARG, bool WIDE>
__device__ __forceinline__ void store_item(const typename Item<ARG, WIDE>::T& it, const void* xr, void* yr, int32_t* yi_row,
                                           int dtype, int64_t i) {
  if constexpr (ARG) {
    const uint32_t src = item_index(it);
    yi_row[i] = (int32_t)src;
    if constexpr (WIDE) ((unsigned long long*)yr)[i] = ((const unsigned long long*)xr)[src];
    else copy_elem(yr, xr, dtype, i, src);
  } else if constexpr (WIDE) {
    ((unsigned long long*)yr)[i] = bits_from_key64(it);
  } else {
    store_from_key(yr, dtype, i, (uint32_t)it);
  }
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
__device__ __forceinline__ int elem_bytes(int dtype) { return dtype == JAXCUDA_F16 ? 2 : dtype == JAXCUDA_F64 ? 8 : 4; }

template <bool ARG, bool WIDE>
__global__ void sort_rows_smem(const void* x, void* y, int32_t* yi, int dtype, int64_t n, int P) {
  typedef typename Item<ARG, WIDE>::T T;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* s = (T*)smem_raw;
  const int eb = elem_bytes(dtype);
  const unsigned char* xr = (const unsigned char*)x + (size_t)blockIdx.x * n * eb;
  unsigned char* yr = (unsigned char*)y + (size_t)blockIdx.x * n * eb;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s[i] = load_item<ARG, WIDE>(xr, dtype, n, i);
  __syncthreads();
  bitonic_smem(s, P, 0, 2, P);
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    store_item<ARG, WIDE>(s[i], xr, yr, ARG ? yi + (size_t)blockIdx.x * n : nullptr, dtype, i);
}

// Large rows: items live in a global work buffer of batch * P items.
template <bool ARG, bool WIDE>
__global__ void sort_fill(const void* x, typename Item<ARG, WIDE>::T* work, int dtype, int64_t n, int64_t P, int64_t total) {
  const int eb = elem_bytes(dtype);
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = t / P, i = t % P;
    work[t] = load_item<ARG, WIDE>((const unsigned char*)x + (size_t)row * n * eb, dtype, n, i);
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

template <bool ARG, bool WIDE>
__global__ void sort_drain(const typename Item<ARG, WIDE>::T* work, const void* x, void* y, int32_t* yi, int dtype,
                           int64_t n, int64_t P, int64_t total) {
  const int eb = elem_bytes(dtype);
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = t / n, i = t % n;
    store_item<ARG, WIDE>(work[row * P + i], (const unsigned char*)x + (size_t)row * n * eb,
                          (unsigned char*)y + (size_t)row * n * eb, ARG ? yi + row * n : nullptr, dtype, i);
  }
}

template <bool ARG, bool WIDE>
cudaError_t run(cudaStream_t st, const void* x, void* y, int32_t* yi, int dtype, int64_t batch, int64_t n,
                void* work, int* launches) {
  typedef typename Item<ARG, WIDE>::T T;
  int64_t P = 2;
  while (P < n) P <<= 1;
  const int64_t smem_items = (128 * 1024) / (int64_t)sizeof(T);  // 128 KiB of items
  if (P <= smem_items) {
    const int threads = (int)(P / 2 < 32 ? 32 : P / 2 > 1024 ? 1024 : P / 2);
    const size_t smem = (size_t)P * sizeof(T);
    cudaError_t e = cudaFuncSetAttribute(sort_rows_smem<ARG, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return e;
    sort_rows_smem<ARG, WIDE><<<(unsigned)batch, threads, smem, st>>>(x, y, yi, dtype, n, (int)P);
    (*launches)++;
    return cudaGetLastError();
  }
  T* w = (T*)work;
  const int C = (int)smem_items / 2;  // chunk items (64 KiB of shared memory)
  const int64_t total = batch * P;
  const unsigned wide = (unsigned)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256);
  cudaError_t e = cudaFuncSetAttribute(sort_chunks<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  if (e != cudaSuccess) return e;
  sort_fill<ARG, WIDE><<<wide, 256, 0, st>>>(x, w, dtype, n, P, total);
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
  sort_drain<ARG, WIDE><<<(unsigned)((out_total + 255) / 256 > 148 * 32 ? 148 * 32 : (out_total + 255) / 256), 256, 0, st>>>(
      w, x, y, yi, dtype, n, P, out_total);
  (*launches)++;
  return cudaGetLastError();
}

}  // namespace jaxcuda_sort

// Bytes of global work space a sort of rows of n items needs (0 when rows fit in shared memory).
extern "C" size_t jaxcuda_sort_work_bytes(int argsort, int dtype, int64_t batch, int64_t n) {
  int64_t P = 2;
  while (P < n) P <<= 1;
  const int64_t item = dtype == JAXCUDA_F64 ? (argsort ? 16 : 8) : (argsort ? 8 : 4);
  if (P <= (128 * 1024) / item) return 0;
  return (size_t)batch * P * item;
}

extern "C" int jaxcuda_sort_launch(void* stream, int argsort, const void* x, void* y, int32_t* yi, int dtype,
                                   int64_t batch, int64_t n, void* work, int* launches) {
  cudaStream_t st = (cudaStream_t)stream;
  if (batch == 0 || n == 0) return 0;
  if (dtype == JAXCUDA_F64)
    return (int)(argsort ? jaxcuda_sort::run<true, true>(st, x, y, yi, dtype, batch, n, work, launches)
                         : jaxcuda_sort::run<false, true>(st, x, y, yi, dtype, batch, n, work, launches));
  return (int)(argsort ? jaxcuda_sort::run<true, false>(st, x, y, yi, dtype, batch, n, work, launches)
                       : jaxcuda_sort::run<false, false>(st, x, y, yi, dtype, batch, n, work, launches));
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
// Two threads that make a device's first call at once both look the address up and store the same
// value; the slots are atomic so that neither reads a torn pointer.
static std::atomic<void*> g_static_work_addr[64];

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
  // the static buffer that is looked up below belongs to the current device: the data must live there too
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, x) == cudaSuccess && at.type == cudaMemoryTypeDevice && at.device != dev)
    return fail(3, "sort_no_alloc: the input lives on another device than the current one");
  void* work = g_static_work_addr[dev].load(std::memory_order_acquire);
  if (!work) {
    cudaError_t e = cudaGetSymbolAddress(&work, jx_sort_static_work);
    if (e != cudaSuccess || !work) return fail(5, cudaGetErrorString(e));
    g_static_work_addr[dev].store(work, std::memory_order_release);
  }
  int launches = 0;
  cudaError_t e = jaxcuda_sort::run<false, false>((cudaStream_t)stream, x, y, nullptr, dtype, batch, n, work, &launches);
  if (e != cudaSuccess) return fail(5, cudaGetErrorString(e));
  return 0;
}

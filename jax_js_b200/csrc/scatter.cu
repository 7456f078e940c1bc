// Scatter routine (src/routine.ts:44-48, CPU reference runScatter :226-296): updates are written
// or accumulated into a zero-filled output at positions given by one int32 index array per
// indexed output axis; the updates array has the non-indexed output dimensions with the
// broadcast index dimensions inserted at `outDim`.  One thread per update element; out-of-range
// coordinates drop the update.
//
//   update, unique indices      plain stores
//   update, possibly repeated   the reference's loop lets the highest update index win: a first
//                               pass takes atomicMax of the update index per destination, a second
//                               writes the winners (deterministic, bit-exact)
//   add                         atomicAdd (integers wrap; float sums depend on arrival order within
//                               rounding), Bool accumulates with OR
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jaxcuda_ir.h"
#include "scatter.hpp"

namespace {

__device__ __forceinline__ long long destination(const jaxcuda_scatter_desc& d, const int32_t* const* idx, long long i) {
  long long out = 0;
  int free_dim = 0;
  for (int ax = 0; ax < d.out_rank; ax++) {
    const int which = d.axis_to_index[ax];
    long long coord;
    if (which < 0) {
      const int ud = d.free_dims[free_dim++];
      coord = (i / d.upd_stride[ud]) % d.upd_shape[ud];
    } else {
      const int first = d.out_dim + d.index_rank - d.idx_rank[which];
      long long off = 0;
      for (int j = 0; j < d.idx_rank[which]; j++) {
        if (d.idx_shape[which][j] == 1) continue;
        const int ud = first + j;
        off += ((i / d.upd_stride[ud]) % d.upd_shape[ud]) * d.idx_stride[which][j];
      }
      coord = idx[which][off];
    }
    if (coord < 0 || coord >= d.out_shape[ax]) return -1;
    out += coord * d.out_stride[ax];
  }
  return out;
}

struct IndexPtrs { const int32_t* p[8]; };

template <class T>
__device__ __forceinline__ void accumulate(T* dst, T v) { atomicAdd(dst, v); }
template <>
__device__ __forceinline__ void accumulate<int32_t>(int32_t* dst, int32_t v) { atomicAdd((unsigned*)dst, (unsigned)v); }

template <class T>
__global__ void scatter_kernel(jaxcuda_scatter_desc d, IndexPtrs idx, const T* upd, T* out, int* winner, int pass) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.n_updates; i += (long long)gridDim.x * blockDim.x) {
    const long long at = destination(d, idx.p, i);
    if (at < 0) continue;
    if (d.mode == 0) {
      if (!winner) out[at] = upd[i];
      else if (pass == 0) atomicMax(&winner[at], (int)i);
      else if (winner[at] == (int)i) out[at] = upd[i];
    } else if (d.mode == 2) {
      atomicOr((unsigned*)&out[at], (unsigned)upd[i]);
    } else {
      accumulate(&out[at], upd[i]);
    }
  }
}
template <>
__global__ void scatter_kernel<__half>(jaxcuda_scatter_desc d, IndexPtrs idx, const __half* upd, __half* out, int* winner, int pass) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.n_updates; i += (long long)gridDim.x * blockDim.x) {
    const long long at = destination(d, idx.p, i);
    if (at < 0) continue;
    if (d.mode == 0) {
      if (!winner) out[at] = upd[i];
      else if (pass == 0) atomicMax(&winner[at], (int)i);
      else if (winner[at] == (int)i) out[at] = upd[i];
    } else {
      atomicAdd(&out[at], upd[i]);
    }
  }
}

template <class T>
cudaError_t launch(cudaStream_t st, const jaxcuda_scatter_desc& d, const IndexPtrs& idx, const void* upd, void* out,
                   int* winner, int* launches) {
  if (d.n_updates == 0) return cudaSuccess;
  const unsigned blocks = (unsigned)((d.n_updates + 255) / 256 > 148 * 32 ? 148 * 32 : (d.n_updates + 255) / 256);
  const int passes = (d.mode == 0 && winner) ? 2 : 1;
  for (int pass = 0; pass < passes; pass++) {
    scatter_kernel<T><<<blocks, 256, 0, st>>>(d, idx, (const T*)upd, (T*)out, winner, pass);
    (*launches)++;
  }
  return cudaGetLastError();
}

}  // namespace

// Bytes of work space: one int per output element when repeated indices must resolve to the last update.
extern "C" size_t jaxcuda_scatter_work_bytes(const jaxcuda_scatter_desc* d) {
  return (d->mode == 0 && !d->unique) ? (size_t)d->out_size * 4 : 0;
}

extern "C" int jaxcuda_scatter_launch(void* stream, const jaxcuda_scatter_desc* d, const void* updates,
                                      const void* const* indices, void* out, void* work, int* launches) {
  cudaStream_t st = (cudaStream_t)stream;
  const int eb = d->dtype == JAXCUDA_F16 ? 2 : d->dtype == JAXCUDA_F64 ? 8 : 4;
  cudaError_t e = cudaSuccess;
  if (d->out_size) e = cudaMemsetAsync(out, 0, (size_t)d->out_size * eb, st);   // the routine zero-fills its output
  if (e != cudaSuccess) return (int)e;
  int* winner = nullptr;
  if (d->mode == 0 && !d->unique && d->n_updates) {
    winner = (int*)work;
    e = cudaMemsetAsync(winner, 0xff, (size_t)d->out_size * 4, st);              // -1: no update yet
    if (e != cudaSuccess) return (int)e;
  }
  IndexPtrs idx;
  for (int k = 0; k < 8; k++) idx.p[k] = k < d->n_index ? (const int32_t*)indices[k] : nullptr;
  switch (d->dtype) {
    case JAXCUDA_F32: e = launch<float>(st, *d, idx, updates, out, winner, launches); break;
    case JAXCUDA_F64: e = launch<double>(st, *d, idx, updates, out, winner, launches); break;
    case JAXCUDA_F16: e = launch<__half>(st, *d, idx, updates, out, winner, launches); break;
    case JAXCUDA_U32: e = launch<unsigned>(st, *d, idx, updates, out, winner, launches); break;
    default: e = launch<int32_t>(st, *d, idx, updates, out, winner, launches); break;
  }
  return (int)e;
}

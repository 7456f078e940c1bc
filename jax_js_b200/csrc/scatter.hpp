// Geometry of one Scatter routine instance, precomputed on the host from `RoutineType` and
// `ScatterParams` (src/routine.ts:104-123) and passed to the kernel by value.
#pragma once

#include <stddef.h>

struct jaxcuda_scatter_desc {
  int out_rank, upd_rank, n_index, index_rank, out_dim;
  int mode;    // 0 store, 1 add, 2 or (Bool add)
  int unique;  // indices promised unique: stores need no ordering pass
  int dtype;   // jaxcuda_dtype of updates and output
  long long out_shape[8], out_stride[8];
  int axis_to_index[8];  // per output axis: which index input addresses it, or -1
  long long upd_shape[8], upd_stride[8];
  int free_dims[8];      // update dimensions that carry the non-indexed output axes, in order
  int idx_rank[8];
  long long idx_shape[8][8], idx_stride[8][8];
  long long n_updates, out_size;
};

extern "C" size_t jaxcuda_scatter_work_bytes(const jaxcuda_scatter_desc* d);
extern "C" int jaxcuda_scatter_launch(void* stream, const jaxcuda_scatter_desc* d, const void* updates,
                                      const void* const* indices, void* out, void* work, int* launches);

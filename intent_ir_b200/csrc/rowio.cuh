// Register-resident row I/O shared by the row kernels (softmax, normalisation): a row of
// `cols` elements is spread over `nthreads` threads, NV vectors of 4 elements per thread.
#pragma once
#include "common.cuh"

namespace ib200 {

// Load this thread's NV vectors of 4 elements: vector i covers columns 4*(i*nthreads + tid).
template <typename T, int NV, bool VEC>
__device__ __forceinline__ void load_row(const T* __restrict__ row, int cols, int tid, int nthreads, float pad, float (&v)[NV][4]) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * (i * nthreads + tid);
    if (VEC) {
      if (c < cols) load4<T>(row + c, v[i]);
      else { v[i][0] = v[i][1] = v[i][2] = v[i][3] = pad; }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[i][k] = (c + k < cols) ? to_f32<T>(row[c + k]) : pad;
    }
  }
}

template <typename T, int NV, bool VEC>
__device__ __forceinline__ void store_row(T* __restrict__ row, int cols, int tid, int nthreads, const float (&v)[NV][4]) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * (i * nthreads + tid);
    if (VEC) {
      if (c < cols) store4<T>(row + c, v[i]);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c + k < cols) row[c + k] = from_f32<T>(v[i][k]);
    }
  }
}

}  // namespace ib200

// Register-resident row I/O shared by the row kernels (softmax, normalisation): a row of
// `cols` elements is spread over `nthreads` threads, NV vectors of 4 elements per thread.
#pragma once
#include "common.cuh"

namespace ib200 {

// Rows are read once and written once: cache-streaming loads and stores (evict first) keep them from displacing what is
// reused (weights, masks, statistics).
template <typename T> __device__ __forceinline__ void load4_stream(const T* p, float (&v)[4]) { load4<T>(p, v); }
template <> __device__ __forceinline__ void load4_stream<float>(const float* p, float (&v)[4]) {
  const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <typename T> __device__ __forceinline__ void store4_stream(T* p, const float (&v)[4]) { store4<T>(p, v); }
template <> __device__ __forceinline__ void store4_stream<float>(float* p, const float (&v)[4]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
}

// Load this thread's NV vectors of 4 elements: vector i covers columns 4*(i*nthreads + tid).
template <typename T, int NV, bool VEC, bool STREAM = false>  // STREAM: global memory read once (never a staged copy in shared memory)
__device__ __forceinline__ void load_row(const T* __restrict__ row, int cols, int tid, int nthreads, float pad, float (&v)[NV][4]) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * (i * nthreads + tid);
    if (VEC) {
      if (c < cols) {
        if (STREAM) load4_stream<T>(row + c, v[i]);
        else load4<T>(row + c, v[i]);
      }
      else { v[i][0] = v[i][1] = v[i][2] = v[i][3] = pad; }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[i][k] = (c + k < cols) ? to_f32<T>(row[c + k]) : pad;
    }
  }
}

template <typename T, int NV, bool VEC, bool STREAM = false>
__device__ __forceinline__ void store_row(T* __restrict__ row, int cols, int tid, int nthreads, const float (&v)[NV][4]) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * (i * nthreads + tid);
    if (VEC) {
      if (c < cols) {
        if (STREAM) store4_stream<T>(row + c, v[i]);
        else store4<T>(row + c, v[i]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c + k < cols) row[c + k] = from_f32<T>(v[i][k]);
    }
  }
}

}  // namespace ib200

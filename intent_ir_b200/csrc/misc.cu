// Layout kernels that are not arithmetic: 2-D transpose through a padded shared-memory
// tile (coalesced 128-byte rows on both sides).  Replaces the generated transpose2d kernel
// of the reference (backends/cuda/codegen/intentir_to_cuda.py:1487-1550).
#include <cstring>

#include "common.cuh"

namespace ib200 {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int64_t cols) {
  __shared__ T tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
  for (int64_t t = blockIdx.x; t < tiles_c * tiles_r; t += gridDim.x) {
    const int64_t r0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
      const int64_t r = r0 + ty + k, c = c0 + tx;
      if (r < rows && c < cols) tile[ty + k][tx] = x[r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
      const int64_t c = c0 + ty + k, r = r0 + tx;
      if (r < rows && c < cols) out[c * rows + r] = tile[tx][ty + k];
    }
    __syncthreads();
  }
}

template <typename T, typename I>
__global__ void __launch_bounds__(256) gather_kernel(const T* __restrict__ data, GatherArgs a, T* __restrict__ out, T other) {
  for (int64_t l = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; l < a.n; l += (int64_t)gridDim.x * blockDim.x) {
    int64_t off = 0;
    bool inside = true;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (k >= a.n_idx) break;
      int64_t i = (int64_t)static_cast<const I*>(a.idx[k])[l];
      if (i < 0) i += a.dim[k];  // numpy wraps negative indices
      inside &= i >= 0 && i < a.dim[k];
      off += i * a.stride[k];
    }
    out[l] = inside ? data[off] : other;
  }
}

template <typename T> int run_gather(const void* data, const GatherArgs& a, void* out, double other, cudaStream_t s) {
  const int64_t blocks = (a.n + 255) / 256;
  const int grid = (int)(blocks < (int64_t)kSmCount * 16 ? blocks : (int64_t)kSmCount * 16);
  T fill;
  if (sizeof(T) == 4) { float f = (float)other; std::memcpy(&fill, &f, sizeof(T)); }
  else if (sizeof(T) == 2) { __nv_bfloat16 h = __float2bfloat16_rn((float)other); std::memcpy(&fill, &h, sizeof(T)); }
  else std::memset(&fill, other != 0.0, sizeof(T));
  if (a.idx_is_64) gather_kernel<T, long long><<<grid, 256, 0, s>>>(static_cast<const T*>(data), a, static_cast<T*>(out), fill);
  else gather_kernel<T, int><<<grid, 256, 0, s>>>(static_cast<const T*>(data), a, static_cast<T*>(out), fill);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "gather launch");
}

}  // namespace

// out[l] = data[idx0[l], idx1[l], ...] (one index tensor per data axis; numpy fancy indexing,
// verify/interpreter.py:284-291).  Out-of-range positions, which numpy rejects, read `other`
// (the reference CUDA backend's gather2d convention, intentir_to_cuda.py:1779-1832).
// `other` is converted as f32 / bf16 for 4- / 2-byte elements.
int launch_gather(const void* data, const GatherArgs& a, void* out, int elem_bytes, double other, cudaStream_t s) {
  if (a.n < 0 || a.n_idx < 1 || a.n_idx > 4) return fail(IB200_ERR_INVALID, "gather: bad arguments");
  if (a.n == 0) return IB200_OK;
  switch (elem_bytes) {
    case 4: return run_gather<uint32_t>(data, a, out, other, s);
    case 2: return run_gather<uint16_t>(data, a, out, other, s);
    case 1: return run_gather<uint8_t>(data, a, out, other, s);
    default: return fail(IB200_ERR_UNSUPPORTED, "gather: element size must be 1, 2 or 4 bytes");
  }
}

int launch_transpose2d(const void* x, void* out, int elem_bytes, int64_t rows, int64_t cols, cudaStream_t s) {
  if (rows < 0 || cols < 0) return fail(IB200_ERR_INVALID, "transpose2d: negative extent");
  if (rows == 0 || cols == 0) return IB200_OK;
  if (beyond_any_device(rows, cols)) return fail(IB200_ERR_INVALID, "transpose2d: more than 2^40 elements");
  if (!x || !out) return fail(IB200_ERR_INVALID, "transpose2d: null pointer");
  const int64_t tiles = ((rows + 31) / 32) * ((cols + 31) / 32);
  const int grid = (int)(tiles < (int64_t)kSmCount * 16 ? tiles : (int64_t)kSmCount * 16);
  switch (elem_bytes) {
    case 4: transpose_kernel<uint32_t><<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(out), rows, cols); break;
    case 2: transpose_kernel<uint16_t><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), rows, cols); break;
    case 1: transpose_kernel<uint8_t><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), rows, cols); break;
    case 8: transpose_kernel<uint64_t><<<grid, 256, 0, s>>>(static_cast<const uint64_t*>(x), static_cast<uint64_t*>(out), rows, cols); break;
    default: return fail(IB200_ERR_UNSUPPORTED, "transpose2d: element size must be 1, 2, 4 or 8 bytes");
  }
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "transpose2d launch");
}

}  // namespace ib200

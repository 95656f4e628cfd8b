// Layout kernels that are not arithmetic: 2-D transpose through a padded shared-memory
// tile (coalesced 128-byte rows on both sides).  Replaces the generated transpose2d kernel
// of the reference (backends/cuda/codegen/intentir_to_cuda.py:1487-1550).
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

}  // namespace

int launch_transpose2d(const void* x, void* out, int elem_bytes, int64_t rows, int64_t cols, cudaStream_t s) {
  if (rows < 0 || cols < 0) return fail(IB200_ERR_INVALID, "transpose2d: negative extent");
  if (rows == 0 || cols == 0) return IB200_OK;
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

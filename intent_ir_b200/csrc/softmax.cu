// Row softmax over the last axis, y = exp(x - max(x)) / sum(exp(x - max(x))), the form
// of verify/interpreter.py:501-506.  HBM-bound single pass: each row is read once into
// registers with 128-bit loads, reduced twice (max, then sum of exponentials) with warp
// shuffles, and written once.  exp runs on the special-function unit (ex2.approx) and the
// normalisation is one reciprocal per row.  No 1024-column ceiling (the reference's kernels/softmax.cuh
// stops there).
//
//   cols <= 1024          : one warp per row (no block barrier at all);
//   cols <= 16384         : one CTA per row, 256..1024 threads, 8..16 elements per thread;
//   larger rows           : one CTA per row streaming the row three times (the second and
//                           third pass hit L2); with scratch memory, rows too few to fill the
//                           GPU that way (or too large for L2) are cut into segments, one CTA
//                           each, in two launches (longrow.cu).
//
// Non-finite inputs need no special cases: IEEE arithmetic gives what numpy gives — a row
// holding NaN or +Inf, or only -Inf, becomes all-NaN; -Inf beside finite values gives 0.
#include <type_traits>

#include "common.cuh"
#include "rowio.cuh"

#ifndef SM_LD
#define SM_LD false
#define SM_ST false
#endif

namespace ib200 {
namespace {

// the masked form is built for f32 rows only
template <typename T, typename TO> constexpr bool kMaskBuilt = std::is_same<T, float>::value && std::is_same<TO, float>::value;

template <int NV> __device__ __forceinline__ float local_max(const float (&v)[NV][4]) {
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) m = max_nan(m, v[i][k]);
  return m;
}

// exp(t) as 2^(t*log2(e)) on the special-function unit: two instructions instead of the ~10 of
// expf.  Relative error ~2^-22 plus |t|*2^-24 from the product, far inside the verifier's
// 1e-4; exp2(-inf) = 0 and NaN propagates, so non-finite rows behave as with expf.
__device__ __forceinline__ float fast_exp(float t) {
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(t * 1.4426950408889634f));
  return r;
}

// v <- exp(v - m); returns the local sum.  Padding slots hold -inf and contribute exp(-inf) = 0
// unless m itself is -inf or NaN, in which case the whole row is NaN anyway.
template <int NV> __device__ __forceinline__ float exp_and_sum(float (&v)[NV][4], float m) {
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[i][k] = fast_exp(v[i][k] - m);
      s += v[i][k];
    }
  return s;
}

// v <- v / s, as one IEEE reciprocal per row and a multiply per element (<= 1.5 ulp from v / s)
template <int NV> __device__ __forceinline__ void scale(float (&v)[NV][4], float s) {
  const float inv = 1.0f / s;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) v[i][k] = v[i][k] * inv;
}

// v <- mask ? v : fill on the valid columns of this thread (the `where` in front of a masked softmax,
// pipeline/tilelang/core.py:1050-1076, applied as the row is loaded); padding keeps its -inf
template <int NV, bool VEC>
__device__ __forceinline__ void apply_mask(float (&v)[NV][4], const uint8_t* __restrict__ mrow, bool mask_vec, float fill, int cols, int tid,
                                           int nthreads) {
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = 4 * (i * nthreads + tid);
    if (VEC && mask_vec) {
      if (c < cols) {
        const uchar4 m = *reinterpret_cast<const uchar4*>(mrow + c);
        v[i][0] = m.x ? v[i][0] : fill; v[i][1] = m.y ? v[i][1] : fill; v[i][2] = m.z ? v[i][2] : fill; v[i][3] = m.w ? v[i][3] : fill;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c + k < cols) v[i][k] = mrow[c + k] ? v[i][k] : fill;
    }
  }
}

// all-reduce over aligned groups of LANES lanes (the whole warp takes part in every shuffle)
template <typename Op, int LANES> __device__ __forceinline__ float lanes_reduce(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// LANES lanes per row: 32 for rows of 65..1024 elements, 16 or 8 for shorter ones (2 or 4 rows per warp
// at a time, no lane holding only padding)
template <typename T, typename TO, int NV, bool VEC, int LANES, bool MASKED>
__global__ void __launch_bounds__(128) softmax_warp(const T* __restrict__ x, TO* __restrict__ y, float* __restrict__ row_max,
                                                    float* __restrict__ row_sum, int64_t rows, int cols, SoftmaxMask mk) {
  constexpr int kRowsPerWarp = 32 / LANES;
  const int lane = (threadIdx.x & 31) % LANES, which = (threadIdx.x & 31) / LANES;
  const int64_t stride = (int64_t)gridDim.x * (blockDim.x >> 5) * kRowsPerWarp;
  // the loop bound is the same for every lane of a warp: the shuffles need all of them
  for (int64_t r0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kRowsPerWarp; r0 < rows; r0 += stride) {
    const bool live = r0 + which < rows;
    const int64_t r = live ? r0 + which : rows - 1;  // lanes past the last row recompute it and store nothing
    float v[NV][4];
    load_row<T, NV, VEC, SM_LD>(x + r * cols, cols, lane, LANES, -INFINITY, v);
    if (MASKED) apply_mask<NV, VEC>(v, mk.mask + r * mk.row_stride, mk.vec != 0, mk.fill, cols, lane, LANES);
    const float m = lanes_reduce<MaxOp, LANES>(local_max<NV>(v));
    const float s = lanes_reduce<SumOp, LANES>(exp_and_sum<NV>(v, m));
    scale<NV>(v, s);
    if (live) {
      store_row<TO, NV, VEC, SM_ST>(y + r * cols, cols, lane, LANES, v);
      if (lane == 0) {
        if (row_max) row_max[r] = m;
        if (row_sum) row_sum[r] = s;
      }
    }
  }
}

template <typename T, typename TO, int THREADS, int NV, bool VEC, bool MASKED>
__global__ void __launch_bounds__(THREADS, (MASKED && THREADS == 256) ? 6 : 1) softmax_block(const T* __restrict__ x, TO* __restrict__ y,
                                                         float* __restrict__ row_max, float* __restrict__ row_sum,
                                                         int64_t rows, int cols, SoftmaxMask mk) {
  __shared__ float slots[2][32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float v[NV][4];
    load_row<T, NV, VEC, SM_LD>(x + r * cols, cols, threadIdx.x, THREADS, -INFINITY, v);
    if (MASKED) apply_mask<NV, VEC>(v, mk.mask + r * mk.row_stride, mk.vec != 0, mk.fill, cols, threadIdx.x, THREADS);
    const float m = block_reduce<MaxOp>(local_max<NV>(v), slots[0]);
    const float s = block_reduce<SumOp>(exp_and_sum<NV>(v, m), slots[1]);
    scale<NV>(v, s);
    store_row<TO, NV, VEC, SM_ST>(y + r * cols, cols, threadIdx.x, THREADS, v);
    if (threadIdx.x == 0) {
      if (row_max) row_max[r] = m;
      if (row_sum) row_sum[r] = s;
    }
  }
}

// Rows too long for registers: three passes over the row (max, sum, write).
template <typename T, typename TO>
__global__ void __launch_bounds__(1024) softmax_stream(const T* __restrict__ x, TO* __restrict__ y, float* __restrict__ row_max,
                                                       float* __restrict__ row_sum, int64_t rows, int64_t cols) {
  __shared__ float slots[2][32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    TO* yr = y + r * cols;
    float m = -INFINITY;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) m = max_nan(m, to_f32<T>(xr[c]));
    m = block_reduce<MaxOp>(m, slots[0]);
    float s = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += fast_exp(to_f32<T>(xr[c]) - m);
    s = block_reduce<SumOp>(s, slots[1]);
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = from_f32<TO>(fast_exp(to_f32<T>(xr[c]) - m) * (1.0f / s));
    if (threadIdx.x == 0) {
      if (row_max) row_max[r] = m;
      if (row_sum) row_sum[r] = s;
    }
  }
}

template <typename T, typename TO, int NV, bool VEC, int LANES = 32>
void launch_warp(const T* x, TO* y, float* mx, float* sm, int64_t rows, int cols, cudaStream_t s, const SoftmaxMask& mk) {
  const int64_t per_cta = 4 * (32 / LANES);
  const int64_t blocks = (rows + per_cta - 1) / per_cta;
  const int grid = (int)(blocks < (int64_t)kSmCount * 32 ? blocks : (int64_t)kSmCount * 32);
  if (!mk.mask) softmax_warp<T, TO, NV, VEC, LANES, false><<<grid, 128, 0, s>>>(x, y, mx, sm, rows, cols, mk);
  else if constexpr (kMaskBuilt<T, TO>) softmax_warp<T, TO, NV, VEC, LANES, true><<<grid, 128, 0, s>>>(x, y, mx, sm, rows, cols, mk);
}
template <typename T, typename TO, int THREADS, int NV, bool VEC>
void launch_block(const T* x, TO* y, float* mx, float* sm, int64_t rows, int cols, cudaStream_t s, const SoftmaxMask& mk) {
  const int per_sm = 2048 / THREADS;
  // about one row per CTA (measured best: the hardware scheduler balances better than a grid-stride loop)
  const int64_t cap = (int64_t)kSmCount * per_sm * 8;
  const int grid = (int)(rows < cap ? rows : cap);
  if (!mk.mask) softmax_block<T, TO, THREADS, NV, VEC, false><<<grid, THREADS, 0, s>>>(x, y, mx, sm, rows, cols, mk);
  else if constexpr (kMaskBuilt<T, TO>) softmax_block<T, TO, THREADS, NV, VEC, true><<<grid, THREADS, 0, s>>>(x, y, mx, sm, rows, cols, mk);
}

template <typename T, typename TO, bool VEC>
void dispatch(const T* x, TO* y, float* mx, float* sm, int64_t rows, int64_t cols, cudaStream_t s, const SoftmaxMask& mk) {
  const int c = (int)cols;
  if (cols <= 32) launch_warp<T, TO, 1, VEC, 8>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 64) launch_warp<T, TO, 1, VEC, 16>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 128) launch_warp<T, TO, 1, VEC>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 256) launch_warp<T, TO, 2, VEC>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 512) launch_warp<T, TO, 4, VEC>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 1024) launch_warp<T, TO, 8, VEC>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 2048) launch_block<T, TO, 256, 2, VEC>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 4096) launch_block<T, TO, 256, 4, VEC>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 8192) launch_block<T, TO, 512, 4, VEC>(x, y, mx, sm, rows, c, s, mk);
  else if (cols <= 16384) launch_block<T, TO, 1024, 4, VEC>(x, y, mx, sm, rows, c, s, mk);
  else {
    const int grid = (int)(rows < (int64_t)kSmCount * 2 ? rows : (int64_t)kSmCount * 2);
    softmax_stream<T, TO><<<grid, 1024, 0, s>>>(x, y, mx, sm, rows, cols);
  }
}

template <typename T, typename TO>
int run(const void* xv, void* yv, float* mx, float* sm, int64_t rows, int64_t cols, cudaStream_t s, SoftmaxMask mk) {
  if (mk.mask && (!kMaskBuilt<T, TO> || cols > 16384)) return fail(IB200_ERR_UNSUPPORTED, "softmax: the masked form covers f32 rows of up to 16384 elements");
  mk.vec = mk.mask && (reinterpret_cast<uintptr_t>(mk.mask) & 3u) == 0 && mk.row_stride % 4 == 0;
  const T* x = static_cast<const T*>(xv);
  TO* y = static_cast<TO*>(yv);
  // every row start is aligned to a 4-element vector when the bases are and cols % 4 == 0
  const bool vec = aligned16(x) && aligned16(y) && cols % 4 == 0;
  if (vec) dispatch<T, TO, true>(x, y, mx, sm, rows, cols, s, mk);
  else dispatch<T, TO, false>(x, y, mx, sm, rows, cols, s, mk);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "softmax launch");
}

}  // namespace

int launch_softmax(const void* x, void* y, float* row_max, float* row_sum, int dtype, int64_t rows, int64_t cols,
                   cudaStream_t s, int out_dtype, const SoftmaxMask* mask, void* scratch, size_t scratch_bytes) {
  const SoftmaxMask mk = mask ? *mask : SoftmaxMask{nullptr, 0, 0.0f, 0};
  if (out_dtype < 0) out_dtype = dtype;
  if (rows < 0 || cols < 0) return fail(IB200_ERR_INVALID, "softmax: negative extent");
  if (rows == 0 || cols == 0) return IB200_OK;
  if (beyond_any_device(rows, cols)) return fail(IB200_ERR_INVALID, "softmax: more than 2^40 elements");
  if (!x || !y) return fail(IB200_ERR_INVALID, "softmax: null pointer");
  if (!mk.mask && scratch) {  // few, very long rows: segments over the whole GPU
    const int rc = try_softmax_segmented(x, y, row_max, row_sum, dtype, out_dtype, rows, cols, scratch, scratch_bytes, s);
    if (rc != 1) return rc;
  }
  if (dtype == IB200_F32 && out_dtype == IB200_F32) return run<float, float>(x, y, row_max, row_sum, rows, cols, s, mk);
  if (dtype == IB200_BF16 && out_dtype == IB200_BF16) return run<__nv_bfloat16, __nv_bfloat16>(x, y, row_max, row_sum, rows, cols, s, mk);
  if (dtype == IB200_F16 && out_dtype == IB200_F16) return run<__half, __half>(x, y, row_max, row_sum, rows, cols, s, mk);
  if (dtype == IB200_BF16 && out_dtype == IB200_F32) return run<__nv_bfloat16, float>(x, y, row_max, row_sum, rows, cols, s, mk);
  if (dtype == IB200_F16 && out_dtype == IB200_F32) return run<__half, float>(x, y, row_max, row_sum, rows, cols, s, mk);
  return fail(IB200_ERR_UNSUPPORTED, "softmax: x must be f32, bf16 or f16; y the same type, or f32 for 16-bit inputs");
}

}  // namespace ib200

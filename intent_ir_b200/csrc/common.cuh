// Shared device/host helpers for the sm_100a kernels: element types, 128-bit loads and
// stores with on-the-fly conversion to fp32, NaN-propagating max/min, warp and block
// reductions, and the host-side error plumbing behind ib200_last_error().
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/intentir_b200.h"

namespace ib200 {

constexpr int kSmCount = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// ---- host-side error state ------------------------------------------------------------
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t err, const char* what);
#define IB200_CUDA_OK(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::ib200::cuda_fail(_e, #expr); \
  } while (0)

inline int dtype_size(int dt) {
  switch (dt) {
    case IB200_F32: case IB200_I32: return 4;
    case IB200_BF16: case IB200_F16: case IB200_I16: return 2;
    case IB200_I64: case IB200_F64: return 8;
    case IB200_BOOL: case IB200_U8: case IB200_I8: return 1;
    default: return 0;
  }
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
// Non-negative extents whose product is more than any device holds (2^40 elements), or wraps: arguments like that are
// uninitialised or mistaken, and index arithmetic downstream is only checked for sizes that can exist.
inline bool beyond_any_device(int64_t a, int64_t b = 1, int64_t c = 1) {
  int64_t n = 0;
  return __builtin_mul_overflow(a, b, &n) || __builtin_mul_overflow(n, c, &n) || n > ((int64_t)1 << 40);
}

// ---- internal launchers (one per .cu file) ----------------------------------------------
// `scratch` (device memory in any state, or null) lets a reduction with too few independent results to
// fill the GPU be split along the reduced axis; reduce_scratch_bytes says how much that takes (0: the
// shape is not split).  With less scratch than that the unsplit kernels run.
size_t reduce_scratch_bytes(int64_t outer, int64_t reduce, int64_t inner);
int launch_reduce(const void* x, void* out, int x_dtype, int out_dtype, int kind, int64_t outer,
                  int64_t reduce, int64_t inner, float scale, cudaStream_t s, void* scratch = nullptr, size_t scratch_bytes = 0);
struct SoftmaxMask {     // softmax(where(mask, x, fill)): the mask is applied while the rows are loaded
  const uint8_t* mask;   // bool / u8, or null for a plain softmax
  int64_t row_stride;    // elements between the mask rows of consecutive rows (0: one mask row for all)
  float fill;
  int vec;               // filled by the launcher: 4 mask bytes can be read as one word
};
// With scratch (softmax_scratch_bytes / norm_scratch_bytes say how much; 0: never used), rows too long for the
// resident kernels and too few to fill the GPU one CTA per row are cut into segments, one CTA each (longrow.cu).
int launch_softmax(const void* x, void* y, float* row_max, float* row_sum, int dtype, int64_t rows,
                   int64_t cols, cudaStream_t s, int out_dtype = -1, const SoftmaxMask* mask = nullptr,
                   void* scratch = nullptr, size_t scratch_bytes = 0);
int launch_norm_rows(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                     int dtype, int affine_dtype, int64_t rows, int64_t cols, int64_t affine_inner,
                     int64_t affine_period, float eps, cudaStream_t s, int32_t* status = nullptr, bool centre = true,
                     const void* res = nullptr, const void* res_bias = nullptr, void* scratch = nullptr, size_t scratch_bytes = 0,
                     int act = 0);  // act: a ReLU on the normalised value (1) or on the affine result (2)
size_t softmax_scratch_bytes(int64_t rows, int64_t cols, int elem_bytes);
size_t norm_scratch_bytes(int64_t rows, int64_t cols, int elem_bytes);
int try_softmax_segmented(const void* x, void* y, float* row_max, float* row_sum, int dtype, int out_dtype, int64_t rows, int64_t cols,
                          void* scratch, size_t scratch_bytes, cudaStream_t s, int32_t* status = nullptr);  // 1: not taken, use the ordinary kernels
int try_norm_segmented(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int dtype, int affine_dtype,
                       int64_t rows, int64_t cols, int64_t inner, int64_t period, float eps, int centre, void* scratch, size_t scratch_bytes,
                       cudaStream_t s, int32_t* status = nullptr);
int32_t* norm_default_status();
// flags: IB200_GEMM_ALLOW_TF32.  With scratch (256-byte aligned, gemm_scratch_bytes says how much) the tiles of a
// last, mostly empty round of the tensor-core kernel are split along K; without it they run whole.
int launch_gemm(const void* a, const void* b, const void* bias, void* c, int in_dtype, int out_dtype,
                int64_t m, int64_t n, int64_t k, int transpose_b, int act, int32_t* status,
                cudaStream_t s, int flags = 0, void* scratch = nullptr, size_t scratch_bytes = 0);
size_t gemm_scratch_bytes(int in_dtype, int out_dtype, int64_t m, int64_t n, int64_t k, int flags, int transpose_b);
bool gemm_uses_tensor_cores(int in_dtype, int out_dtype, int64_t n, int64_t k, int flags);
bool prefers_cta_pairs(int64_t m, int64_t n, int flags);
int launch_transpose2d(const void* x, void* out, int elem_bytes, int64_t rows, int64_t cols,
                       cudaStream_t s);
struct GatherArgs {
  const void* idx[4];  // one index tensor per data axis, each of n elements
  int64_t dim[4], stride[4];
  int64_t n;
  int n_idx, idx_is_64;
};
int launch_gather(const void* data, const GatherArgs& a, void* out, int elem_bytes, double other, cudaStream_t s);
int launch_rope(const float* x, const float* cos, const float* sin, float* y, int64_t seq, int64_t rows_per_pos, int64_t d, cudaStream_t s);
int launch_correlation(const int8_t* src0, const int8_t* src1, int8_t* out, int64_t in_c, int64_t out_c, int64_t h, int64_t w,
                       const void* shift_ptr, int shift_dtype, int shift_value, cudaStream_t s);
int launch_resize2x(const int8_t* src, int8_t* out, int64_t c, int64_t h, int64_t w, int hw_fl, cudaStream_t s);
int launch_warp(const int8_t* src, const int16_t* offset, int8_t* out, int64_t c, int64_t h, int64_t w, cudaStream_t s);
// p and seed come from device scalars when their pointers are given, else from the values
int launch_dropout(const float* x, float* y, int64_t n, const void* p_ptr, int p_dtype, float p_value, const void* seed_ptr, int seed_dtype,
                   long long seed_value, int rounds, cudaStream_t s);

#ifdef __CUDACC__
// ---- element conversion ---------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<uint8_t>(uint8_t v) { return v ? 1.0f : 0.0f; }

template <typename T> __device__ __forceinline__ T from_f32(float v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ uint8_t from_f32<uint8_t>(float v) { return v != 0.0f ? 1 : 0; }
template <> __device__ __forceinline__ int32_t from_f32<int32_t>(float v) { return __float2int_rz(v); }

// 4 consecutive elements as fp32.  `p` must be aligned to 4 elements of T.
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 t = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(&t.x), hi = *reinterpret_cast<__nv_bfloat162*>(&t.y);
  v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
template <> __device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
  uint2 t = *reinterpret_cast<const uint2*>(p);
  __half2 lo = *reinterpret_cast<__half2*>(&t.x), hi = *reinterpret_cast<__half2*>(&t.y);
  v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}
template <> __device__ __forceinline__ void load4<uint8_t>(const uint8_t* p, float (&v)[4]) {
  uchar4 t = *reinterpret_cast<const uchar4*>(p);
  v[0] = t.x ? 1.f : 0.f; v[1] = t.y ? 1.f : 0.f; v[2] = t.z ? 1.f : 0.f; v[3] = t.w ? 1.f : 0.f;
}
template <> __device__ __forceinline__ void load4<int32_t>(const int32_t* p, float (&v)[4]) {
  int4 t = *reinterpret_cast<const int4*>(p);
  v[0] = (float)t.x; v[1] = (float)t.y; v[2] = (float)t.z; v[3] = (float)t.w;
}

template <typename T> __device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&lo); t.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = t;
}
template <> __device__ __forceinline__ void store4<__half>(__half* p, const float (&v)[4]) {
  __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&lo); t.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = t;
}
template <> __device__ __forceinline__ void store4<uint8_t>(uint8_t* p, const float (&v)[4]) {
  *reinterpret_cast<uchar4*>(p) = make_uchar4(v[0] != 0.f, v[1] != 0.f, v[2] != 0.f, v[3] != 0.f);
}
template <> __device__ __forceinline__ void store4<int32_t>(int32_t* p, const float (&v)[4]) {
  *reinterpret_cast<int4*>(p) = make_int4(__float2int_rz(v[0]), __float2int_rz(v[1]), __float2int_rz(v[2]), __float2int_rz(v[3]));
}

// numpy's maximum/minimum/max propagate NaN; fmaxf/fminf drop it.
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float min_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

struct SumOp {
  static __device__ __forceinline__ float identity() { return 0.0f; }
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
struct MaxOp {
  static __device__ __forceinline__ float identity() { return -INFINITY; }
  static __device__ __forceinline__ float apply(float a, float b) { return max_nan(a, b); }
};
struct AnyOp {  // operands are 0.0 / 1.0 flags
  static __device__ __forceinline__ float identity() { return 0.0f; }
  static __device__ __forceinline__ float apply(float a, float b) { return (a != 0.0f || b != 0.0f) ? 1.0f : 0.0f; }
};

template <typename Op> __device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide all-reduce.  `slots` is a shared array of at least blockDim.x/32 floats that no
// other reduction is using between the two barriers of this call; callers alternate between
// two arrays so that back-to-back reductions need no extra barrier.
template <typename Op> __device__ __forceinline__ float block_reduce(float v, float* slots) {
  v = warp_reduce<Op>(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  if (lane == 0) slots[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? slots[lane] : Op::identity();
  return warp_reduce<Op>(r);
}

// unsigned division by a runtime constant, valid for dividends below 2^31.
struct FastDiv {
  uint32_t d, mul, shr;
  __host__ __device__ FastDiv() : d(1), mul(0), shr(0) {}
  __host__ explicit FastDiv(uint32_t div) : d(div), mul(0), shr(0) {
    if (div > 1) {
      uint32_t lg = 0;
      while ((1ull << lg) < div) ++lg;
      const unsigned p = 31 + lg;
      mul = static_cast<uint32_t>(((1ull << p) + div - 1) / div);
      shr = p - 32;
    }
  }
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : (__umulhi(n, mul) >> shr); }
  __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
    q = div(n);
    r = n - q * d;
  }
};
#endif  // __CUDACC__

}  // namespace ib200

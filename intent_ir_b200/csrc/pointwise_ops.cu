// Single-op kernels of the reference's benchmark set that are not expressible as micro-op
// chains: rotary position embedding, Philox dropout, and the int8 image ops (correlation, 2x
// fixed-point resize, Q8.8 horizontal warp).  Each is one pass over the data and reproduces
// the interpreter's arithmetic exactly: float products and sums are rounded separately (no
// fused multiply-add), the dropout keep mask is the same integer Philox-4x32 stream, and the
// image ops keep the interpreter's integer widths, wrap-arounds and arithmetic shifts.
#include "common.cuh"

namespace ib200 {
namespace {

// y[s,b,h,:half] = lo*cos - hi*sin ; y[s,b,h,half:] = lo*sin + hi*cos   (verify/interpreter.py:455-477)
template <int V>  // V consecutive columns per thread (4 when half % 4 == 0, else 1)
__global__ void __launch_bounds__(256) rope_kernel(const float* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                                                   float* __restrict__ y, int64_t rows, int64_t rows_per_pos, int half) {
  const int per_row = half / V;
  const int64_t total = rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / per_row;
    const int j = (int)(i - row * per_row) * V;
    const int64_t pos = row / rows_per_pos;
    const float* xr = x + row * 2 * half;
    float* yr = y + row * 2 * half;
    float lo[V], hi[V], c[V], s[V];
    if (V == 4) {
      const float4 a = __ldcs(reinterpret_cast<const float4*>(xr + j)), b = __ldcs(reinterpret_cast<const float4*>(xr + half + j));  // read once: streaming
      const float4 cc = *reinterpret_cast<const float4*>(cs + pos * half + j), ss = *reinterpret_cast<const float4*>(sn + pos * half + j);
      lo[0] = a.x; lo[V > 1 ? 1 : 0] = a.y; lo[V > 2 ? 2 : 0] = a.z; lo[V > 3 ? 3 : 0] = a.w;
      hi[0] = b.x; hi[V > 1 ? 1 : 0] = b.y; hi[V > 2 ? 2 : 0] = b.z; hi[V > 3 ? 3 : 0] = b.w;
      c[0] = cc.x; c[V > 1 ? 1 : 0] = cc.y; c[V > 2 ? 2 : 0] = cc.z; c[V > 3 ? 3 : 0] = cc.w;
      s[0] = ss.x; s[V > 1 ? 1 : 0] = ss.y; s[V > 2 ? 2 : 0] = ss.z; s[V > 3 ? 3 : 0] = ss.w;
    } else {
      lo[0] = xr[j]; hi[0] = xr[half + j]; c[0] = cs[pos * half + j]; s[0] = sn[pos * half + j];
    }
    float o1[V], o2[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
      o1[k] = __fsub_rn(__fmul_rn(lo[k], c[k]), __fmul_rn(hi[k], s[k]));
      o2[k] = __fadd_rn(__fmul_rn(lo[k], s[k]), __fmul_rn(hi[k], c[k]));
    }
    if (V == 4) {
      __stcs(reinterpret_cast<float4*>(yr + j), make_float4(o1[0], o1[V > 1 ? 1 : 0], o1[V > 2 ? 2 : 0], o1[V > 3 ? 3 : 0]));
      __stcs(reinterpret_cast<float4*>(yr + half + j), make_float4(o2[0], o2[V > 1 ? 1 : 0], o2[V > 2 ? 2 : 0], o2[V > 3 ? 3 : 0]));
    } else {
      yr[j] = o1[0];
      yr[half + j] = o2[0];
    }
  }
}

// counter (index, 0, 0, 0), key (seed low, seed high): the first output word of Philox-4x32
// (verify/interpreter.py:303-329)
// ROUNDS > 0 unrolls completely: the zero counter words then cost nothing in the first round and
// the second round's key-only product is hoisted out of the element loop by the compiler.
template <int ROUNDS>
__device__ __forceinline__ uint32_t philox_c0(uint32_t index, uint32_t k0, uint32_t k1, int rounds) {
  uint32_t c0 = index, c1 = 0, c2 = 0, c3 = 0;
  const int n = ROUNDS > 0 ? ROUNDS : rounds;
#pragma unroll
  for (int r = 0; r < n; ++r) {
    const uint64_t pa = (uint64_t)0xD2511F53u * c0, pb = (uint64_t)0xCD9E8D57u * c2;  // one wide multiply each
    c0 = (uint32_t)(pb >> 32) ^ c1 ^ k0;
    c1 = (uint32_t)pb;
    c2 = (uint32_t)(pa >> 32) ^ c3 ^ k1;
    c3 = (uint32_t)pa;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

struct DropoutArgs {
  const void* p_ptr;     // device scalar, or null when p_value applies
  const void* seed_ptr;  // device scalar, or null when seed_value applies
  int p_dtype, seed_dtype;
  float p_value;
  long long seed_value;
  int rounds;
};

// y = u > p ? x / (1 - p) : 0 with u = uniform(philox(seed, index)); p >= 1 gives zeros, p <= 0
// gives x (verify/interpreter.py:697-742)
template <int ROUNDS>
__global__ void __launch_bounds__(256) dropout_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n, DropoutArgs a) {
  float p = a.p_value;
  if (a.p_ptr) p = a.p_dtype == IB200_F32 ? *static_cast<const float*>(a.p_ptr)
                 : a.p_dtype == IB200_BF16 ? __bfloat162float(*static_cast<const __nv_bfloat16*>(a.p_ptr))
                 : a.p_dtype == IB200_F16 ? __half2float(*static_cast<const __half*>(a.p_ptr))
                                           : (float)*static_cast<const double*>(a.p_ptr);
  long long seed = a.seed_value;
  if (a.seed_ptr) seed = a.seed_dtype == IB200_I64 ? *static_cast<const long long*>(a.seed_ptr) : (long long)*static_cast<const int*>(a.seed_ptr);
  const double keep_d = 1.0 - (double)p;
  const float keep = (float)keep_d;
  const int mode = keep_d <= 0.0 ? 0 : ((double)p <= 0.0 ? 1 : 2);  // zeros / copy / sample
  const uint32_t k0 = (uint32_t)((unsigned long long)seed & 0xFFFFFFFFull), k1 = (uint32_t)(((unsigned long long)seed >> 32) & 0xFFFFFFFFull);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float v = 0.0f;
    if (mode == 1) {
      v = x[i];
    } else if (mode == 2) {
      int r = (int)philox_c0<ROUNDS>((uint32_t)i, k0, k1, a.rounds);
      if (r < 0) r = ~r;
      const float u = __fmul_rn(__int2float_rn(r), 4.6566127342e-10f);
      v = u > p ? __fdiv_rn(x[i], keep) : 0.0f;
    }
    y[i] = v;
  }
}

// out[oc, h, w] = int8((sum_k src0[k, h, w] * src1[k, h, w - oc]) >> shift), 0 where w < oc
// (verify/interpreter.py:330-362)
__global__ void __launch_bounds__(256) correlation_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b, int8_t* __restrict__ out,
                                                         int in_c, int out_c, int h, int w, const void* shift_ptr, int shift_dtype, int shift_value) {
  int shift = shift_value;
  if (shift_ptr) shift = shift_dtype == IB200_I64 ? (int)*static_cast<const long long*>(shift_ptr) : *static_cast<const int*>(shift_ptr);
  shift = shift > 31 ? 31 : shift;  // an arithmetic shift saturates there
  const int64_t plane = (int64_t)h * w, total = plane * out_c;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int oc = (int)(i / plane);
    const int64_t hw = i - (int64_t)oc * plane;
    const int x = (int)(hw % w);
    int acc = 0;
    if (x >= oc)
      for (int k = 0; k < in_c; ++k) acc += (int)a[k * plane + hw] * (int)b[k * plane + hw - oc];
    out[i] = (int8_t)(acc >> shift);
  }
}

// 2x bilinear upsample with hw_fl fractional bits (verify/interpreter.py:363-413)
__global__ void __launch_bounds__(256) resize_kernel(const int8_t* __restrict__ src, int8_t* __restrict__ out, int c, int h, int w, int fl) {
  const int oh = 2 * h, ow = 2 * w, one = 1 << fl;
  const int64_t total = (int64_t)c * oh * ow;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int ox = (int)(i % ow), oy = (int)((i / ow) % oh), ch = (int)(i / ((int64_t)ow * oh));
    const int py = oy << (fl - 1), y0 = py >> fl, fy = py - (y0 << fl), y1 = min(y0 + 1, h - 1);
    const int px = ox << (fl - 1), x0 = px >> fl, fx = px - (x0 << fl), x1 = min(x0 + 1, w - 1);
    const int8_t* s = src + (int64_t)ch * h * w;
    const int top = ((int)s[y0 * w + x0] * (one - fx) + (int)s[y0 * w + x1] * fx) >> fl;
    const int bot = ((int)s[y1 * w + x0] * (one - fx) + (int)s[y1 * w + x1] * fx) >> fl;
    out[i] = (int8_t)((top * (one - fy) + bot * fy) >> fl);
  }
}

// horizontal warp by a Q8.8 offset per pixel; the column counter and the tap positions are
// 8 bits wide and wrap, the blend is 16 bits wide and wraps (verify/interpreter.py:414-454)
__global__ void __launch_bounds__(256) warp_kernel(const int8_t* __restrict__ src, const int16_t* __restrict__ offset, int8_t* __restrict__ out,
                                                  int c, int h, int w) {
  const int64_t plane = (int64_t)h * w, total = plane * c;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t hw = i % plane;
    const int x = (int)(hw % w);
    const int16_t off = offset[hw];
    const int8_t whole = (int8_t)(off >> 8);
    const int16_t frac = (int16_t)(int8_t)(off & 0xFF);
    const int8_t col = (int8_t)(x & 0xFF);
    const int8_t right = (int8_t)((int)col - (int)whole);
    const int8_t left = (int8_t)((int)right - 1);
    const int8_t* row = src + (i - x);
    const int rv = right >= 0 ? (int)row[min((int)right, w - 1)] : 0;
    const int lv = left >= 0 ? (int)row[min((int)left, w - 1)] : 0;
    const int16_t mixed = (int16_t)((rv << 8) + (lv - rv) * (int)frac);
    out[i] = (int8_t)(mixed >> 8);
  }
}

int elementwise_grid(int64_t n) {
  const int64_t blocks = (n + 255) / 256;
  return (int)(blocks < (int64_t)kSmCount * 32 ? blocks : (int64_t)kSmCount * 32);
}

}  // namespace

int launch_correlation(const int8_t* src0, const int8_t* src1, int8_t* out, int64_t in_c, int64_t out_c, int64_t h, int64_t w,
                       const void* shift_ptr, int shift_dtype, int shift_value, cudaStream_t s) {
  if (in_c < 0 || out_c < 0 || h < 0 || w < 0) return fail(IB200_ERR_INVALID, "correlation: negative extent");
  if (out_c * h * w == 0) return IB200_OK;
  if (out_c - 1 > w) return fail(IB200_ERR_INVALID, "correlation: output channels need shifts beyond the width");
  if (in_c > INT32_MAX || out_c > INT32_MAX || h > INT32_MAX || w > INT32_MAX) return fail(IB200_ERR_UNSUPPORTED, "correlation: extent above 2^31-1");
  if (!out || (in_c > 0 && (!src0 || !src1))) return fail(IB200_ERR_INVALID, "correlation: null pointer");
  if (shift_ptr && shift_dtype != IB200_I32 && shift_dtype != IB200_I64) return fail(IB200_ERR_UNSUPPORTED, "correlation: out_shift must be an i32 or i64 scalar");
  if (!shift_ptr && shift_value < 0) return fail(IB200_ERR_INVALID, "correlation: negative out_shift");
  correlation_kernel<<<elementwise_grid(out_c * h * w), 256, 0, s>>>(src0, src1, out, (int)in_c, (int)out_c, (int)h, (int)w, shift_ptr, shift_dtype, shift_value);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "correlation launch");
}

int launch_resize2x(const int8_t* src, int8_t* out, int64_t c, int64_t h, int64_t w, int hw_fl, cudaStream_t s) {
  if (c < 0 || h < 0 || w < 0) return fail(IB200_ERR_INVALID, "resize: negative extent");
  if (hw_fl < 1 || hw_fl > 14) return fail(IB200_ERR_UNSUPPORTED, "resize: hw_fl must be between 1 and 14");
  if (c * h * w == 0) return IB200_OK;
  if (c > INT32_MAX || 2 * h > INT32_MAX >> hw_fl || 2 * w > INT32_MAX >> hw_fl) return fail(IB200_ERR_UNSUPPORTED, "resize: extent too large for the fixed-point coordinates");
  if (!src || !out) return fail(IB200_ERR_INVALID, "resize: null pointer");
  resize_kernel<<<elementwise_grid(4 * c * h * w), 256, 0, s>>>(src, out, (int)c, (int)h, (int)w, hw_fl);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "resize launch");
}

int launch_warp(const int8_t* src, const int16_t* offset, int8_t* out, int64_t c, int64_t h, int64_t w, cudaStream_t s) {
  if (c < 0 || h < 0 || w < 0) return fail(IB200_ERR_INVALID, "warp: negative extent");
  if (c * h * w == 0) return IB200_OK;
  if (c > INT32_MAX || h > INT32_MAX || w > INT32_MAX) return fail(IB200_ERR_UNSUPPORTED, "warp: extent above 2^31-1");
  if (!src || !offset || !out) return fail(IB200_ERR_INVALID, "warp: null pointer");
  warp_kernel<<<elementwise_grid(c * h * w), 256, 0, s>>>(src, offset, out, (int)c, (int)h, (int)w);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "warp launch");
}

int launch_rope(const float* x, const float* cos, const float* sin, float* y, int64_t seq, int64_t rows_per_pos, int64_t d, cudaStream_t s) {
  if (seq < 0 || rows_per_pos < 0 || d < 0 || d % 2) return fail(IB200_ERR_INVALID, "rope: the last axis must be even");
  const int64_t rows = seq * rows_per_pos;
  if (rows == 0 || d == 0) return IB200_OK;
  if (!x || !cos || !sin || !y) return fail(IB200_ERR_INVALID, "rope: null pointer");
  if (d / 2 > INT32_MAX) return fail(IB200_ERR_UNSUPPORTED, "rope: last axis too long");
  const int half = (int)(d / 2);
  const bool vec = half % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(cos) && aligned16(sin);
  const int64_t work = rows * (vec ? half / 4 : half);
  const int64_t blocks = (work + 255) / 256;
  const int grid = (int)(blocks < (int64_t)kSmCount * 16 ? blocks : (int64_t)kSmCount * 16);
  if (vec) rope_kernel<4><<<grid, 256, 0, s>>>(x, cos, sin, y, rows, rows_per_pos, half);
  else rope_kernel<1><<<grid, 256, 0, s>>>(x, cos, sin, y, rows, rows_per_pos, half);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "rope launch");
}

int launch_dropout(const float* x, float* y, int64_t n, const void* p_ptr, int p_dtype, float p_value, const void* seed_ptr, int seed_dtype,
                   long long seed_value, int rounds, cudaStream_t s) {
  if (n < 0) return fail(IB200_ERR_INVALID, "dropout: negative extent");
  if (n == 0) return IB200_OK;
  if (n > (int64_t)UINT32_MAX) return fail(IB200_ERR_UNSUPPORTED, "dropout: more than 2^32-1 elements (the Philox counter is 32 bits)");
  if (!x || !y) return fail(IB200_ERR_INVALID, "dropout: null pointer");
  if (p_ptr && !(p_dtype == IB200_F32 || p_dtype == IB200_BF16 || p_dtype == IB200_F16 || p_dtype == IB200_F64))
    return fail(IB200_ERR_UNSUPPORTED, "dropout: p must be a floating-point scalar");
  if (seed_ptr && !(seed_dtype == IB200_I32 || seed_dtype == IB200_I64)) return fail(IB200_ERR_UNSUPPORTED, "dropout: seed must be an i32 or i64 scalar");
  DropoutArgs a{p_ptr, seed_ptr, p_dtype, seed_dtype, p_value, seed_value, rounds > 0 ? rounds : 10};
  const int64_t blocks = (n + 255) / 256;
  const int grid = (int)(blocks < (int64_t)kSmCount * 32 ? blocks : (int64_t)kSmCount * 32);
  if (a.rounds == 10) dropout_kernel<10><<<grid, 256, 0, s>>>(x, y, n, a);
  else if (a.rounds == 7) dropout_kernel<7><<<grid, 256, 0, s>>>(x, y, n, a);
  else dropout_kernel<0><<<grid, 256, 0, s>>>(x, y, n, a);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "dropout launch");
}

}  // namespace ib200

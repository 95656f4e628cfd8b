// Device helpers shared by the kernels that interpret micro-op programs (elementwise.cu,
// rowfuse.cu): cp.async staging, typed scalar / 4-wide loads and stores, and the per-opcode
// arithmetic over a thread's register values.
#pragma once
#include "common.cuh"
#include "ew_program.h"

namespace ib200 {
namespace {

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_committed() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }  // all but the newest group

__device__ __forceinline__ float load_scalar(const void* p, int dtype, int64_t off) {
  switch (dtype) {
    case IB200_F32: return static_cast<const float*>(p)[off];
    case IB200_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[off]);
    case IB200_F16: return __half2float(static_cast<const __half*>(p)[off]);
    case IB200_BOOL: case IB200_U8: return static_cast<const uint8_t*>(p)[off] ? 1.0f : 0.0f;
    case IB200_I32: return (float)static_cast<const int32_t*>(p)[off];
    case IB200_I64: return (float)static_cast<const long long*>(p)[off];
    case IB200_I8: return (float)static_cast<const int8_t*>(p)[off];
    case IB200_I16: return (float)static_cast<const int16_t*>(p)[off];
    default: return 0.0f;
  }
}

__device__ __forceinline__ void store_scalar(void* p, int dtype, int64_t off, float v) {
  switch (dtype) {
    case IB200_F32: static_cast<float*>(p)[off] = v; break;
    case IB200_BF16: static_cast<__nv_bfloat16*>(p)[off] = __float2bfloat16_rn(v); break;
    case IB200_F16: static_cast<__half*>(p)[off] = __float2half_rn(v); break;
    case IB200_BOOL: case IB200_U8: static_cast<uint8_t*>(p)[off] = v != 0.0f ? 1 : 0; break;
    case IB200_I32: static_cast<int32_t*>(p)[off] = __float2int_rz(v); break;
    case IB200_I64: static_cast<long long*>(p)[off] = __float2ll_rz(v); break;
    case IB200_I8: static_cast<int8_t*>(p)[off] = (int8_t)__float2int_rz(v); break;
    case IB200_I16: static_cast<int16_t*>(p)[off] = (int16_t)__float2int_rz(v); break;
    default: break;
  }
}

__device__ __forceinline__ void store_vec4(void* p, int dtype, int64_t off, const float (&v)[4]) {
  switch (dtype) {
    case IB200_F32: __stcs(reinterpret_cast<float4*>(static_cast<float*>(p) + off), make_float4(v[0], v[1], v[2], v[3])); break;  // written once: evict first
    case IB200_BF16: store4<__nv_bfloat16>(static_cast<__nv_bfloat16*>(p) + off, v); break;
    case IB200_F16: store4<__half>(static_cast<__half*>(p) + off, v); break;
    case IB200_BOOL: case IB200_U8: store4<uint8_t>(static_cast<uint8_t*>(p) + off, v); break;
    case IB200_I32: store4<int32_t>(static_cast<int32_t*>(p) + off, v); break;
    default:
#pragma unroll
      for (int k = 0; k < 4; ++k) store_scalar(p, dtype, off + k, v[k]);
  }
}

// one micro-op over the thread's 8 values; the opcode is uniform across the grid, so the
// switch is a single uniform branch per instruction, not per element
template <int N>
__device__ __forceinline__ void apply(uint8_t op, const float (&a)[N], const float (&b)[N], float (&acc)[N]) {
#define EW_CASE(OP, EXPR)                      \
  case OP:                                     \
    _Pragma("unroll") for (int j = 0; j < N; ++j) { \
      const float x = a[j], y = b[j];          \
      (void)y;                                 \
      acc[j] = (EXPR);                         \
    }                                          \
    break;
  // the opcodes of almost every chain first: one compare each instead of a walk down the switch's
  // comparison tree
  if (op == EW_ADD) {
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = a[j] + b[j];
    return;
  }
  if (op == EW_MUL) {
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = a[j] * b[j];
    return;
  }
  switch (op) {
    EW_CASE(EW_MOV, x)
    EW_CASE(EW_ADD, x + y)
    EW_CASE(EW_SUB, x - y)
    EW_CASE(EW_MUL, x * y)
    EW_CASE(EW_DIV, x / y)
    EW_CASE(EW_MAX, max_nan(x, y))
    EW_CASE(EW_MIN, min_nan(x, y))
    EW_CASE(EW_RELU, max_nan(x, 0.0f))
    EW_CASE(EW_EXP, expf(x))
    EW_CASE(EW_RSQRT, 1.0f / sqrtf(x))
    EW_CASE(EW_ABS, fabsf(x))
    EW_CASE(EW_FLOOR, floorf(x))
    EW_CASE(EW_NE, x != y ? 1.0f : 0.0f)
    EW_CASE(EW_LT, x < y ? 1.0f : 0.0f)
    EW_CASE(EW_LE, x <= y ? 1.0f : 0.0f)
    EW_CASE(EW_GT, x > y ? 1.0f : 0.0f)
    EW_CASE(EW_GE, x >= y ? 1.0f : 0.0f)
    EW_CASE(EW_AND, (x != 0.0f && y != 0.0f) ? 1.0f : 0.0f)
    EW_CASE(EW_OR, (x != 0.0f || y != 0.0f) ? 1.0f : 0.0f)
    EW_CASE(EW_NOT, x != 0.0f ? 0.0f : 1.0f)
    EW_CASE(EW_TO_BOOL, x != 0.0f ? 1.0f : 0.0f)
    EW_CASE(EW_TO_INT, truncf(x))
    EW_CASE(EW_ROUND_BF16, __bfloat162float(__float2bfloat16_rn(x)))
    EW_CASE(EW_ROUND_F16, __half2float(__float2half_rn(x)))
    EW_CASE(EW_RSUB, y - x)
    EW_CASE(EW_RDIV, y / x)
    EW_CASE(EW_LOADB, y)
    default: break;
  }
#undef EW_CASE
}

// acc = op(acc, y) for one value y shared by all N lanes of the thread (an immediate or a
// per-row scalar): the binary opcodes only, no broadcast of y into registers
template <int N> __device__ __forceinline__ void apply_scalar(uint8_t op, float (&acc)[N], float y) {
#define EW_CASE(OP, EXPR)                      \
  case OP:                                     \
    _Pragma("unroll") for (int j = 0; j < N; ++j) { \
      const float x = acc[j];                  \
      (void)x;                                 \
      acc[j] = (EXPR);                         \
    }                                          \
    break;
  switch (op) {
    EW_CASE(EW_ADD, x + y)
    EW_CASE(EW_SUB, x - y)
    EW_CASE(EW_MUL, x * y)
    EW_CASE(EW_DIV, x / y)
    EW_CASE(EW_MAX, max_nan(x, y))
    EW_CASE(EW_MIN, min_nan(x, y))
    EW_CASE(EW_NE, x != y ? 1.0f : 0.0f)
    EW_CASE(EW_LT, x < y ? 1.0f : 0.0f)
    EW_CASE(EW_LE, x <= y ? 1.0f : 0.0f)
    EW_CASE(EW_GT, x > y ? 1.0f : 0.0f)
    EW_CASE(EW_GE, x >= y ? 1.0f : 0.0f)
    EW_CASE(EW_AND, (x != 0.0f && y != 0.0f) ? 1.0f : 0.0f)
    EW_CASE(EW_OR, (x != 0.0f || y != 0.0f) ? 1.0f : 0.0f)
    EW_CASE(EW_RSUB, y - x)
    EW_CASE(EW_RDIV, y / x)
    EW_CASE(EW_LOADB, y)
    default: break;
  }
#undef EW_CASE
}

// One micro-op with its opcode as a template argument, for programs that are compiled in (elementwise.cu,
// rowfuse.cu): the same expressions per opcode as apply() above.
// (the explicitly rounded intrinsics keep the compiler from contracting a multiply and the add of the NEXT micro-op into
// one FMA, which it would do here, where the chain is straight-line code, and cannot do across the interpreter's
// branches: every micro-op rounds on its own, as numpy's does)
template <uint8_t OP> __device__ __forceinline__ float static_op(float x, float y) {
  if constexpr (OP == EW_MOV) return x;
  else if constexpr (OP == EW_ADD) return __fadd_rn(x, y);
  else if constexpr (OP == EW_SUB) return __fsub_rn(x, y);
  else if constexpr (OP == EW_MUL) return __fmul_rn(x, y);
  else if constexpr (OP == EW_DIV) return x / y;
  else if constexpr (OP == EW_MAX) return max_nan(x, y);
  else if constexpr (OP == EW_MIN) return min_nan(x, y);
  else if constexpr (OP == EW_RELU) return max_nan(x, 0.0f);
  else if constexpr (OP == EW_EXP) return expf(x);
  else if constexpr (OP == EW_RSQRT) return 1.0f / sqrtf(x);
  else if constexpr (OP == EW_ABS) return fabsf(x);
  else if constexpr (OP == EW_FLOOR) return floorf(x);
  else if constexpr (OP == EW_NE) return x != y ? 1.0f : 0.0f;
  else if constexpr (OP == EW_LT) return x < y ? 1.0f : 0.0f;
  else if constexpr (OP == EW_LE) return x <= y ? 1.0f : 0.0f;
  else if constexpr (OP == EW_GT) return x > y ? 1.0f : 0.0f;
  else if constexpr (OP == EW_GE) return x >= y ? 1.0f : 0.0f;
  else if constexpr (OP == EW_AND) return (x != 0.0f && y != 0.0f) ? 1.0f : 0.0f;
  else if constexpr (OP == EW_OR) return (x != 0.0f || y != 0.0f) ? 1.0f : 0.0f;
  else if constexpr (OP == EW_NOT) return x != 0.0f ? 0.0f : 1.0f;
  else if constexpr (OP == EW_TO_BOOL) return x != 0.0f ? 1.0f : 0.0f;
  else if constexpr (OP == EW_TO_INT) return truncf(x);
  else if constexpr (OP == EW_ROUND_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  else if constexpr (OP == EW_ROUND_F16) return __half2float(__float2half_rn(x));
  else if constexpr (OP == EW_RSUB) return __fsub_rn(y, x);
  else if constexpr (OP == EW_RDIV) return y / x;
  else return y;  // EW_LOADB
}

}  // namespace
}  // namespace ib200

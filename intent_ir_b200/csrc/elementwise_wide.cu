// Fused elementwise / broadcast chains whose values do not fit f32 lanes: f64 tensors, and i32 / i64
// tensors (an f32 holds integers exactly only up to 2^24).  The same micro-op programs as
// elementwise.cu (ew_program.h), executed with every value carried as a double — exact for f64 and for
// integers up to 2^53 — one output element per thread and iteration, the slot file in per-thread local
// memory.  The interpreter the reference checks against computes these graphs in numpy's f64 / int64
// (verify/interpreter.py:212-252, :633-643); its CUDA backend has no f64 path at all
// (frontends/cuda/runtime.py:74-93).  This kernel is about exactness, not bandwidth: integer index
// arithmetic and f64 graphs are small.
#include <cuda_runtime.h>

#include "common.cuh"
#include "ew_program.h"

namespace ib200 {
namespace {

struct WideImm {
  double v[kEwMaxInstr];
};
struct WideDivs {
  FastDiv d[kEwMaxRank];
};

__device__ __forceinline__ double load_wide(const void* p, int dtype, int64_t off) {
  switch (dtype) {
    case IB200_F32: return (double)static_cast<const float*>(p)[off];
    case IB200_F64: return static_cast<const double*>(p)[off];
    case IB200_BF16: return (double)__bfloat162float(static_cast<const __nv_bfloat16*>(p)[off]);
    case IB200_F16: return (double)__half2float(static_cast<const __half*>(p)[off]);
    case IB200_BOOL: case IB200_U8: return static_cast<const uint8_t*>(p)[off] ? 1.0 : 0.0;
    case IB200_I32: return (double)static_cast<const int32_t*>(p)[off];
    case IB200_I64: return (double)static_cast<const long long*>(p)[off];
    case IB200_I8: return (double)static_cast<const int8_t*>(p)[off];
    case IB200_I16: return (double)static_cast<const int16_t*>(p)[off];
    default: return 0.0;
  }
}

__device__ __forceinline__ void store_wide(void* p, int dtype, int64_t off, double v) {
  switch (dtype) {
    case IB200_F32: static_cast<float*>(p)[off] = (float)v; break;
    case IB200_F64: static_cast<double*>(p)[off] = v; break;
    case IB200_BF16: static_cast<__nv_bfloat16*>(p)[off] = __float2bfloat16_rn((float)v); break;
    case IB200_F16: static_cast<__half*>(p)[off] = __float2half_rn((float)v); break;
    case IB200_BOOL: case IB200_U8: static_cast<uint8_t*>(p)[off] = v != 0.0 ? 1 : 0; break;
    case IB200_I32: static_cast<int32_t*>(p)[off] = (int32_t)__double2ll_rz(v); break;
    case IB200_I64: static_cast<long long*>(p)[off] = __double2ll_rz(v); break;
    case IB200_I8: static_cast<int8_t*>(p)[off] = (int8_t)__double2ll_rz(v); break;
    case IB200_I16: static_cast<int16_t*>(p)[off] = (int16_t)__double2ll_rz(v); break;
    default: break;
  }
}

// numpy's maximum / minimum propagate NaN
__device__ __forceinline__ double max_nan_d(double a, double b) { return (a != a || b != b) ? (a != a ? a : b) : (a > b ? a : b); }
__device__ __forceinline__ double min_nan_d(double a, double b) { return (a != a || b != b) ? (a != a ? a : b) : (a < b ? a : b); }

__device__ __forceinline__ double apply_wide(uint8_t op, double x, double y, double z) {
  switch (op) {
    case EW_MOV: return x;
    case EW_ADD: return x + y;
    case EW_SUB: return x - y;
    case EW_MUL: return x * y;
    case EW_DIV: return x / y;
    case EW_MAX: return max_nan_d(x, y);
    case EW_MIN: return min_nan_d(x, y);
    case EW_RELU: return max_nan_d(x, 0.0);
    case EW_EXP: return exp(x);
    case EW_RSQRT: return 1.0 / sqrt(x);
    case EW_ABS: return fabs(x);
    case EW_FLOOR: return floor(x);
    case EW_NE: return x != y ? 1.0 : 0.0;
    case EW_LT: return x < y ? 1.0 : 0.0;
    case EW_LE: return x <= y ? 1.0 : 0.0;
    case EW_GT: return x > y ? 1.0 : 0.0;
    case EW_GE: return x >= y ? 1.0 : 0.0;
    case EW_AND: return (x != 0.0 && y != 0.0) ? 1.0 : 0.0;
    case EW_OR: return (x != 0.0 || y != 0.0) ? 1.0 : 0.0;
    case EW_NOT: return x != 0.0 ? 0.0 : 1.0;
    case EW_WHERE: return x != 0.0 ? y : z;
    case EW_TO_BOOL: return x != 0.0 ? 1.0 : 0.0;
    case EW_TO_INT: return trunc(x);
    case EW_ROUND_BF16: return (double)__bfloat162float(__float2bfloat16_rn((float)x));
    case EW_ROUND_F16: return (double)__half2float(__float2half_rn((float)x));
    case EW_RSUB: return y - x;
    case EW_RDIV: return y / x;
    case EW_LOADB: return y;
    default: return 0.0;
  }
}

__global__ void __launch_bounds__(256) ew_kernel_wide(const __grid_constant__ EwProgram prog, const __grid_constant__ WideImm imm,
                                                      const __grid_constant__ WideDivs divs) {
  double slot[kEwMaxSlots];
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < prog.total; e += stride) {
    uint32_t coord[kEwMaxRank];
    uint32_t rem = (uint32_t)e;
    for (int d = prog.rank - 1; d > 0; --d) {
      uint32_t q;
      divs.d[d].divmod(rem, q, coord[d]);
      rem = q;
    }
    coord[0] = rem;
    for (int k = 0; k < prog.n_inputs; ++k) {
      const EwInput& in = prog.in[k];
      int64_t off = 0;
      for (int d = 0; d < prog.rank; ++d) off += (int64_t)coord[d] * in.stride[d];
      slot[k] = in.kind == EW_IN_IOTA ? (double)off : load_wide(in.ptr, in.dtype, off);
    }
    double acc = 0.0;
    for (int ip = 0; ip < prog.n_instr; ++ip) {
      const EwInstr ins = prog.instr[ip];
      const double im = imm.v[ip];
      const double a = ins.a == EW_ACC ? acc : ins.a == EW_IMM ? im : slot[ins.a];
      const double b = ins.b == EW_ACC ? acc : ins.b == EW_IMM ? im : slot[ins.b];
      const double c = ins.c == EW_ACC ? acc : ins.c == EW_IMM ? im : slot[ins.c];
      acc = apply_wide(ins.op, a, b, c);
      if (ins.dst != EW_NODST) slot[ins.dst] = acc;
    }
    for (int o = 0; o < prog.n_outputs; ++o) {
      const EwOutput& out = prog.out[o];
      store_wide(out.ptr, out.dtype, e, out.src == EW_ACC ? acc : slot[out.src]);
    }
  }
}

}  // namespace

int launch_elementwise_wide(const EwProgram& prog, const double* imm, cudaStream_t s) {
  if (prog.total == 0) return IB200_OK;
  if (prog.total < 0 || prog.total >= ((int64_t)1 << 31)) return fail(IB200_ERR_UNSUPPORTED, "elementwise: more than 2^31-1 output elements");
  if (prog.rank < 1 || prog.rank > kEwMaxRank || prog.n_inputs > kEwMaxInputs || prog.n_outputs < 1 || prog.n_outputs > kEwMaxOutputs ||
      prog.n_instr > kEwMaxInstr || prog.n_slots > kEwMaxSlots || prog.n_slots < prog.n_inputs || !imm)
    return fail(IB200_ERR_INVALID, "elementwise: malformed program");
  WideImm wi;
  for (int i = 0; i < kEwMaxInstr; ++i) wi.v[i] = imm[i];
  WideDivs divs;
  for (int d = 0; d < prog.rank; ++d) divs.d[d] = FastDiv(prog.dim[d]);
  const int64_t blocks = (prog.total + 255) / 256;
  const int grid = (int)(blocks < (int64_t)kSmCount * 16 ? blocks : (int64_t)kSmCount * 16);
  ew_kernel_wide<<<grid, 256, 0, s>>>(prog, wi, divs);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "elementwise (f64 lanes) launch");
}

}  // namespace ib200

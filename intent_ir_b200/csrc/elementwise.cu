// Fused elementwise / broadcast chains: one pass over the output, executing the micro-op
// program of ew_program.h.  Replaces the per-graph generated source of the reference
// (backends/cuda/codegen/intentir_to_cuda.py:229-534, one thread per element with int64
// div/mod and scalar loads) with one pre-compiled kernel:
//
//   * each thread owns 8 output elements: two 128-bit vectors when the innermost extent is
//     a multiple of 4 and the operands are aligned (VEC), else 8 strided scalars;
//   * output coordinates come from 32-bit multiply-shift division by the collapsed extents,
//     once per vector, and give each operand's offset through its (possibly zero) strides —
//     numpy broadcasting and broadcast_in_dim are just zero strides, iota is a ramp;
//   * contiguous f32 / bf16 / f16 operands are staged global -> shared with cp.async (all
//     operands in flight at once, no register round trip); the slot file lives in shared
//     memory, one conflict-free column per thread, so no barrier is ever needed;
//   * the chain itself runs on an accumulator held in registers.
//
// HBM-bound: bytes moved = each distinct operand once + each output once.
#include <cuda_runtime.h>

#include <cstdlib>
#include <map>
#include <string>

#include "common.cuh"
#include "ew_device.cuh"
#include "ew_program.h"

namespace ib200 {
namespace {

constexpr int kThreads = 256;
constexpr int kPerThread = 8;
constexpr int kTile = kThreads * kPerThread;

struct EwDivs {
  FastDiv d[kEwMaxRank];
};

// Slot file: slot s, value j (0..N-1), thread t.  VEC: values 4u..4u+3 form one float4 at
// ((s*N/4+u)*kThreads + t)*16 bytes; scalar: value j at ((s*N+j)*kThreads + t)*4 bytes.
template <bool VEC, int N> __device__ __forceinline__ float* slot_ptr(float* file, int s, int j, int t) {
  return VEC ? file + ((size_t)(s * (N / 4) + (j >> 2)) * kThreads + t) * 4 + (j & 3) : file + ((size_t)(s * N + j) * kThreads + t);
}

template <bool VEC, int N>
__device__ __forceinline__ void fetch(float (&dst)[N], uint8_t code, const float (&acc)[N], float imm, float* file, int t) {
  if (code == EW_ACC) {
#pragma unroll
    for (int j = 0; j < N; ++j) dst[j] = acc[j];
  } else if (code == EW_IMM) {
#pragma unroll
    for (int j = 0; j < N; ++j) dst[j] = imm;
  } else if (VEC) {
#pragma unroll
    for (int u = 0; u < N / 4; ++u) {
      const float4 q = *reinterpret_cast<const float4*>(slot_ptr<true, N>(file, code, 4 * u, t));
      dst[4 * u] = q.x; dst[4 * u + 1] = q.y; dst[4 * u + 2] = q.z; dst[4 * u + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) dst[j] = *slot_ptr<false, N>(file, code, j, t);
  }
}

template <bool VEC, int N> __device__ __forceinline__ void put(const float (&src)[N], int s, float* file, int t) {
  if (VEC) {
#pragma unroll
    for (int u = 0; u < N / 4; ++u)
      *reinterpret_cast<float4*>(slot_ptr<true, N>(file, s, 4 * u, t)) = make_float4(src[4 * u], src[4 * u + 1], src[4 * u + 2], src[4 * u + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) *slot_ptr<false, N>(file, s, j, t) = src[j];
  }
}

// The instruction loop.  Operands that are the previous result are used in place (no copy of
// the accumulator); the opcode and operand codes are uniform, so every branch here is uniform.
template <bool VEC, int N>
__device__ __forceinline__ void run_chain(const EwProgram& prog, float (&acc)[N], float* file, int t) {
#pragma unroll
  for (int j = 0; j < N; ++j) acc[j] = 0.0f;
  for (int ip = 0; ip < prog.n_instr; ++ip) {
    const EwInstr ins = prog.instr[ip];
    if (ins.op == EW_WHERE) {
      float a[N], b[N], c[N];
      fetch<VEC, N>(a, ins.a, acc, ins.imm, file, t);
      fetch<VEC, N>(b, ins.b, acc, ins.imm, file, t);
      fetch<VEC, N>(c, ins.c, acc, ins.imm, file, t);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = a[j] != 0.0f ? b[j] : c[j];
    } else if (ins.a == EW_ACC && ins.b == EW_ACC) {
      apply<N>(ins.op, acc, acc, acc);
    } else if (ins.a == EW_ACC) {
      float b[N];
      fetch<VEC, N>(b, ins.b, acc, ins.imm, file, t);
      apply<N>(ins.op, acc, b, acc);
    } else if (ins.b == EW_ACC) {
      float a[N];
      fetch<VEC, N>(a, ins.a, acc, ins.imm, file, t);
      apply<N>(ins.op, a, acc, acc);
    } else {
      float a[N], b[N];
      fetch<VEC, N>(a, ins.a, acc, ins.imm, file, t);
      fetch<VEC, N>(b, ins.b, acc, ins.imm, file, t);
      apply<N>(ins.op, a, b, acc);
    }
    if (ins.dst != EW_NODST) put<VEC, N>(acc, ins.dst, file, t);
  }
}

template <bool VEC, int N>
__device__ __forceinline__ void write_outputs(const EwProgram& prog, const float (&acc)[N], float* file, int t, int64_t base) {
  constexpr int W = VEC ? 4 : 1, U = N / W;
  for (int o = 0; o < prog.n_outputs; ++o) {
    const EwOutput& out = prog.out[o];
    float v[N];
    fetch<VEC, N>(v, out.src, acc, 0.0f, file, t);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = base + (int64_t)(u * kThreads + t) * W;
      if (e >= prog.total) continue;
      if (VEC) {
        const float q[4] = {v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]};
        store_vec4(out.ptr, out.dtype, e, q);
      } else {
        store_scalar(out.ptr, out.dtype, e, v[u]);
      }
    }
  }
}

// Specialised staging for the common shapes: at most MAXIN operands, collapsed rank RANK,
// every operand offset below 2^31.  Operand descriptors (pointer, 32-bit strides, staging
// mode) are read once per CTA into registers; the per-tile work is RANK-1 multiply-shift
// divisions per vector and one 32-bit multiply-add per operand and dimension.
template <int MAXIN, int RANK, bool VEC, int N>
__global__ void __launch_bounds__(kThreads, N == 8 ? 4 : 2) ew_kernel_fast(const __grid_constant__ EwProgram prog, const __grid_constant__ EwDivs divs) {
  extern __shared__ __align__(16) float file[];
  const int t = threadIdx.x;
  constexpr int W = VEC ? 4 : 1, U = N / W;
  constexpr int kTileN = kThreads * N;
  const char* ptr[MAXIN];
  uint32_t stride[MAXIN][RANK];
  int mode[MAXIN], dtype[MAXIN];
  bool convert = false;
#pragma unroll
  for (int k = 0; k < MAXIN; ++k) {
    const bool live = k < prog.n_inputs;
    ptr[k] = live ? static_cast<const char*>(prog.in[k].ptr) : nullptr;
    mode[k] = live ? prog.in[k].mode : EW_STAGE_NONE;
    dtype[k] = live ? prog.in[k].dtype : IB200_F32;
#pragma unroll
    for (int d = 0; d < RANK; ++d) stride[k][d] = live ? (uint32_t)prog.in[k].stride[d] : 0u;
    convert |= mode[k] == EW_STAGE_ASYNC_HALF4;
  }
  const int64_t ntiles = (prog.total + kTileN - 1) / kTileN;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t base = tile * kTileN;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = base + (int64_t)(u * kThreads + t) * W;
      if (e >= prog.total) continue;
      uint32_t coord[RANK];
      uint32_t rem = (uint32_t)e;
#pragma unroll
      for (int d = RANK - 1; d > 0; --d) {
        uint32_t q;
        divs.d[d].divmod(rem, q, coord[d]);
        rem = q;
      }
      coord[0] = rem;
#pragma unroll
      for (int k = 0; k < MAXIN; ++k) {
        if (mode[k] == EW_STAGE_NONE) continue;
        uint32_t off = 0;
#pragma unroll
        for (int d = 0; d < RANK; ++d) off += coord[d] * stride[k][d];
        float* dst = slot_ptr<VEC, N>(file, k, u * W, t);
        switch (mode[k]) {
          case EW_STAGE_ASYNC_F32X4: cp_async16(dst, reinterpret_cast<const float*>(ptr[k]) + off); break;
          case EW_STAGE_ASYNC_HALF4: cp_async8(dst, reinterpret_cast<const uint16_t*>(ptr[k]) + off); break;
          case EW_STAGE_ASYNC_F32: cp_async4(dst, reinterpret_cast<const float*>(ptr[k]) + off); break;
          case EW_STAGE_BROADCAST: {
            const float v = load_scalar(ptr[k], dtype[k], off);
#pragma unroll
            for (int j = 0; j < W; ++j) dst[j] = v;
            break;
          }
          case EW_STAGE_IOTA:
#pragma unroll
            for (int j = 0; j < W; ++j) dst[j] = (float)(off + j * stride[k][RANK - 1]);
            break;
          case EW_STAGE_BYTE4:
            if (VEC) {
              float v[4];
              load4<uint8_t>(reinterpret_cast<const uint8_t*>(ptr[k]) + off, v);
              *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            }
            break;
          default:  // EW_STAGE_GATHER
#pragma unroll
            for (int j = 0; j < W; ++j) dst[j] = load_scalar(ptr[k], dtype[k], (int64_t)off + (int64_t)j * stride[k][RANK - 1]);
        }
      }
    }
    cp_async_wait_all();
    if (VEC && convert) {
#pragma unroll
      for (int k = 0; k < MAXIN; ++k) {
        if (mode[k] != EW_STAGE_ASYNC_HALF4) continue;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float* dst = slot_ptr<VEC, N>(file, k, u * W, t);
          float v[4];
          if (dtype[k] == IB200_BF16) load4<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(dst), v);
          else load4<__half>(reinterpret_cast<const __half*>(dst), v);
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        }
      }
    }
    float acc[N];
    run_chain<VEC, N>(prog, acc, file, t);
    write_outputs<VEC, N>(prog, acc, file, t, base);
  }
}

// ---- register path -------------------------------------------------------------------------
// Linear chains over at most three f32 / bf16 / f16 / bool operands (the common case: y = f(x, col, row, consts))
// never touch shared memory: every operand vector is loaded straight into registers with one
// 128-bit (64-bit for 16-bit types) load (or one scalar load when the operand is constant along the innermost axis),
// all loads are issued before the first use, and each micro-op is acc = op(acc, B) with B an
// operand register set, an immediate or acc itself.  Operand count, which operands are
// inner-broadcast, and the collapsed rank are template parameters, so staging is branch-free.
struct EwRegInstr {
  uint8_t op, src;     // src: 0..2 operand, 3 immediate, 4 acc, 5..6 temporary; EW_WHERE: the condition
  uint8_t b, c;        // EW_WHERE: the two values (same codes)
  uint8_t dst, pad[3]; // 0, or 1..2: also keep the result in that temporary (extended form only)
  float imm;
};
struct EwRegCode {
  int32_t n_instr;
  EwRegInstr ins[kEwMaxInstr + 1];
};

// The run-time form of the instruction loop: one uniform branch per field of the register code.
struct InterpExec {
  template <int NIN, int N, bool EXT>
  __device__ __forceinline__ void run(const float (&in)[NIN > 0 ? NIN : 1][N], float (&acc)[N], const EwRegCode& code) const {
    float tmp[EXT ? 2 : 1][N];  // values used more than once (extended form)
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = tmp[0][j] = tmp[EXT ? 1 : 0][j] = 0.0f;
    for (int ip = 0; ip < code.n_instr; ++ip) {
        const EwRegInstr ins = code.ins[ip];
        if (EXT && ins.op == EW_WHERE) {  // acc = cond != 0 ? b : c, each an operand, the immediate, acc or a temporary
          float sel[3][N];
#pragma unroll
          for (int q = 0; q < 3; ++q) {
            const uint8_t src = q == 0 ? ins.src : q == 1 ? ins.b : ins.c;
#pragma unroll
            for (int j = 0; j < N; ++j)
              sel[q][j] = src == 0 ? in[0][j] : src == 1 ? in[NIN > 1 ? 1 : 0][j] : src == 2 ? in[NIN > 2 ? 2 : 0][j] : src == 3 ? ins.imm
                          : src == 4 ? acc[j] : src == 5 ? tmp[0][j] : tmp[1][j];
          }
#pragma unroll
          for (int j = 0; j < N; ++j) acc[j] = sel[0][j] != 0.0f ? sel[1][j] : sel[2][j];
        } else
        switch (ins.src) {
          case 0: apply<N>(ins.op, acc, in[0], acc); break;
          case 1: if (NIN > 1) apply<N>(ins.op, acc, in[NIN > 1 ? 1 : 0], acc); break;
          case 2: if (NIN > 2) apply<N>(ins.op, acc, in[NIN > 2 ? 2 : 0], acc); break;
          case 3: apply_scalar<N>(ins.op, acc, ins.imm); break;
          case 5: if (EXT) apply<N>(ins.op, acc, tmp[0], acc); break;
          case 6: if (EXT) apply<N>(ins.op, acc, tmp[1], acc); break;
          default: apply<N>(ins.op, acc, acc, acc);
        }
        if (EXT && ins.dst) {
#pragma unroll
          for (int j = 0; j < N; ++j) tmp[ins.dst == 1 ? 0 : 1][j] = acc[j];
        }
      }
  }
};

// EXT adds `where` and bool / u8 operands; it is a separate instantiation because that code costs
// the plain arithmetic chains registers.  Occupancy is what this kernel lives on: the plain form
// is held to 32 registers so that eight CTAs (all 64 warps) are resident per SM -- measured on the
// 4-op broadcast chain: 0.68 of HBM peak at four CTAs per SM, 0.79 at six, 0.83 at eight.
template <int NIN, int BMASK, int RANK, bool EXT, typename Exec>
__device__ __forceinline__ void ew_reg_body(const EwProgram& prog, const EwDivs& divs, const EwRegCode& code, const Exec& exec) {
  constexpr int N = 8, U = 2;  // 16 values per thread were measured slower (half the resident warps)
  const int t = threadIdx.x;
  const char* ptr[NIN > 0 ? NIN : 1];
  uint32_t stride[NIN > 0 ? NIN : 1][RANK];
  int half_kind[NIN > 0 ? NIN : 1];  // 0: f32, 1: bf16, 2: f16, 3: bool / u8 (uniform over the grid)
#pragma unroll
  for (int k = 0; k < NIN; ++k) {
    ptr[k] = static_cast<const char*>(prog.in[k].ptr);
    half_kind[k] = prog.in[k].dtype == IB200_BF16 ? 1 : prog.in[k].dtype == IB200_F16 ? 2 : (EXT && (prog.in[k].dtype == IB200_BOOL || prog.in[k].dtype == IB200_U8)) ? 3 : 0;
#pragma unroll
    for (int d = 0; d < RANK; ++d) stride[k][d] = (uint32_t)prog.in[k].stride[d];
  }
  const int64_t ntiles = (prog.total + kTile - 1) / kTile;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t base = tile * kTile;
    float in[NIN > 0 ? NIN : 1][N];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = base + (int64_t)(u * kThreads + t) * 4;
      const bool live = e < prog.total;
      uint32_t coord[RANK];
      uint32_t rem = live ? (uint32_t)e : 0u;
#pragma unroll
      for (int d = RANK - 1; d > 0; --d) {
        uint32_t q;
        divs.d[d].divmod(rem, q, coord[d]);
        rem = q;
      }
      coord[0] = rem;
#pragma unroll
      for (int k = 0; k < NIN; ++k) {
        uint32_t off = 0;
#pragma unroll
        for (int d = 0; d < RANK; ++d) off += coord[d] * stride[k][d];
        float* dst = &in[k][4 * u];
        if ((BMASK >> k) & 1) {
          float v = 0.0f;
          if (live) {
            if (half_kind[k] == 0) v = __ldg(reinterpret_cast<const float*>(ptr[k]) + off);
            else if (half_kind[k] == 1) v = __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(ptr[k]) + off));
            else if (!EXT || half_kind[k] == 2) v = __half2float(__ldg(reinterpret_cast<const __half*>(ptr[k]) + off));
            else v = __ldg(reinterpret_cast<const uint8_t*>(ptr[k]) + off) ? 1.0f : 0.0f;
          }
          dst[0] = dst[1] = dst[2] = dst[3] = v;
        } else if (half_kind[k] == 0) {
          // (a full-size operand is read once: cache-streaming load; with the streaming store of the result the 4-op chain over [8192,4096] gains 1 %)
          const float4 q = live ? __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ptr[k]) + off)) : make_float4(0.f, 0.f, 0.f, 0.f);
          dst[0] = q.x; dst[1] = q.y; dst[2] = q.z; dst[3] = q.w;
        } else if (EXT && half_kind[k] == 3) {  // four bytes in one 32-bit load
          const uchar4 q = live ? __ldg(reinterpret_cast<const uchar4*>(reinterpret_cast<const uint8_t*>(ptr[k]) + off)) : make_uchar4(0, 0, 0, 0);
          dst[0] = q.x ? 1.0f : 0.0f; dst[1] = q.y ? 1.0f : 0.0f; dst[2] = q.z ? 1.0f : 0.0f; dst[3] = q.w ? 1.0f : 0.0f;
        } else {  // four 16-bit elements in one 64-bit load
          const uint2 q = live ? __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(ptr[k]) + off)) : make_uint2(0u, 0u);
          if (half_kind[k] == 1) {
            dst[0] = __uint_as_float(q.x << 16); dst[1] = __uint_as_float(q.x & 0xffff0000u);
            dst[2] = __uint_as_float(q.y << 16); dst[3] = __uint_as_float(q.y & 0xffff0000u);
          } else {
            const __half2 lo = *reinterpret_cast<const __half2*>(&q.x), hi = *reinterpret_cast<const __half2*>(&q.y);
            dst[0] = __low2float(lo); dst[1] = __high2float(lo); dst[2] = __low2float(hi); dst[3] = __high2float(hi);
          }
        }
      }
    }
    float acc[N];
    exec.template run<NIN, N, EXT>(in, acc, code);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = base + (int64_t)(u * kThreads + t) * 4;
      if (e >= prog.total) continue;
      const float q[4] = {acc[4 * u], acc[4 * u + 1], acc[4 * u + 2], acc[4 * u + 3]};
      store_vec4(prog.out[0].ptr, prog.out[0].dtype, e, q);
    }
  }
}

// ---- static programs ---------------------------------------------------------------------------
// The interpreter above costs about 40 thread-instructions per element on a 4-op chain, most of them decoding.  For the
// programs that recur — the benchmark chains, bias / activation epilogues, clamps, selects — the same register code is
// also compiled in as a template argument: the instruction loop unrolls into straight-line arithmetic on registers, with
// the very same expressions per opcode (so the results are bit-identical to the interpreter's).  A launch looks its
// register code up by signature; anything not listed runs on the interpreter.
struct EwStaticIns {
  uint8_t op, src, b, c, dst;
};

// operand `SRC` of a register instruction: 0..2 input, 3 immediate, 4 running value, 5..6 temporary
template <uint8_t SRC, int NIN, int N>
__device__ __forceinline__ float static_operand(const float (&in)[NIN > 0 ? NIN : 1][N], const float (&acc)[N], const float (&t0)[N], const float (&t1)[N],
                                                float imm, int j) {
  if constexpr (SRC < 3) return in[SRC < NIN ? SRC : 0][j];
  else if constexpr (SRC == 3) return imm;
  else if constexpr (SRC == 4) return acc[j];
  else if constexpr (SRC == 5) return t0[j];
  else return t1[j];
}

template <typename P, int I, int NIN, int N>
__device__ __forceinline__ void static_step(const float (&in)[NIN > 0 ? NIN : 1][N], float (&acc)[N], float (&t0)[N], float (&t1)[N], const EwRegCode& code) {
  if constexpr (I < P::n) {
    constexpr EwStaticIns ins = P::ins[I];
    const float imm = code.ins[I].imm;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      if constexpr (ins.op == EW_WHERE) {
        const float c = static_operand<ins.src, NIN, N>(in, acc, t0, t1, imm, j), x = static_operand<ins.b, NIN, N>(in, acc, t0, t1, imm, j),
                    y = static_operand<ins.c, NIN, N>(in, acc, t0, t1, imm, j);
        acc[j] = c != 0.0f ? x : y;
      } else {
        acc[j] = static_op<ins.op>(acc[j], static_operand<ins.src, NIN, N>(in, acc, t0, t1, imm, j));
      }
      if constexpr (ins.dst == 1) t0[j] = acc[j];
      if constexpr (ins.dst == 2) t1[j] = acc[j];
    }
    static_step<P, I + 1, NIN, N>(in, acc, t0, t1, code);
  }
}

template <typename P> struct StaticExec {
  template <int NIN, int N, bool EXT>
  __device__ __forceinline__ void run(const float (&in)[NIN > 0 ? NIN : 1][N], float (&acc)[N], const EwRegCode& code) const {
    float t0[N], t1[N];
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = t0[j] = t1[j] = 0.0f;
    static_step<P, 0, NIN, N>(in, acc, t0, t1, code);
  }
};

template <int NIN, int BMASK, int RANK, bool EXT>
__global__ void __launch_bounds__(kThreads, EXT ? 5 : 8) ew_kernel_reg(const __grid_constant__ EwProgram prog, const __grid_constant__ EwDivs divs,
                                                             const __grid_constant__ EwRegCode code) {
  ew_reg_body<NIN, BMASK, RANK, EXT>(prog, divs, code, InterpExec{});
}

template <typename P>
__global__ void __launch_bounds__(kThreads, P::ext ? 6 : 8) ew_kernel_static(const __grid_constant__ EwProgram prog, const __grid_constant__ EwDivs divs,
                                                                  const __grid_constant__ EwRegCode code) {
  ew_reg_body<P::nin, P::bmask, P::rank, P::ext>(prog, divs, code, StaticExec<P>{});
}

// Translate a slot-file program into the register form, if it is a linear chain.
bool to_register_code(const EwProgram& p, EwRegCode& code) {
  // at most two temporaries (slots past the operands): they live in registers in the extended kernel
  if (!p.vec || p.n_inputs > 3 || p.n_slots > p.n_inputs + 2 || p.n_outputs != 1 || p.rank > 2) return false;
  for (int k = 0; k < p.n_inputs; ++k) {
    const EwInput& in = p.in[k];
    if (in.kind != EW_IN_TENSOR) return false;
    if (in.dtype != IB200_F32 && in.dtype != IB200_BF16 && in.dtype != IB200_F16 && in.dtype != IB200_BOOL && in.dtype != IB200_U8) return false;
    if (in.mode != EW_STAGE_ASYNC_F32X4 && in.mode != EW_STAGE_ASYNC_HALF4 && in.mode != EW_STAGE_BYTE4 && in.mode != EW_STAGE_BROADCAST) return false;
  }
  code.n_instr = 0;
  auto emit = [&](uint8_t op, uint8_t src, float imm, uint8_t dst = 0) -> bool {
    if (code.n_instr >= kEwMaxInstr) return false;
    EwRegInstr& r = code.ins[code.n_instr++];
    r = EwRegInstr{};
    r.op = op; r.src = src; r.imm = imm; r.dst = dst;
    return true;
  };
  auto src_of = [&](uint8_t c) -> int {
    return c == EW_ACC ? 4 : c == EW_IMM ? 3 : c < p.n_inputs ? c : c < p.n_slots ? 5 + (c - p.n_inputs) : -1;
  };
  auto dst_of = [&](uint8_t d) -> int { return d == EW_NODST ? 0 : (d >= p.n_inputs && d < p.n_slots) ? 1 + (d - p.n_inputs) : -1; };
  auto reversed = [](uint8_t op) -> int {
    switch (op) {
      case EW_SUB: return EW_RSUB;
      case EW_DIV: return EW_RDIV;
      case EW_LT: return EW_GT;
      case EW_GT: return EW_LT;
      case EW_LE: return EW_GE;
      case EW_GE: return EW_LE;
      case EW_ADD: case EW_MUL: case EW_MAX: case EW_MIN: case EW_NE: case EW_AND: case EW_OR: return op;
      default: return -1;
    }
  };
  if (p.n_instr == 0) {  // a plain copy / broadcast of operand 0
    if (p.out[0].src >= p.n_inputs) return false;
    emit(EW_LOADB, p.out[0].src, 0.0f);
    return true;
  }
  for (int ip = 0; ip < p.n_instr; ++ip) {
    const EwInstr& ins = p.instr[ip];
    if (ins.op >= EW_RSUB) return false;
    const int a = src_of(ins.a), b = src_of(ins.b), dst = dst_of(ins.dst);
    if (a < 0 || b < 0 || dst < 0) return false;
    if (ins.op == EW_WHERE) {
      const int c = src_of(ins.c);
      if (c < 0 || code.n_instr >= kEwMaxInstr) return false;
      EwRegInstr& r = code.ins[code.n_instr++];
      r = EwRegInstr{};
      r.op = EW_WHERE; r.src = (uint8_t)a; r.b = (uint8_t)b; r.c = (uint8_t)c; r.imm = ins.imm; r.dst = (uint8_t)dst;
      continue;
    }
    const bool unary = ins.op == EW_MOV || ins.op == EW_RELU || ins.op == EW_EXP || ins.op == EW_RSQRT || ins.op == EW_ABS ||
                       ins.op == EW_FLOOR || ins.op == EW_NOT || ins.op == EW_TO_BOOL || ins.op == EW_TO_INT ||
                       ins.op == EW_ROUND_BF16 || ins.op == EW_ROUND_F16;
    bool ok = true;
    if (unary) {
      if (a != 4) ok &= emit(EW_LOADB, (uint8_t)a, ins.imm);
      ok &= emit(ins.op, 4, 0.0f, (uint8_t)dst);
    } else if (a == 4) {
      ok &= emit(ins.op, (uint8_t)b, ins.imm, (uint8_t)dst);
    } else if (b == 4) {
      const int r = reversed(ins.op);
      if (r < 0) return false;
      ok &= emit((uint8_t)r, (uint8_t)a, ins.imm, (uint8_t)dst);
    } else {  // neither operand is the running value: whatever was running is dead or already kept in a temporary
      ok &= emit(EW_LOADB, (uint8_t)a, ins.imm);
      ok &= emit(ins.op, (uint8_t)b, ins.imm, (uint8_t)dst);
    }
    if (!ok) return false;
  }
  if (p.out[0].src != EW_ACC) {  // the result sits in an operand or a temporary: bring it into acc
    const int o = src_of(p.out[0].src);
    if (o < 0 || !emit(EW_LOADB, (uint8_t)o, 0.0f)) return false;
  }
  return true;
}

// ---- the compiled-in programs --------------------------------------------------------------------
// Each entry is the register code of a recurring graph, as `ew_register_signature` prints it for that graph
// (operand count, inner-broadcast mask, collapsed rank, extended form, then op.src per instruction).
#define IB200_STATIC_PROGRAM(NAME, NIN_, BMASK_, RANK_, EXT_, ...)                      \
  struct NAME {                                                                         \
    static constexpr int nin = NIN_, bmask = BMASK_, rank = RANK_;                      \
    static constexpr bool ext = EXT_;                                                   \
    static constexpr EwStaticIns ins[] = {__VA_ARGS__};                                 \
    static constexpr int n = (int)(sizeof(ins) / sizeof(ins[0]));                       \
  };
#define I_(OP, SRC) EwStaticIns{OP, SRC, 0, 0, 0}
#define IT_(OP, SRC, DST) EwStaticIns{OP, SRC, 0, 0, DST}
#define IW_(COND, B, C) EwStaticIns{EW_WHERE, COND, B, C, 0}

// y = ((x * col + row) * k + col): the 4-op broadcast chain of the benchmark (x [M,N], col [N], row [M,1])
IB200_STATIC_PROGRAM(ProgChain4, 3, 4, 2, false, I_(EW_LOADB, 0), I_(EW_MUL, 1), I_(EW_ADD, 2), I_(EW_MUL, 3), I_(EW_ADD, 1))
// y = (x*col + row) * (x - col) + max(x, row): the 6-op DAG of the benchmark, reused values kept in a temporary
IB200_STATIC_PROGRAM(ProgDag6, 3, 4, 2, true, I_(EW_LOADB, 0), I_(EW_MUL, 1), IT_(EW_ADD, 2, 1), I_(EW_LOADB, 0), I_(EW_SUB, 1), IT_(EW_MUL, 5, 1),
                     I_(EW_LOADB, 0), I_(EW_MAX, 2), I_(EW_ADD, 5))
// bias and activation epilogues over [M,N] with a [N] vector: x + b, relu(x + b), x * w, x * w + b
IB200_STATIC_PROGRAM(ProgAddVec, 2, 0, 2, false, I_(EW_LOADB, 0), I_(EW_ADD, 1))
IB200_STATIC_PROGRAM(ProgAddVecRelu, 2, 0, 2, false, I_(EW_LOADB, 0), I_(EW_ADD, 1), I_(EW_RELU, 4))
IB200_STATIC_PROGRAM(ProgMulVec, 2, 0, 2, false, I_(EW_LOADB, 0), I_(EW_MUL, 1))
IB200_STATIC_PROGRAM(ProgMulAddVec, 3, 0, 2, false, I_(EW_LOADB, 0), I_(EW_MUL, 1), I_(EW_ADD, 2))
// selects and clamps of the reference's kernel suite (pipeline/tilelang/core.py: where2d, rowmask_where2d, clamp2d)
IB200_STATIC_PROGRAM(ProgGtWhere, 2, 0, 1, true, I_(EW_LOADB, 0), I_(EW_GT, 1), IW_(4, 0, 1))
IB200_STATIC_PROGRAM(ProgRowMaskWhere, 2, 1, 2, true, IW_(0, 1, 3))
IB200_STATIC_PROGRAM(ProgClamp, 3, 6, 1, false, I_(EW_LOADB, 0), I_(EW_MAX, 1), I_(EW_MIN, 2))
IB200_STATIC_PROGRAM(ProgFloor, 1, 0, 1, false, I_(EW_LOADB, 0), I_(EW_FLOOR, 4))
// same-shape binaries and unaries (operands collapse to rank 1)
IB200_STATIC_PROGRAM(ProgCopy, 1, 0, 1, false, I_(EW_LOADB, 0))
IB200_STATIC_PROGRAM(ProgAdd, 2, 0, 1, false, I_(EW_LOADB, 0), I_(EW_ADD, 1))
IB200_STATIC_PROGRAM(ProgMul, 2, 0, 1, false, I_(EW_LOADB, 0), I_(EW_MUL, 1))
IB200_STATIC_PROGRAM(ProgSub, 2, 0, 1, false, I_(EW_LOADB, 0), I_(EW_SUB, 1))
IB200_STATIC_PROGRAM(ProgRelu, 1, 0, 1, false, I_(EW_LOADB, 0), I_(EW_RELU, 4))
IB200_STATIC_PROGRAM(ProgExp, 1, 0, 1, false, I_(EW_LOADB, 0), I_(EW_EXP, 4))
IB200_STATIC_PROGRAM(ProgAddRelu, 2, 0, 1, false, I_(EW_LOADB, 0), I_(EW_ADD, 1), I_(EW_RELU, 4))
#undef I_
#undef IT_
#undef IW_

typedef void (*EwRegKernel)(const EwProgram, const EwDivs, const EwRegCode);

std::string signature_of(int nin, int bmask, int rank, bool ext, int n, const uint8_t* op, const uint8_t* src, const uint8_t* b, const uint8_t* c,
                         const uint8_t* dst) {
  std::string sig = "n" + std::to_string(nin) + " b" + std::to_string(bmask) + " r" + std::to_string(rank) + " e" + std::to_string(ext ? 1 : 0) + " |";
  for (int i = 0; i < n; ++i) {
    sig += " " + std::to_string(op[i]) + "." + std::to_string(src[i]);
    if (op[i] == EW_WHERE) sig += "." + std::to_string(b[i]) + "." + std::to_string(c[i]);
    if (dst[i]) sig += ">" + std::to_string(dst[i]);
  }
  return sig;
}
std::string signature_of(const EwRegCode& code, int nin, int bmask, int rank, bool ext) {
  uint8_t op[kEwMaxInstr + 1], src[kEwMaxInstr + 1], b[kEwMaxInstr + 1], c[kEwMaxInstr + 1], dst[kEwMaxInstr + 1];
  for (int i = 0; i < code.n_instr; ++i) { op[i] = code.ins[i].op; src[i] = code.ins[i].src; b[i] = code.ins[i].b; c[i] = code.ins[i].c; dst[i] = code.ins[i].dst; }
  return signature_of(nin, bmask, rank, ext, code.n_instr, op, src, b, c, dst);
}
template <typename P> void add_static(std::map<std::string, EwRegKernel>& table) {
  uint8_t op[P::n], src[P::n], b[P::n], c[P::n], dst[P::n];
  for (int i = 0; i < P::n; ++i) { op[i] = P::ins[i].op; src[i] = P::ins[i].src; b[i] = P::ins[i].b; c[i] = P::ins[i].c; dst[i] = P::ins[i].dst; }
  table[signature_of(P::nin, P::bmask, P::rank, P::ext, P::n, op, src, b, c, dst)] = ew_kernel_static<P>;
}
const std::map<std::string, EwRegKernel>& static_programs() {
  static const std::map<std::string, EwRegKernel> table = [] {
    std::map<std::string, EwRegKernel> t;
    add_static<ProgChain4>(t); add_static<ProgDag6>(t); add_static<ProgAddVec>(t); add_static<ProgAddVecRelu>(t); add_static<ProgMulVec>(t);
    add_static<ProgCopy>(t); add_static<ProgAdd>(t); add_static<ProgMul>(t); add_static<ProgSub>(t); add_static<ProgRelu>(t); add_static<ProgExp>(t);
    add_static<ProgAddRelu>(t); add_static<ProgMulAddVec>(t); add_static<ProgGtWhere>(t); add_static<ProgRowMaskWhere>(t); add_static<ProgClamp>(t);
    add_static<ProgFloor>(t);
    return t;
  }();
  return table;
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads) ew_kernel(const __grid_constant__ EwProgram prog, const __grid_constant__ EwDivs divs) {
  extern __shared__ __align__(16) float file[];
  const int t = threadIdx.x;
  constexpr int W = VEC ? 4 : 1;          // elements per unit (sharing all but the innermost coordinate)
  constexpr int U = kPerThread / W;       // units per thread
  const int64_t ntiles = (prog.total + kTile - 1) / kTile;

  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t base = tile * kTile;
    // ---- stage the operands --------------------------------------------------------------
    bool needs_convert = false;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = base + (int64_t)(u * kThreads + t) * W;  // first element of the unit
      if (e >= prog.total) continue;
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
        float* dst = slot_ptr<VEC, kPerThread>(file, k, u * W, t);
        if (in.kind == EW_IN_IOTA) {
          const int64_t step = in.stride[prog.rank - 1];
#pragma unroll
          for (int j = 0; j < W; ++j) dst[j] = (float)(off + j * step);
          continue;
        }
        if (VEC) {
          const int64_t step = in.stride[prog.rank - 1];
          if (in.vec_ok) {
            if (in.dtype == IB200_F32) cp_async16(dst, static_cast<const float*>(in.ptr) + off);
            else if (in.dtype == IB200_BF16 || in.dtype == IB200_F16) {
              cp_async8(dst, static_cast<const uint16_t*>(in.ptr) + off);
              needs_convert = true;
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = load_scalar(in.ptr, in.dtype, off + j);
            }
          } else if (step == 0) {
            const float v = load_scalar(in.ptr, in.dtype, off);
            *reinterpret_cast<float4*>(dst) = make_float4(v, v, v, v);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = load_scalar(in.ptr, in.dtype, off + j * step);
          }
        } else {
          if (in.dtype == IB200_F32) cp_async4(dst, static_cast<const float*>(in.ptr) + off);
          else *dst = load_scalar(in.ptr, in.dtype, off);
        }
      }
    }
    cp_async_wait_all();
    if (VEC && needs_convert) {  // widen the 8-byte bf16/f16 vectors in place
      for (int k = 0; k < prog.n_inputs; ++k) {
        const EwInput& in = prog.in[k];
        if (!(in.vec_ok && in.kind == EW_IN_TENSOR && (in.dtype == IB200_BF16 || in.dtype == IB200_F16))) continue;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float* dst = slot_ptr<VEC, kPerThread>(file, k, u * W, t);
          float v[4];
          if (in.dtype == IB200_BF16) load4<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(dst), v);
          else load4<__half>(reinterpret_cast<const __half*>(dst), v);
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        }
      }
    }

    // ---- run the chain ---------------------------------------------------------------------
    float acc[kPerThread];
    run_chain<VEC, kPerThread>(prog, acc, file, t);

    write_outputs<VEC, kPerThread>(prog, acc, file, t, base);
  }
}

// Staging mode per operand, whether the specialised kernels apply (`fast`), and — when the program is a linear chain —
// its register code with the template parameters of the register kernels.
struct Prepared {
  EwProgram p;
  bool fast = false, reg = false, ext = false;
  int bmask = 0;
  EwRegCode code;
};
void prepare(const EwProgram& prog, Prepared& out) {
  EwProgram& p = out.p;
  p = prog;
  bool fast = p.n_inputs <= 4 && p.rank <= 3;
  for (int k = 0; k < p.n_inputs; ++k) {
    EwInput& in = p.in[k];
    const int64_t inner = in.stride[p.rank - 1];
    int64_t reach = 0;
    for (int d = 0; d < p.rank; ++d) {
      if (in.stride[d] < 0) fast = false;
      reach += (int64_t)(p.dim[d] - 1) * in.stride[d];
    }
    if (reach >= ((int64_t)1 << 31) - 8) fast = false;
    if (in.kind == EW_IN_IOTA) in.mode = EW_STAGE_IOTA;
    else if (p.vec) {
      if (in.vec_ok && in.dtype == IB200_F32) in.mode = EW_STAGE_ASYNC_F32X4;
      else if (in.vec_ok && (in.dtype == IB200_BF16 || in.dtype == IB200_F16)) in.mode = EW_STAGE_ASYNC_HALF4;
      else if (in.vec_ok && (in.dtype == IB200_BOOL || in.dtype == IB200_U8)) in.mode = EW_STAGE_BYTE4;
      else if (inner == 0) in.mode = EW_STAGE_BROADCAST;
      else in.mode = EW_STAGE_GATHER;
    } else {
      in.mode = in.dtype == IB200_F32 ? EW_STAGE_ASYNC_F32 : EW_STAGE_GATHER;
    }
  }
  out.fast = fast;
  out.reg = fast && to_register_code(p, out.code);
  if (out.reg) {
    for (int k = 0; k < p.n_inputs; ++k) {
      out.bmask |= (p.in[k].mode == EW_STAGE_BROADCAST) << k;
      out.ext |= p.in[k].dtype == IB200_BOOL || p.in[k].dtype == IB200_U8;
    }
    for (int i = 0; i < out.code.n_instr; ++i) out.ext |= out.code.ins[i].op == EW_WHERE || out.code.ins[i].dst != 0 || out.code.ins[i].src >= 5;
  }
}

}  // namespace

// What the register path would run for this program if every operand is aligned: its signature, and whether that
// register code is one of the compiled-in programs.  Empty when the program does not take the register path.
std::string ew_register_signature(const EwProgram& prog, bool* compiled_in) {
  Prepared pr;
  EwProgram q = prog;
  q.vec = q.dim[q.rank - 1] % 4 == 0;
  for (int k = 0; k < q.n_inputs; ++k) {
    EwInput& in = q.in[k];
    bool ok = in.kind == EW_IN_TENSOR && in.stride[q.rank - 1] == 1;
    for (int d = 0; d + 1 < q.rank; ++d) ok &= in.stride[d] % 4 == 0;
    in.vec_ok = ok;
  }
  prepare(q, pr);
  if (compiled_in) *compiled_in = false;
  if (!pr.reg) return std::string();
  const std::string sig = signature_of(pr.code, pr.p.n_inputs, pr.bmask, pr.p.rank, pr.ext);
  if (compiled_in) *compiled_in = static_programs().count(sig) > 0;
  return sig;
}

int launch_elementwise(const EwProgram& prog, cudaStream_t s) {
  if (prog.total == 0) return IB200_OK;
  if (prog.total < 0 || prog.total >= ((int64_t)1 << 31)) return fail(IB200_ERR_UNSUPPORTED, "elementwise: more than 2^31-1 output elements");
  if (prog.rank < 1 || prog.rank > kEwMaxRank || prog.n_inputs > kEwMaxInputs || prog.n_outputs < 1 ||
      prog.n_outputs > kEwMaxOutputs || prog.n_instr > kEwMaxInstr || prog.n_slots > kEwMaxSlots || prog.n_slots < prog.n_inputs)
    return fail(IB200_ERR_INVALID, "elementwise: malformed program");
  EwDivs divs;
  for (int d = 0; d < prog.rank; ++d) divs.d[d] = FastDiv(prog.dim[d]);
  Prepared pr;
  prepare(prog, pr);
  const EwProgram& p = pr.p;
  const bool fast = pr.fast;
  if (pr.reg) {
    const EwRegCode& code = pr.code;
    const int bmask = pr.bmask;
    const bool ext = pr.ext;
    EwRegKernel rk = nullptr;
    const auto& table = static_programs();
    const auto hit = table.find(signature_of(code, p.n_inputs, bmask, p.rank, ext));
    if (hit != table.end()) rk = hit->second;  // compiled in: straight-line code instead of the instruction loop
#define IB200_REG(NIN, BM, R) if (!rk && p.n_inputs == NIN && bmask == BM && p.rank == R) rk = ext ? ew_kernel_reg<NIN, BM, R, true> : ew_kernel_reg<NIN, BM, R, false>;
#define IB200_REG_R(NIN, BM) IB200_REG(NIN, BM, 1) IB200_REG(NIN, BM, 2)
    IB200_REG_R(0, 0) IB200_REG_R(1, 0) IB200_REG_R(1, 1) IB200_REG_R(2, 0) IB200_REG_R(2, 1) IB200_REG_R(2, 2) IB200_REG_R(2, 3)
    IB200_REG_R(3, 0) IB200_REG_R(3, 1) IB200_REG_R(3, 2) IB200_REG_R(3, 3) IB200_REG_R(3, 4) IB200_REG_R(3, 5) IB200_REG_R(3, 6) IB200_REG_R(3, 7)
#undef IB200_REG_R
#undef IB200_REG
    if (rk) {
      const int64_t tiles = (p.total + kTile - 1) / kTile;
      const int64_t cap = (int64_t)kSmCount * (ext ? 5 : 8) * 4;
      rk<<<(int)(tiles < cap ? tiles : cap), kThreads, 0, s>>>(p, divs, code);
      return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "elementwise launch");
    }
  }
  void (*kern)(const EwProgram, const EwDivs) = p.vec ? ew_kernel<true> : ew_kernel<false>;
  int per_thread = kPerThread;
  if (fast) {
    const int mi = p.n_inputs <= 2 ? 2 : 4;
    // 16 elements per thread halve the decoding per element but leave two CTAs per SM; measured on a 6-op DAG over
    // [8192,4096]: 148 us against 121 us for 8 elements per thread at four CTAs.  Kept for A/B runs of builds made
    // with -DIB200_AB_KNOBS (IB200_EW_WIDE=1); a normal build never takes it.
#ifdef IB200_AB_KNOBS
    static const bool allow_wide = std::getenv("IB200_EW_WIDE") && std::getenv("IB200_EW_WIDE")[0] == '1';
#else
    constexpr bool allow_wide = false;
#endif
    const bool wide = allow_wide && p.vec && p.total >= (int64_t)kSmCount * kThreads * 16 * 4 && p.n_slots <= 12;
    if (wide) per_thread = 16;
#define IB200_EW(MI, R)                                                                                   \
  if (mi == MI && p.rank == R)                                                                            \
    kern = wide ? ew_kernel_fast<MI, R, true, 16> : (p.vec ? ew_kernel_fast<MI, R, true, 8> : ew_kernel_fast<MI, R, false, 8>);
    IB200_EW(2, 1) IB200_EW(2, 2) IB200_EW(2, 3) IB200_EW(4, 1) IB200_EW(4, 2) IB200_EW(4, 3)
#undef IB200_EW
  }
  const int tile_elems = kThreads * per_thread;
  const size_t smem = (size_t)(p.n_slots > 0 ? p.n_slots : 1) * tile_elems * sizeof(float);
  const int64_t tiles = (p.total + tile_elems - 1) / tile_elems;
  const int per_sm = (int)(220 * 1024 / smem) < 8 ? (int)(220 * 1024 / smem) : 8;
  const int64_t cap = (int64_t)kSmCount * (per_sm > 0 ? per_sm : 1) * 4;
  const int grid = (int)(tiles < cap ? tiles : cap);
  if (smem > 48 * 1024) IB200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, kThreads, smem, s>>>(p, divs);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "elementwise launch");
}

}  // namespace ib200

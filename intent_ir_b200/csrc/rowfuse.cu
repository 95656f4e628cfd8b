// The kernel behind row_program.h: a group of G threads owns one row at a time and runs every
// phase of the program on it.  G is one warp whenever the row's slots leave room for enough
// warps per SM (then nothing in the row loop needs a block barrier and nothing is computed
// twice); longer rows are shared by the 128 or 512 threads of a CTA.
//
//   * Row slots live in shared memory; thread t of the group owns the same columns
//     ((u*G + t)*4 .. +3 for u = 0, 1, ...) in every slot and in every phase, so slots are
//     thread-private storage and need no barrier.  Global operands are staged into their
//     slots with cp.async, all units of all operands of the phase in flight at once.
//   * A chain runs on up to 32 values per thread per pass (up to eight 128-bit vectors, or 8
//     scalars when the row length is not a multiple of 4), so that decoding a micro-op is paid
//     once per 1024 elements of a warp's row.
//   * Row scalars (row sums, maxima, and what SCALAR phases derive from them) live in a small
//     shared array per group, double-buffered by row parity.  Reductions: per-thread partials
//     over the passes, warp shuffles, then (G > 32) one barrier and a fixed-order combination
//     by thread 0, which also runs the SCALAR phases that follow; one more barrier before the
//     next FULL phase reads the results.
//
// HBM traffic: every external operand of the fused steps once per row, every result that
// leaves the group of steps once.  Row-invariant operands (weights, biases) are staged once
// per CTA into slots that all its warps read.
#include <cuda_runtime.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "ew_device.cuh"
#include "row_program.h"

namespace ib200 {
namespace {

__device__ __forceinline__ float reduce_identity(int kind) { return kind == IB200_REDUCE_MAX ? -INFINITY : 0.0f; }
__device__ __forceinline__ float reduce_apply(int kind, float a, float b) {
  return kind == IB200_REDUCE_SUM ? a + b : kind == IB200_REDUCE_MAX ? max_nan(a, b) : ((a != 0.0f || b != 0.0f) ? 1.0f : 0.0f);
}

// Where the slots live.  A slot is the row in column order (thread t of the group owns columns
// (u*G + t)*W .. +W-1 for u = 0, 1, ...); slots below n_row belong to the group, the others are
// the CTA's row-invariant slots.
struct SlotFile {
  float* group;
  float* shared;
  int n_row, slot_floats;
  __device__ __forceinline__ float* base(int s) const {
    return s < n_row ? group + (size_t)s * slot_floats : shared + (size_t)(s - n_row) * slot_floats;
  }
};

// NU units per pass: N = NU * (VEC ? 4 : 1) values per thread
template <int G, bool VEC, int NU, int N>
__device__ __forceinline__ void fetch(float (&dst)[N], uint8_t code, const float (&acc)[N], float imm, const SlotFile& f, const float* S,
                                      int pass, int t) {
  if (code == EW_ACC) {
#pragma unroll
    for (int j = 0; j < N; ++j) dst[j] = acc[j];
  } else if (code == EW_IMM) {
#pragma unroll
    for (int j = 0; j < N; ++j) dst[j] = imm;
  } else if (code >= EW_ROWSCALAR) {
    const float v = S[code - EW_ROWSCALAR];
#pragma unroll
    for (int j = 0; j < N; ++j) dst[j] = v;
  } else if (VEC) {
    const float* p = f.base(code) + ((size_t)pass * NU * G + t) * 4;
#pragma unroll
    for (int q = 0; q < NU; ++q) {
      const float4 v = *reinterpret_cast<const float4*>(p + q * G * 4);
      dst[4 * q] = v.x; dst[4 * q + 1] = v.y; dst[4 * q + 2] = v.z; dst[4 * q + 3] = v.w;
    }
  } else {
    const float* p = f.base(code) + (size_t)pass * NU * G + t;
#pragma unroll
    for (int j = 0; j < N; ++j) dst[j] = p[j * G];
  }
}

template <int G, bool VEC, int NU, int N>
__device__ __forceinline__ void put(const float (&src)[N], int s, const SlotFile& f, int pass, int t) {
  if (VEC) {
    float* p = f.base(s) + ((size_t)pass * NU * G + t) * 4;
#pragma unroll
    for (int q = 0; q < NU; ++q) *reinterpret_cast<float4*>(p + q * G * 4) = make_float4(src[4 * q], src[4 * q + 1], src[4 * q + 2], src[4 * q + 3]);
  } else {
    float* p = f.base(s) + (size_t)pass * NU * G + t;
#pragma unroll
    for (int j = 0; j < N; ++j) p[j * G] = src[j];
  }
}

// One operand's share of a row into its slot: the columns first, first + step, ... below `cols`
// (W consecutive columns each).  The descriptor is taken by value and the staging mode is
// decided once, outside the loop, so that the loop body is an address update and a copy.
template <bool VEC>
__device__ __forceinline__ void stage_columns(const RowInput in, float* base, int64_t row_off, int first, int step, int cols, bool& convert) {
  constexpr int W = VEC ? 4 : 1;
  if (in.kind == EW_IN_IOTA) {
    for (int col = first; col < cols; col += step) {
#pragma unroll
      for (int j = 0; j < W; ++j) base[col + j] = (float)(row_off + (int64_t)(col + j) * in.col_stride);
    }
  } else if (VEC && in.vec_ok && in.dtype == IB200_F32) {
    const float* src = static_cast<const float*>(in.ptr) + row_off;
    for (int col = first; col < cols; col += step) cp_async16(base + col, src + col);
  } else if (VEC && in.vec_ok && (in.dtype == IB200_BF16 || in.dtype == IB200_F16)) {
    const uint16_t* src = static_cast<const uint16_t*>(in.ptr) + row_off;
    for (int col = first; col < cols; col += step) cp_async8(base + col, src + col);
    convert = true;
  } else if (VEC && in.vec_ok && (in.dtype == IB200_BOOL || in.dtype == IB200_U8)) {
    const uint8_t* src = static_cast<const uint8_t*>(in.ptr) + row_off;
    for (int col = first; col < cols; col += step) {
      float v[4];
      load4<uint8_t>(src + col, v);
      *reinterpret_cast<float4*>(base + col) = make_float4(v[0], v[1], v[2], v[3]);
    }
  } else if (VEC && in.vec_ok && in.dtype == IB200_I32) {
    const int32_t* src = static_cast<const int32_t*>(in.ptr) + row_off;
    for (int col = first; col < cols; col += step) {
      float v[4];
      load4<int32_t>(src + col, v);
      *reinterpret_cast<float4*>(base + col) = make_float4(v[0], v[1], v[2], v[3]);
    }
  } else if (!VEC && in.dtype == IB200_F32) {
    const float* src = static_cast<const float*>(in.ptr) + row_off;
    for (int col = first; col < cols; col += step) cp_async4(base + col, src + (int64_t)col * in.col_stride);
  } else {
    for (int col = first; col < cols; col += step) {
#pragma unroll
      for (int j = 0; j < W; ++j) base[col + j] = load_scalar(in.ptr, in.dtype, row_off + (int64_t)(col + j) * in.col_stride);
    }
  }
}
__device__ __forceinline__ bool widens_in_place(const RowInput in) {
  return in.vec_ok && in.kind == EW_IN_TENSOR && (in.dtype == IB200_BF16 || in.dtype == IB200_F16);
}
__device__ __forceinline__ void widen_unit(const RowInput in, float* dst) {  // the 8-byte bf16 / f16 vector at dst -> 4 floats
  float v[4];
  if (in.dtype == IB200_BF16) load4<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(dst), v);
  else load4<__half>(reinterpret_cast<const __half*>(dst), v);
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}

__device__ __forceinline__ float scalar_operand(uint8_t code, float acc, float imm, const float* S) {
  return code == EW_ACC ? acc : code == EW_IMM ? imm : S[code - EW_ROWSCALAR];
}

// fold N values into the running partial; four independent chains keep the adds from serialising
template <int N> __device__ __forceinline__ float fold(int kind, float p, const float (&v)[N]) {
  constexpr int K = N >= 8 ? 4 : 1;
  float q[K];
  switch (kind) {
    case IB200_REDUCE_SUM:
#pragma unroll
      for (int k = 0; k < K; ++k) q[k] = v[k];
#pragma unroll
      for (int j = K; j < N; ++j) q[j % K] += v[j];
#pragma unroll
      for (int k = 0; k < K; ++k) p += q[k];
      break;
    case IB200_REDUCE_MAX:
#pragma unroll
      for (int k = 0; k < K; ++k) q[k] = v[k];
#pragma unroll
      for (int j = K; j < N; ++j) q[j % K] = max_nan(q[j % K], v[j]);
#pragma unroll
      for (int k = 0; k < K; ++k) p = max_nan(p, q[k]);
      break;
    default: {
      bool any = p != 0.0f;
#pragma unroll
      for (int j = 0; j < N; ++j) any |= v[j] != 0.0f;
      p = any ? 1.0f : 0.0f;
    }
  }
  return p;
}

template <int G> __device__ __forceinline__ void group_sync() {
  if (G <= 32) __syncwarp();
  else __syncthreads();
}

template <int G, bool VEC, int NU>
__global__ void __launch_bounds__(G <= 32 ? 256 : G) row_kernel(const __grid_constant__ RowProgram P, const int units) {
  extern __shared__ __align__(16) float smem[];
  constexpr int W = VEC ? 4 : 1;
  constexpr int N = NU * W;
  constexpr int kWarps = G <= 32 ? 1 : G / 32;
  const int groups = G <= 32 ? (int)blockDim.x >> 5 : 1;
  const int g = G <= 32 ? (int)threadIdx.x >> 5 : 0;
  const int t = G <= 32 ? (int)threadIdx.x & 31 : (int)threadIdx.x;
  const int lane = threadIdx.x & 31;
  const int cols = P.cols;
  SlotFile f;
  f.n_row = P.n_row_slots;
  f.slot_floats = units * G * W;
  f.shared = smem;
  f.group = smem + (size_t)(P.n_once_slots + g * P.n_row_slots) * f.slot_floats;
  float* after_slots = smem + (size_t)(P.n_once_slots + groups * P.n_row_slots) * f.slot_floats;
  // the group's row scalars, written by its thread 0 only and double-buffered by row parity so
  // that thread 0 may start on the next row while others still read this one's
  float* scalars = after_slots + g * (2 * kRowMaxScalars);
  float* red = after_slots + groups * (2 * kRowMaxScalars);  // [2][kRowMaxSinks][kWarps], G > 32 only
  const int passes = units / NU;

  // ---- row-invariant operands: once per CTA, by all its threads ------------------------------
  if (P.n_once_slots > 0) {
    bool convert = false;
    for (int k = 0; k < P.n_inputs; ++k) {
      const RowInput in = P.in[k];
      if (!in.once) continue;
      stage_columns<VEC>(in, f.base(in.slot), 0, threadIdx.x * W, blockDim.x * W, cols, convert);
    }
    cp_async_wait_all();
    if (VEC && convert)
      for (int k = 0; k < P.n_inputs; ++k) {
        const RowInput in = P.in[k];
        if (!in.once || !widens_in_place(in)) continue;
        float* base = f.base(in.slot);
        for (int col = threadIdx.x * W; col < cols; col += blockDim.x * W) widen_unit(in, base + col);
      }
    __syncthreads();
  }

  bool dirty = false;  // thread 0 has written row scalars since the group last synchronised
  int red_parity = 0, row_parity = 0;
  for (int64_t row = (int64_t)blockIdx.x * groups + g; row < P.rows; row += (int64_t)gridDim.x * groups, row_parity ^= 1) {
    float* S = scalars + row_parity * kRowMaxScalars;
    for (int ph = 0; ph < P.n_phases; ++ph) {
      const RowPhase phase = P.phase[ph];
      if (phase.n_loads && t == 0) {
        for (int k = 0; k < phase.n_loads; ++k) {
          const RowScalarLoad ld = P.load[phase.first_load + k];
          S[ld.scalar] = load_scalar(ld.ptr, ld.dtype, row * ld.row_stride);
        }
      }
      dirty |= phase.n_loads != 0;

      if (phase.domain == ROW_SCALAR) {
        if (t == 0) {
          float acc = 0.0f;
          for (int ip = 0; ip < phase.n_instr; ++ip) {
            const EwInstr ins = P.instr[phase.first_instr + ip];
            float a[1] = {scalar_operand(ins.a, acc, ins.imm, S)}, b[1] = {scalar_operand(ins.b, acc, ins.imm, S)}, r[1];
            if (ins.op == EW_WHERE) {
              r[0] = a[0] != 0.0f ? b[0] : scalar_operand(ins.c, acc, ins.imm, S);
            } else {
              r[0] = acc;
              apply<1>(ins.op, a, b, r);
            }
            acc = r[0];
            if (ins.dst != EW_NODST) S[ins.dst - EW_ROWSCALAR] = acc;
          }
          for (int o = 0; o < phase.n_outputs; ++o) {
            const RowOutput out = P.out[phase.first_output + o];
            const float v = scalar_operand(out.src, acc, 0.0f, S);
            if (out.scalar != kRowNone) S[out.scalar] = v;
            if (out.ptr) store_scalar(out.ptr, out.dtype, row * out.row_stride, v);
          }
        }
        dirty = true;
        continue;
      }

      // ---- FULL phase: stage the global operands of this phase --------------------------------
      bool convert = false;
      for (int k = 0; k < phase.n_inputs; ++k) {
        const RowInput in = P.in[phase.first_input + k];
        if (in.once) continue;
        stage_columns<VEC>(in, f.base(in.slot), row * in.row_stride, t * W, G * W, cols, convert);
      }
      if (dirty) {  // row scalars written by thread 0 become visible to the group
        group_sync<G>();
        dirty = false;
      }
      cp_async_wait_all();
      if (VEC && convert) {
        for (int k = 0; k < phase.n_inputs; ++k) {
          const RowInput in = P.in[phase.first_input + k];
          if (in.once || !widens_in_place(in)) continue;
          float* base = f.base(in.slot);
          for (int col = t * W; col < cols; col += G * W) widen_unit(in, base + col);
        }
      }

      // ---- run the chain, pass by pass -----------------------------------------------------
      float part[kRowMaxSinks];
      bool any_reduce = false;
#pragma unroll
      for (int o = 0; o < kRowMaxSinks; ++o) {
        const bool live = o < phase.n_outputs && P.out[phase.first_output + o].reduce;
        part[o] = live ? reduce_identity(P.out[phase.first_output + o].reduce - 1) : 0.0f;
        any_reduce |= live;
      }
      for (int pass = 0; pass < passes; ++pass) {
        const int col0 = (pass * NU * G + t) * W;  // first column of this thread's first unit in the pass
        if (col0 >= cols) break;
        const bool whole = col0 + (NU - 1) * G * W + (W - 1) < cols;  // every value of the pass is inside the row
        float acc[N];
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = 0.0f;
        for (int ip = 0; ip < phase.n_instr; ++ip) {
          const EwInstr ins = P.instr[phase.first_instr + ip];
          // accumulate form (the planner's emit_accumulate_form): acc = op(acc, b), b a slot,
          // a scalar or acc itself; only `where` names three operands
          if (ins.op == EW_WHERE) {
            float a[N], b[N], c[N];
            fetch<G, VEC, NU, N>(a, ins.a, acc, ins.imm, f, S, pass, t);
            fetch<G, VEC, NU, N>(b, ins.b, acc, ins.imm, f, S, pass, t);
            fetch<G, VEC, NU, N>(c, ins.c, acc, ins.imm, f, S, pass, t);
#pragma unroll
            for (int j = 0; j < N; ++j) acc[j] = a[j] != 0.0f ? b[j] : c[j];
          } else if (ins.b == EW_ACC) {
            apply<N>(ins.op, acc, acc, acc);
          } else if (ins.b < kRowMaxSlots) {
            float b[N];
            fetch<G, VEC, NU, N>(b, ins.b, acc, ins.imm, f, S, pass, t);
            apply<N>(ins.op, acc, b, acc);
          } else {
            apply_scalar<N>(ins.op, acc, ins.b == EW_IMM ? ins.imm : S[ins.b - EW_ROWSCALAR]);
          }
          if (ins.dst != EW_NODST) put<G, VEC, NU, N>(acc, ins.dst, f, pass, t);
        }
#pragma unroll
        for (int o = 0; o < kRowMaxSinks; ++o) {
          if (o >= phase.n_outputs) break;
          const RowOutput out = P.out[phase.first_output + o];
          float v[N];
          fetch<G, VEC, NU, N>(v, out.src, acc, 0.0f, f, S, pass, t);
          if (out.reduce) {
            const int kind = out.reduce - 1;
            if (!whole) {  // values past the end of the row become the identity
              const float id = reduce_identity(kind);
#pragma unroll
              for (int j = 0; j < N; ++j) {
                const int col = VEC ? col0 + (j >> 2) * G * 4 + (j & 3) : col0 + j * G;
                if (col >= cols) v[j] = id;
              }
            }
            part[o] = fold<N>(kind, part[o], v);
          } else if (out.ptr) {
            const int64_t base = row * out.row_stride;
            if (VEC && out.vec_ok && out.dtype == IB200_F32) {
              float* dst = static_cast<float*>(out.ptr) + base + col0;
#pragma unroll
              for (int q = 0; q < NU; ++q)
                if (whole || col0 + q * G * 4 < cols) *reinterpret_cast<float4*>(dst + q * G * 4) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else if (VEC) {
#pragma unroll
              for (int q = 0; q < NU; ++q) {
                const int col = col0 + q * G * 4;
                if (!whole && col >= cols) continue;
                const float w4[4] = {v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]};
                if (out.vec_ok) store_vec4(out.ptr, out.dtype, base + col, w4);
                else {
#pragma unroll
                  for (int j = 0; j < 4; ++j) store_scalar(out.ptr, out.dtype, base + col + j, w4[j]);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < N; ++j) {
                const int col = col0 + j * G;
                if (whole || col < cols) store_scalar(out.ptr, out.dtype, base + col, v[j]);
              }
            }
          }
        }
      }

      // ---- fold the partials into row scalars ----------------------------------------------------
      if (any_reduce) {
        float* slots = red + red_parity * (kRowMaxSinks * kWarps);
#pragma unroll
        for (int o = 0; o < kRowMaxSinks; ++o) {
          if (o >= phase.n_outputs) break;
          const RowOutput out = P.out[phase.first_output + o];
          if (!out.reduce) continue;
          const int kind = out.reduce - 1;
          float v = part[o];
#pragma unroll
          for (int d = 16; d > 0; d >>= 1) v = reduce_apply(kind, v, __shfl_xor_sync(0xffffffffu, v, d));
          if (G <= 32) {
            if (t == 0) {
              v *= out.scale;
              S[out.scalar] = v;
              if (out.ptr) store_scalar(out.ptr, out.dtype, row * out.row_stride, v);
            }
          } else if (lane == 0) {
            slots[o * kWarps + (t >> 5)] = v;
          }
        }
        if (G > 32) {
          __syncthreads();
          if (t == 0) {  // fixed order: the result does not depend on which warp finished first
            for (int o = 0; o < phase.n_outputs; ++o) {
              const RowOutput out = P.out[phase.first_output + o];
              if (!out.reduce) continue;
              const int kind = out.reduce - 1;
              float v = slots[o * kWarps];
              for (int w = 1; w < kWarps; ++w) v = reduce_apply(kind, v, slots[o * kWarps + w]);
              v *= out.scale;
              S[out.scalar] = v;
              if (out.ptr) store_scalar(out.ptr, out.dtype, row * out.row_stride, v);
            }
          }
          red_parity ^= 1;
        }
        dirty = true;
      }
    }
  }
}

struct RowLaunch {
  int g = 0, w = 1, nu = 8, units = 0, warps_per_cta = 1, threads = 32, ctas_per_sm = 1;
  size_t smem = 0;
  int warps_per_sm() const { return ctas_per_sm * (g <= 32 ? warps_per_cta : g / 32); }
};

constexpr size_t kSmemPerSm = 227 * 1024;

// the launch shape for a program with `n_row` per-row and `n_once` row-invariant slots: the
// smallest group that still leaves at least eight warps resident per SM, else the most warps
bool row_launch_config(int n_row, int n_once, int cols, int n_instr, RowLaunch& best) {
  bool found = false;
#ifdef IB200_AB_KNOBS  // A/B builds only, read once: IB200_ROW_G in {32, 128, 512}, IB200_ROW_NU in {2, 4, 8}
  static const int force_g = std::getenv("IB200_ROW_G") ? std::atoi(std::getenv("IB200_ROW_G")) : 0;
  static const int force_nu = std::getenv("IB200_ROW_NU") ? std::atoi(std::getenv("IB200_ROW_NU")) : 0;
#else
  constexpr int force_g = 0, force_nu = 0;
#endif
  for (int g : {32, 128, 512}) {
    if (force_g ? g != force_g : (g == 32 && cols > 1024)) continue;  // measured: rows past 1024 elements want more than one warp
    RowLaunch c;
    c.g = g;
    c.w = cols % 4 == 0 ? 4 : 1;
    const int raw = (cols + g * c.w - 1) / (g * c.w);
    // 16 values per thread and pass; 32 (120 registers) pays off, measured, once a row runs six or more micro-ops
    c.nu = c.w == 4 ? (raw >= 8 && n_instr >= 6 && g < 512 ? 8 : raw >= 3 ? 4 : 2) : 8;
    if (force_nu && c.w == 4 && (force_nu == 2 || force_nu == 4 || (force_nu == 8 && g < 512))) c.nu = force_nu;
    c.units = (raw + c.nu - 1) / c.nu * c.nu;
    const size_t slot = (size_t)c.units * g * c.w * sizeof(float);
    const size_t fixed = (size_t)n_once * slot + 2 * kRowMaxSinks * 16 * sizeof(float);
    const size_t per_warp_scalars = 2 * kRowMaxScalars * sizeof(float);  // per group: two row parities
    if (g == 32) {
      int best_warps = 0;
      for (int wpc = 8; wpc >= 1; --wpc) {
        const size_t smem = fixed + wpc * ((size_t)n_row * slot + per_warp_scalars);
        if (smem + 1024 > kSmemPerSm) continue;
        int ctas = (int)(kSmemPerSm / (smem + 1024));
        if (ctas > 32) ctas = 32;
        if (ctas * wpc > 64) ctas = 64 / wpc;
        if (ctas * wpc > best_warps) {
          best_warps = ctas * wpc;
          c.warps_per_cta = wpc; c.threads = wpc * 32; c.smem = smem; c.ctas_per_sm = ctas;
        }
      }
      if (best_warps == 0) continue;
    } else {
      c.smem = fixed + (size_t)n_row * slot + per_warp_scalars;
      if (c.smem + 1024 > kSmemPerSm) continue;
      c.threads = g;
      c.ctas_per_sm = (int)(kSmemPerSm / (c.smem + 1024));
      if (c.ctas_per_sm > 2048 / g) c.ctas_per_sm = 2048 / g;
    }
    if (!found || c.warps_per_sm() > best.warps_per_sm()) best = c;
    found = true;
    if (c.warps_per_sm() >= 8) break;
  }
  return found;
}

}  // namespace

bool row_program_fits(int n_row_slots, int n_once_slots, int cols) {
  RowLaunch c;
  return row_launch_config(n_row_slots > 0 ? n_row_slots : 1, n_once_slots, cols, 0, c);
}

int launch_row_program(const RowProgram& prog, cudaStream_t s) {
  if (prog.rows == 0 || prog.cols == 0) return IB200_OK;
  if (prog.n_phases < 1 || prog.n_phases > kRowMaxPhases || prog.n_row_slots < 0 || prog.n_once_slots < 0 ||
      prog.n_row_slots + prog.n_once_slots > kRowMaxSlots || prog.n_scalars > kRowMaxScalars || prog.n_inputs > kRowMaxInputs ||
      prog.n_loads > kRowMaxLoads || prog.n_outputs > kRowMaxOutputs || prog.n_instr > kRowMaxInstr)
    return fail(IB200_ERR_INVALID, "row program: malformed program");
  for (int ph = 0; ph < prog.n_phases; ++ph)
    if (prog.phase[ph].domain == ROW_FULL && prog.phase[ph].n_outputs > kRowMaxSinks) return fail(IB200_ERR_INVALID, "row program: too many outputs in one phase");
  RowLaunch c;
  const int n_row = prog.n_row_slots > 0 ? prog.n_row_slots : 1;
  int full_instr = 0;  // micro-ops executed per element
  for (int ph = 0; ph < prog.n_phases; ++ph)
    if (prog.phase[ph].domain == ROW_FULL) full_instr += prog.phase[ph].n_instr;
  if (!row_launch_config(n_row, prog.n_once_slots, prog.cols, full_instr, c) && !row_launch_config(n_row, prog.n_once_slots, prog.cols, 0, c))
    return fail(IB200_ERR_UNSUPPORTED, "row program: rows of " + std::to_string(prog.cols) + " elements do not fit in shared memory");
  RowProgram p = prog;
  if (p.n_row_slots == 0) p.n_row_slots = 1;  // the layout always has one per-row slot
  void (*kern)(const RowProgram, const int) = nullptr;
#define IB200_ROW(GG)                                                                                                 \
  if (c.g == GG)                                                                                                      \
    kern = c.w == 1 ? row_kernel<GG, false, 8> : c.nu == 8 ? row_kernel<(GG < 512 ? GG : 128), true, 8> : c.nu == 4 ? row_kernel<GG, true, 4> : row_kernel<GG, true, 2>;
  IB200_ROW(32) IB200_ROW(128) IB200_ROW(512)
#undef IB200_ROW
  // a persistent grid: exactly as many CTAs as are resident at once, rows dealt round-robin
  static std::mutex mu;
  static std::map<std::tuple<const void*, size_t, int, int>, int> resident;
  int per_sm = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    int dev = 0;
    IB200_CUDA_OK(cudaGetDevice(&dev));
    const auto key = std::make_tuple(reinterpret_cast<const void*>(kern), c.smem, c.threads, dev);
    auto it = resident.find(key);
    if (it == resident.end()) {
      // opt in to the full shared memory once; the launch itself passes what this program needs
      IB200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemPerSm));
      int n = 0;
      IB200_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, c.threads, c.smem));
      it = resident.emplace(key, n > 0 ? n : 1).first;
    }
    per_sm = it->second;
  }
  const int groups = c.g <= 32 ? c.warps_per_cta : 1;
  const int64_t ctas = (p.rows + groups - 1) / groups;
  const int64_t cap = (int64_t)kSmCount * per_sm;
  kern<<<(int)(ctas < cap ? ctas : cap), c.threads, c.smem, s>>>(p, c.units);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "row program launch");
}

}  // namespace ib200

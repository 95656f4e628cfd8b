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

// ---- the kernel, in pieces shared by its two forms ---------------------------------------------------------
// A row program runs either decoded at run time (any program the planner emits) or compiled in: for the row
// programs that recur (the softmax of an attention, with its scale and mask; the benchmark's rms-norm) the very
// same phases are also template arguments, so that the loops over phases, micro-ops and outputs unroll into
// straight-line code on registers.  Decoding costs about 30 thread-instructions per element on a seven-op
// program; compiled in, the arithmetic and the loads and stores are what remains.  Staging, reductions, row
// scalars and stores are the same functions in both forms.

template <int G, bool VEC, int NU> struct RowCtx {
  static constexpr int kWarps = G <= 32 ? 1 : G / 32;
  SlotFile f;
  float* group_slots;  // this group's slots (two copies when nbuf == 2)
  float* scalars;      // [2][kRowMaxScalars], by row parity
  float* red;          // [2][kRowMaxSinks][kWarps], G > 32 only
  float* S;            // the current row's scalars
  int t, lane, cols, passes, nbuf, first_full;
  int64_t row, row_step;
  bool dirty;   // thread 0 has written row scalars since the group last synchronised
  bool staged;  // the first phase's operands of the current row are already on their way
  int red_parity, row_parity;
};

template <int G, bool VEC, int NU>
__device__ __forceinline__ void row_setup(RowCtx<G, VEC, NU>& c, const RowProgram& P, float* smem, int units, int nbuf) {
  constexpr int W = VEC ? 4 : 1;
  const int groups = G <= 32 ? (int)blockDim.x >> 5 : 1;
  const int g = G <= 32 ? (int)threadIdx.x >> 5 : 0;
  c.t = G <= 32 ? (int)threadIdx.x & 31 : (int)threadIdx.x;
  c.lane = threadIdx.x & 31;
  c.cols = P.cols;
  c.nbuf = nbuf;
  c.f.n_row = P.n_row_slots;
  c.f.slot_floats = units * G * W;
  c.f.shared = smem;
  // with nbuf == 2 a group holds two copies of its slots, used by alternate rows, so that the first
  // phase's operands of the next row travel while this row is computed
  c.group_slots = smem + (size_t)(P.n_once_slots + g * nbuf * P.n_row_slots) * c.f.slot_floats;
  c.f.group = c.group_slots;
  float* after_slots = smem + (size_t)(P.n_once_slots + groups * nbuf * P.n_row_slots) * c.f.slot_floats;
  // the group's row scalars, written by its thread 0 only and double-buffered by row parity so
  // that thread 0 may start on the next row while others still read this one's
  c.scalars = after_slots + g * (2 * kRowMaxScalars);
  c.red = after_slots + groups * (2 * kRowMaxScalars);
  c.passes = units / NU;

  // ---- row-invariant operands: once per CTA, by all its threads ------------------------------
  if (P.n_once_slots > 0) {
    bool convert = false;
    for (int k = 0; k < P.n_inputs; ++k) {
      const RowInput in = P.in[k];
      if (!in.once) continue;
      stage_columns<VEC>(in, c.f.base(in.slot), 0, threadIdx.x * W, blockDim.x * W, c.cols, convert);
    }
    cp_async_wait_all();
    if (VEC && convert)
      for (int k = 0; k < P.n_inputs; ++k) {
        const RowInput in = P.in[k];
        if (!in.once || !widens_in_place(in)) continue;
        float* base = c.f.base(in.slot);
        for (int col = threadIdx.x * W; col < c.cols; col += blockDim.x * W) widen_unit(in, base + col);
      }
    __syncthreads();
  }
  c.first_full = 0;  // the phase whose operands are fetched a row ahead
  while (c.first_full < P.n_phases && P.phase[c.first_full].domain != ROW_FULL) ++c.first_full;
  c.dirty = false;
  c.staged = false;
  c.red_parity = 0;
  c.row_parity = 0;
  c.row_step = (int64_t)gridDim.x * groups;
  c.row = (int64_t)blockIdx.x * groups + g;
}

template <int G, bool VEC, int NU> __device__ __forceinline__ void row_begin(RowCtx<G, VEC, NU>& c, const RowProgram& P) {
  c.S = c.scalars + c.row_parity * kRowMaxScalars;
  if (c.nbuf == 2) c.f.group = c.group_slots + (size_t)c.row_parity * P.n_row_slots * c.f.slot_floats;
}

// what every phase starts with: the row scalars it reads from global memory
template <int G, bool VEC, int NU> __device__ __forceinline__ void phase_loads(RowCtx<G, VEC, NU>& c, const RowProgram& P, const RowPhase& phase) {
  if (phase.n_loads && c.t == 0) {
    for (int k = 0; k < phase.n_loads; ++k) {
      const RowScalarLoad ld = P.load[phase.first_load + k];
      c.S[ld.scalar] = load_scalar(ld.ptr, ld.dtype, c.row * ld.row_stride);
    }
  }
  c.dirty |= phase.n_loads != 0;
}

// a FULL phase's global operands into their slots (those of the first FULL phase one row ahead, when the
// group has two copies of its slots); returns when this row's are in shared memory and widened
template <int G, bool VEC, int NU>
__device__ __forceinline__ void phase_stage(RowCtx<G, VEC, NU>& c, const RowProgram& P, const RowPhase& phase, int ph) {
  constexpr int W = VEC ? 4 : 1;
  bool convert = false, unused = false;
  for (int k = 0; k < phase.n_inputs; ++k) convert |= !P.in[phase.first_input + k].once && widens_in_place(P.in[phase.first_input + k]);
  if (!(c.staged && ph == c.first_full)) {
    for (int k = 0; k < phase.n_inputs; ++k) {
      const RowInput in = P.in[phase.first_input + k];
      if (in.once) continue;
      stage_columns<VEC>(in, c.f.base(in.slot), c.row * in.row_stride, c.t * W, G * W, c.cols, unused);
    }
    cp_async_commit();
  }
  bool ahead = false;
  if (c.nbuf == 2 && ph == c.first_full && c.row + c.row_step < P.rows) {  // the next row's operands, into the other copy
    SlotFile nf = c.f;
    nf.group = c.group_slots + (size_t)(c.row_parity ^ 1) * P.n_row_slots * c.f.slot_floats;
    for (int k = 0; k < phase.n_inputs; ++k) {
      const RowInput in = P.in[phase.first_input + k];
      if (in.once) continue;
      stage_columns<VEC>(in, nf.base(in.slot), (c.row + c.row_step) * in.row_stride, c.t * W, G * W, c.cols, unused);
    }
    cp_async_commit();
    ahead = true;
  }
  if (ph == c.first_full) c.staged = ahead;
  if (c.dirty) {  // row scalars written by thread 0 become visible to the group
    group_sync<G>();
    c.dirty = false;
  }
  if (ahead) cp_async_wait_but_one();
  else cp_async_wait_committed();
  if (VEC && convert) {
    for (int k = 0; k < phase.n_inputs; ++k) {
      const RowInput in = P.in[phase.first_input + k];
      if (in.once || !widens_in_place(in)) continue;
      float* base = c.f.base(in.slot);
      for (int col = c.t * W; col < c.cols; col += G * W) widen_unit(in, base + col);
    }
  }
}

// one output of a FULL phase for one pass: folded into the running partial, or stored
template <int G, bool VEC, int NU, int N>
__device__ __forceinline__ void phase_sink(const RowCtx<G, VEC, NU>& c, const RowOutput& out, uint8_t src, uint8_t reduce, const float (&acc)[N],
                                           float& part, int pass, int col0, bool whole) {
  float v[N];
  fetch<G, VEC, NU, N>(v, src, acc, 0.0f, c.f, c.S, pass, c.t);
  const int cols = c.cols;
  if (reduce) {
    const int kind = reduce - 1;
    if (!whole) {  // values past the end of the row become the identity
      const float id = reduce_identity(kind);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const int col = VEC ? col0 + (j >> 2) * G * 4 + (j & 3) : col0 + j * G;
        if (col >= cols) v[j] = id;
      }
    }
    part = fold<N>(kind, part, v);
  } else if (out.ptr) {
    const int64_t base = c.row * out.row_stride;
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

// warp-level fold of one reducing output's partial; G <= 32 finishes here, wider groups leave one value per warp
template <int G, bool VEC, int NU>
__device__ __forceinline__ void sink_reduce_warp(const RowCtx<G, VEC, NU>& c, const RowOutput& out, uint8_t reduce, float v, float* slots, int o) {
  constexpr int kWarps = RowCtx<G, VEC, NU>::kWarps;
  const int kind = reduce - 1;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = reduce_apply(kind, v, __shfl_xor_sync(0xffffffffu, v, d));
  if (G <= 32) {
    if (c.t == 0) {
      v *= out.scale;
      c.S[out.scalar] = v;
      if (out.ptr) store_scalar(out.ptr, out.dtype, c.row * out.row_stride, v);
    }
  } else if (c.lane == 0) {
    slots[o * kWarps + (c.t >> 5)] = v;
  }
}
// G > 32, thread 0, after the barrier: the warps' values in a fixed order, so that the result does not depend on
// which warp finished first
template <int G, bool VEC, int NU>
__device__ __forceinline__ void sink_reduce_block(const RowCtx<G, VEC, NU>& c, const RowOutput& out, uint8_t reduce, const float* slots, int o) {
  constexpr int kWarps = RowCtx<G, VEC, NU>::kWarps;
  const int kind = reduce - 1;
  float v = slots[o * kWarps];
  for (int w = 1; w < kWarps; ++w) v = reduce_apply(kind, v, slots[o * kWarps + w]);
  v *= out.scale;
  c.S[out.scalar] = v;
  if (out.ptr) store_scalar(out.ptr, out.dtype, c.row * out.row_stride, v);
}

// ---- decoded at run time -----------------------------------------------------------------------------------
template <int G, bool VEC, int NU>
__device__ __forceinline__ void interp_row(RowCtx<G, VEC, NU>& c, const RowProgram& P) {
  constexpr int W = VEC ? 4 : 1;
  constexpr int N = NU * W;
  constexpr int kWarps = RowCtx<G, VEC, NU>::kWarps;
  const int t = c.t, cols = c.cols;
  float* const S = c.S;
  for (int ph = 0; ph < P.n_phases; ++ph) {
    const RowPhase phase = P.phase[ph];
    phase_loads(c, P, phase);
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
          if (out.ptr) store_scalar(out.ptr, out.dtype, c.row * out.row_stride, v);
        }
      }
      c.dirty = true;
      continue;
    }
    phase_stage(c, P, phase, ph);

    // ---- run the chain, pass by pass -----------------------------------------------------
    float part[kRowMaxSinks];
    bool any_reduce = false;
#pragma unroll
    for (int o = 0; o < kRowMaxSinks; ++o) {
      const bool live = o < phase.n_outputs && P.out[phase.first_output + o].reduce;
      part[o] = live ? reduce_identity(P.out[phase.first_output + o].reduce - 1) : 0.0f;
      any_reduce |= live;
    }
    for (int pass = 0; pass < c.passes; ++pass) {
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
          float a[N], b[N], cc[N];
          fetch<G, VEC, NU, N>(a, ins.a, acc, ins.imm, c.f, S, pass, t);
          fetch<G, VEC, NU, N>(b, ins.b, acc, ins.imm, c.f, S, pass, t);
          fetch<G, VEC, NU, N>(cc, ins.c, acc, ins.imm, c.f, S, pass, t);
#pragma unroll
          for (int j = 0; j < N; ++j) acc[j] = a[j] != 0.0f ? b[j] : cc[j];
        } else if (ins.b == EW_ACC) {
          apply<N>(ins.op, acc, acc, acc);
        } else if (ins.b < kRowMaxSlots) {
          float b[N];
          fetch<G, VEC, NU, N>(b, ins.b, acc, ins.imm, c.f, S, pass, t);
          apply<N>(ins.op, acc, b, acc);
        } else {
          apply_scalar<N>(ins.op, acc, ins.b == EW_IMM ? ins.imm : S[ins.b - EW_ROWSCALAR]);
        }
        if (ins.dst != EW_NODST) put<G, VEC, NU, N>(acc, ins.dst, c.f, pass, t);
      }
#pragma unroll
      for (int o = 0; o < kRowMaxSinks; ++o) {
        if (o >= phase.n_outputs) break;
        const RowOutput out = P.out[phase.first_output + o];
        phase_sink<G, VEC, NU, N>(c, out, out.src, out.reduce, acc, part[o], pass, col0, whole);
      }
    }

    // ---- fold the partials into row scalars ----------------------------------------------------
    if (any_reduce) {
      float* slots = c.red + c.red_parity * (kRowMaxSinks * kWarps);
#pragma unroll
      for (int o = 0; o < kRowMaxSinks; ++o) {
        if (o >= phase.n_outputs) break;
        const RowOutput out = P.out[phase.first_output + o];
        if (out.reduce) sink_reduce_warp(c, out, out.reduce, part[o], slots, o);
      }
      if (G > 32) {
        __syncthreads();
        if (t == 0)
          for (int o = 0; o < phase.n_outputs; ++o) {
            const RowOutput out = P.out[phase.first_output + o];
            if (out.reduce) sink_reduce_block(c, out, out.reduce, slots, o);
          }
        c.red_parity ^= 1;
      }
      c.dirty = true;
    }
  }
}

template <int G, bool VEC, int NU>
__global__ void __launch_bounds__(G <= 32 ? 256 : G) row_kernel(const __grid_constant__ RowProgram P, const int units, const int nbuf) {
  extern __shared__ __align__(16) float smem[];
  RowCtx<G, VEC, NU> c;
  row_setup(c, P, smem, units, nbuf);
  for (; c.row < P.rows; c.row += c.row_step, c.row_parity ^= 1) {
    row_begin(c, P);
    interp_row(c, P);
  }
}

// ---- compiled in -------------------------------------------------------------------------------------------
// A static program repeats, as constants, what the planner writes into RowProgram for one shape of graph: the
// phases, the micro-ops (opcode and operand codes) and where each phase's results go.  Pointers, strides, types,
// immediates, scales and the operands to stage are still read from the RowProgram of the launch.
struct RowStaticIns {
  uint8_t op, a, b, c, dst;
};
struct RowStaticOut {
  uint8_t src, reduce, scalar, stored;
};
struct RowStaticPhase {
  uint8_t domain, first_instr, n_instr, first_output, n_outputs;
};

template <class SP, int I, int END, int G, int NU, int N>
__device__ __forceinline__ void static_chain(float (&acc)[N], const RowCtx<G, true, NU>& c, const RowProgram& P, int pass) {
  if constexpr (I < END) {
    constexpr RowStaticIns ins = SP::ins[I];
    const float imm = P.instr[I].imm;
    if constexpr (ins.op == EW_WHERE) {
      float a[N], b[N], cc[N];
      fetch<G, true, NU, N>(a, ins.a, acc, imm, c.f, c.S, pass, c.t);
      fetch<G, true, NU, N>(b, ins.b, acc, imm, c.f, c.S, pass, c.t);
      fetch<G, true, NU, N>(cc, ins.c, acc, imm, c.f, c.S, pass, c.t);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = a[j] != 0.0f ? b[j] : cc[j];
    } else if constexpr (ins.b == EW_ACC) {
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = static_op<ins.op>(acc[j], acc[j]);
    } else if constexpr (ins.b < kRowMaxSlots) {
      float b[N];
      fetch<G, true, NU, N>(b, ins.b, acc, imm, c.f, c.S, pass, c.t);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = static_op<ins.op>(acc[j], b[j]);
    } else {
      const float y = ins.b == EW_IMM ? imm : c.S[ins.b - EW_ROWSCALAR];
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = static_op<ins.op>(acc[j], y);
    }
    if constexpr (ins.dst != EW_NODST) put<G, true, NU, N>(acc, ins.dst, c.f, pass, c.t);
    static_chain<SP, I + 1, END, G, NU, N>(acc, c, P, pass);
  }
}

template <class SP, int O, int END, int G, int NU, int N>
__device__ __forceinline__ void static_sinks(const RowCtx<G, true, NU>& c, const RowProgram& P, const float (&acc)[N], float (&part)[kRowMaxSinks],
                                             int first, int pass, int col0, bool whole) {
  if constexpr (O < END) {
    constexpr RowStaticOut so = SP::out[O];
    phase_sink<G, true, NU, N>(c, P.out[O], so.src, so.reduce, acc, part[O - first], pass, col0, whole);
    static_sinks<SP, O + 1, END, G, NU, N>(c, P, acc, part, first, pass, col0, whole);
  }
}
template <class SP, int O, int END, int G, int NU>
__device__ __forceinline__ void static_reduce_warp(const RowCtx<G, true, NU>& c, const RowProgram& P, const float (&part)[kRowMaxSinks], float* slots, int first) {
  if constexpr (O < END) {
    constexpr RowStaticOut so = SP::out[O];
    if constexpr (so.reduce != 0) sink_reduce_warp(c, P.out[O], so.reduce, part[O - first], slots, O - first);
    static_reduce_warp<SP, O + 1, END, G, NU>(c, P, part, slots, first);
  }
}
template <class SP, int O, int END, int G, int NU>
__device__ __forceinline__ void static_reduce_block(const RowCtx<G, true, NU>& c, const RowProgram& P, const float* slots, int first) {
  if constexpr (O < END) {
    constexpr RowStaticOut so = SP::out[O];
    if constexpr (so.reduce != 0) sink_reduce_block(c, P.out[O], so.reduce, slots, O - first);
    static_reduce_block<SP, O + 1, END, G, NU>(c, P, slots, first);
  }
}
template <class SP, int O, int END> __device__ __forceinline__ void static_part_init(float (&part)[kRowMaxSinks], int first) {
  if constexpr (O < END) {
    constexpr RowStaticOut so = SP::out[O];
    if constexpr (so.reduce != 0) part[O - first] = reduce_identity(so.reduce - 1);
    static_part_init<SP, O + 1, END>(part, first);
  }
}
template <class SP, int O, int END> __host__ __device__ constexpr bool static_any_reduce() {
  if constexpr (O < END) return SP::out[O].reduce != 0 || static_any_reduce<SP, O + 1, END>();
  else return false;
}

template <class SP, int I, int END> __device__ __forceinline__ void static_scalar_chain(float& acc, float* S, const RowProgram& P) {
  if constexpr (I < END) {
    constexpr RowStaticIns ins = SP::ins[I];
    const float imm = P.instr[I].imm;
    const float a = scalar_operand(ins.a, acc, imm, S), b = scalar_operand(ins.b, acc, imm, S);
    if constexpr (ins.op == EW_WHERE) acc = a != 0.0f ? b : scalar_operand(ins.c, acc, imm, S);
    else acc = static_op<ins.op>(a, b);
    if constexpr (ins.dst != EW_NODST) S[ins.dst - EW_ROWSCALAR] = acc;
    static_scalar_chain<SP, I + 1, END>(acc, S, P);
  }
}
template <class SP, int O, int END, int G, int NU>
__device__ __forceinline__ void static_scalar_outputs(const RowCtx<G, true, NU>& c, const RowProgram& P, float acc) {
  if constexpr (O < END) {
    constexpr RowStaticOut so = SP::out[O];
    const RowOutput out = P.out[O];
    const float v = scalar_operand(so.src, acc, 0.0f, c.S);
    if constexpr (so.scalar != kRowNone) c.S[so.scalar] = v;
    if (out.ptr) store_scalar(out.ptr, out.dtype, c.row * out.row_stride, v);
    static_scalar_outputs<SP, O + 1, END, G, NU>(c, P, acc);
  }
}

template <class SP, int PH, int G, int NU> __device__ __forceinline__ void static_row(RowCtx<G, true, NU>& c, const RowProgram& P) {
  if constexpr (PH < SP::n_phases) {
    constexpr RowStaticPhase sp = SP::phase[PH];
    constexpr int N = NU * 4;
    constexpr int kWarps = RowCtx<G, true, NU>::kWarps;
    const RowPhase phase = P.phase[PH];
    phase_loads(c, P, phase);
    if constexpr (sp.domain == ROW_SCALAR) {
      if (c.t == 0) {
        float acc = 0.0f;
        static_scalar_chain<SP, sp.first_instr, sp.first_instr + sp.n_instr>(acc, c.S, P);
        static_scalar_outputs<SP, sp.first_output, sp.first_output + sp.n_outputs, G, NU>(c, P, acc);
      }
      c.dirty = true;
    } else {
      phase_stage(c, P, phase, PH);
      float part[kRowMaxSinks] = {};
      static_part_init<SP, sp.first_output, sp.first_output + sp.n_outputs>(part, sp.first_output);
      for (int pass = 0; pass < c.passes; ++pass) {
        const int col0 = (pass * NU * G + c.t) * 4;
        if (col0 >= c.cols) break;
        const bool whole = col0 + (NU - 1) * G * 4 + 3 < c.cols;
        float acc[N];
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = 0.0f;
        static_chain<SP, sp.first_instr, sp.first_instr + sp.n_instr, G, NU, N>(acc, c, P, pass);
        static_sinks<SP, sp.first_output, sp.first_output + sp.n_outputs, G, NU, N>(c, P, acc, part, sp.first_output, pass, col0, whole);
      }
      if constexpr (static_any_reduce<SP, sp.first_output, sp.first_output + sp.n_outputs>()) {
        float* slots = c.red + c.red_parity * (kRowMaxSinks * kWarps);
        static_reduce_warp<SP, sp.first_output, sp.first_output + sp.n_outputs, G, NU>(c, P, part, slots, sp.first_output);
        if (G > 32) {
          __syncthreads();
          if (c.t == 0) static_reduce_block<SP, sp.first_output, sp.first_output + sp.n_outputs, G, NU>(c, P, slots, sp.first_output);
          c.red_parity ^= 1;
        }
        c.dirty = true;
      }
    }
    static_row<SP, PH + 1, G, NU>(c, P);
  }
}

template <class SP, int G, int NU>
__global__ void __launch_bounds__(G <= 32 ? 256 : G) row_kernel_static(const __grid_constant__ RowProgram P, const int units, const int nbuf) {
  extern __shared__ __align__(16) float smem[];
  RowCtx<G, true, NU> c;
  row_setup(c, P, smem, units, nbuf);
  for (; c.row < P.rows; c.row += c.row_step, c.row_parity ^= 1) {
    row_begin(c, P);
    static_row<SP, 0, G, NU>(c, P);
  }
}

// ---- the programs compiled in ------------------------------------------------------------------------------
// Each table is what the planner emits for the named graph shape (plan descriptions show the same numbers);
// a launch whose program differs in any micro-op, operand or sink runs decoded.  Operand codes: 0..15 slot,
// 64 + k row scalar k, 128 the running value, 129 the immediate; sinks: {source, reduction + 1, row scalar, -}.
constexpr uint8_t kAcc = EW_ACC, kImm = EW_IMM, kNo = EW_NODST, kS0 = EW_ROWSCALAR, kS1 = EW_ROWSCALAR + 1, kS2 = EW_ROWSCALAR + 2;
constexpr uint8_t kSum = IB200_REDUCE_SUM + 1, kMax = IB200_REDUCE_MAX + 1;

// softmax(scores + bias) * ... of an attention: (q.k + mask) * scale, row maximum, exp and row sum, division
struct RowProgAttnBiasScaleSoftmax {
  static constexpr int n_phases = 4, n_instr = 8, n_outputs = 3;
  static constexpr RowStaticPhase phase[4] = {{ROW_FULL, 0, 3, 0, 0}, {ROW_FULL, 3, 0, 0, 1}, {ROW_FULL, 3, 3, 1, 1}, {ROW_FULL, 6, 2, 2, 1}};
  static constexpr RowStaticIns ins[8] = {{EW_LOADB, kAcc, 0, kAcc, kNo}, {EW_ADD, kAcc, 1, kAcc, kNo}, {EW_MUL, kAcc, kS0, kAcc, 2},
                                          {EW_LOADB, kAcc, 2, kAcc, kNo}, {EW_SUB, kAcc, kS1, kAcc, kNo}, {EW_EXP, kAcc, kAcc, kAcc, 0},
                                          {EW_LOADB, kAcc, 0, kAcc, kNo}, {EW_DIV, kAcc, kS2, kAcc, kNo}};
  static constexpr RowStaticOut out[3] = {{2, kMax, 1, 0}, {kAcc, kSum, 2, 0}, {kAcc, 0, kRowNone, 1}};
};
// the causal form: scores * scale where the key index does not exceed the query index, a fill value elsewhere
struct RowProgAttnScaleCausalSoftmax {
  static constexpr int n_phases = 4, n_instr = 10, n_outputs = 3;
  static constexpr RowStaticPhase phase[4] = {{ROW_FULL, 0, 5, 0, 0}, {ROW_FULL, 5, 0, 0, 1}, {ROW_FULL, 5, 3, 1, 1}, {ROW_FULL, 8, 2, 2, 1}};
  static constexpr RowStaticIns ins[10] = {{EW_LOADB, kAcc, 2, kAcc, kNo}, {EW_MUL, kAcc, kS0, kAcc, 3}, {EW_LOADB, kAcc, 0, kAcc, kNo},
                                           {EW_LE, kAcc, 1, kAcc, kNo}, {EW_WHERE, kAcc, 3, kImm, 4},
                                           {EW_LOADB, kAcc, 4, kAcc, kNo}, {EW_SUB, kAcc, kS1, kAcc, kNo}, {EW_EXP, kAcc, kAcc, kAcc, 0},
                                           {EW_LOADB, kAcc, 0, kAcc, kNo}, {EW_DIV, kAcc, kS2, kAcc, kNo}};
  static constexpr RowStaticOut out[3] = {{4, kMax, 1, 0}, {kAcc, kSum, 2, 0}, {kAcc, 0, kRowNone, 1}};
};
// rms-norm with |x| between the normalisation and the weight (the benchmark's row program); rstd is an output
struct RowProgRmsAbsWeight {
  static constexpr int n_phases = 4, n_instr = 8, n_outputs = 4;
  static constexpr RowStaticPhase phase[4] = {{ROW_FULL, 0, 2, 0, 1}, {ROW_SCALAR, 2, 2, 1, 1}, {ROW_FULL, 4, 4, 2, 1}, {ROW_SCALAR, 8, 0, 3, 1}};
  static constexpr RowStaticIns ins[8] = {{EW_LOADB, kAcc, 0, kAcc, kNo}, {EW_MUL, kAcc, 0, kAcc, kNo},
                                          {EW_ADD, kS0, kImm, kS0, kNo}, {EW_RSQRT, kAcc, kAcc, kAcc, kNo},
                                          {EW_LOADB, kAcc, 0, kAcc, kNo}, {EW_MUL, kAcc, kS1, kAcc, kNo}, {EW_ABS, kAcc, kAcc, kAcc, kNo},
                                          {EW_MUL, kAcc, 1, kAcc, kNo}};
  static constexpr RowStaticOut out[4] = {{kAcc, kSum, 0, 0}, {kAcc, 0, 1, 0}, {kAcc, 0, kRowNone, 1}, {kS1, 0, kRowNone, 1}};
};

template <class SP> bool static_matches(const RowProgram& p) {
  if (p.n_phases != SP::n_phases || p.n_instr != SP::n_instr || p.n_outputs != SP::n_outputs) return false;
  for (int i = 0; i < SP::n_phases; ++i) {
    const RowPhase& a = p.phase[i];
    const RowStaticPhase& b = SP::phase[i];
    if (a.domain != b.domain || a.first_instr != b.first_instr || a.n_instr != b.n_instr || a.first_output != b.first_output || a.n_outputs != b.n_outputs)
      return false;
  }
  for (int i = 0; i < SP::n_instr; ++i) {
    const EwInstr& a = p.instr[i];
    const RowStaticIns& b = SP::ins[i];
    if (a.op != b.op || a.a != b.a || a.b != b.b || a.c != b.c || a.dst != b.dst) return false;
  }
  for (int i = 0; i < SP::n_outputs; ++i) {
    const RowOutput& a = p.out[i];
    const RowStaticOut& b = SP::out[i];
    if (a.src != b.src || a.reduce != b.reduce || a.scalar != b.scalar) return false;
  }
  return true;
}

using RowKernel = void (*)(const RowProgram, const int, const int);
template <class SP> RowKernel static_kernel(int g, int nu) {
  if (g == 32) return nu == 8 ? row_kernel_static<SP, 32, 8> : nu == 4 ? row_kernel_static<SP, 32, 4> : row_kernel_static<SP, 32, 2>;
  if (g == 128) return nu == 8 ? row_kernel_static<SP, 128, 8> : nu == 4 ? row_kernel_static<SP, 128, 4> : row_kernel_static<SP, 128, 2>;
  return nu == 4 ? row_kernel_static<SP, 512, 4> : nu == 2 ? row_kernel_static<SP, 512, 2> : nullptr;
}
// the compiled-in kernel for this program and launch shape, or null (vector form only: row length a multiple of 4)
RowKernel find_static(const RowProgram& p, int g, int w, int nu) {
  if (w != 4) return nullptr;
#ifdef IB200_AB_KNOBS  // A/B builds only: IB200_ROW_STATIC=0 keeps every program on the decoder
  static const bool off = std::getenv("IB200_ROW_STATIC") && std::getenv("IB200_ROW_STATIC")[0] == '0';
  if (off) return nullptr;
#endif
  if (static_matches<RowProgAttnBiasScaleSoftmax>(p)) return static_kernel<RowProgAttnBiasScaleSoftmax>(g, nu);
  if (static_matches<RowProgAttnScaleCausalSoftmax>(p)) return static_kernel<RowProgAttnScaleCausalSoftmax>(g, nu);
  if (static_matches<RowProgRmsAbsWeight>(p)) return static_kernel<RowProgRmsAbsWeight>(g, nu);
  return nullptr;
}

struct RowLaunch {
  int g = 0, w = 1, nu = 8, units = 0, warps_per_cta = 1, threads = 32, ctas_per_sm = 1, nbuf = 1;
  size_t smem = 0;
  int warps_per_sm() const { return ctas_per_sm * (g <= 32 ? warps_per_cta : g / 32); }
};

constexpr size_t kSmemPerSm = 227 * 1024;

bool single_buffered() {
#ifdef IB200_AB_KNOBS  // A/B builds only: IB200_ROW_NBUF=1 keeps one copy of the slots
  static const bool one = std::getenv("IB200_ROW_NBUF") && std::atoi(std::getenv("IB200_ROW_NBUF")) == 1;
  return one;
#else
  return false;
#endif
}

// the launch shape for a program with `n_row` per-row and `n_once` row-invariant slots: the
// smallest group that still leaves at least eight warps resident per SM, else the most warps
bool row_launch_config(int n_row_slots, int n_once, int cols, int n_instr, int nbuf, RowLaunch& best) {
  bool found = false;
  const int n_row = n_row_slots * nbuf;
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
    c.nbuf = nbuf;
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

bool row_program_compiled_in(const RowProgram& prog) {
  return prog.cols % 4 == 0 && (static_matches<RowProgAttnBiasScaleSoftmax>(prog) || static_matches<RowProgAttnScaleCausalSoftmax>(prog) ||
                                static_matches<RowProgRmsAbsWeight>(prog));
}

bool row_program_fits(int n_row_slots, int n_once_slots, int cols) {
  RowLaunch c;
  return row_launch_config(n_row_slots > 0 ? n_row_slots : 1, n_once_slots, cols, 0, 1, c);
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
  // A compiled-in program has nothing to decode: 16 values per thread and pass, and a second copy of the slots only
  // where it costs no resident CTA (rms with |x| over [8192,4096]: 49.4 us with 32 values and two copies at four CTAs
  // per SM, 47.1 us with 16 values and one copy at six)
  const bool compiled_in = row_program_compiled_in(prog);
  if (compiled_in) full_instr = 0;
  if (!row_launch_config(n_row, prog.n_once_slots, prog.cols, full_instr, 1, c) && !row_launch_config(n_row, prog.n_once_slots, prog.cols, 0, 1, c))
    return fail(IB200_ERR_UNSUPPORTED, "row program: rows of " + std::to_string(prog.cols) + " elements do not fit in shared memory");
  // Two copies of the slots (the next row's operands travel during this row's arithmetic) whenever a
  // group works on several rows and the copies cost at most half of the resident warps.
  {
    RowLaunch d;
    const int64_t row_groups = (int64_t)kSmCount * c.warps_per_sm() / (c.g <= 32 ? 1 : c.g / 32);
    if (prog.rows > row_groups && row_launch_config(n_row, prog.n_once_slots, prog.cols, full_instr, 2, d) && d.g == c.g && d.nu == c.nu &&
        (compiled_in ? d.warps_per_sm() >= c.warps_per_sm() : 2 * d.warps_per_sm() >= c.warps_per_sm()) && !single_buffered())
      c = d;
  }
  RowProgram p = prog;
  if (p.n_row_slots == 0) p.n_row_slots = 1;  // the layout always has one per-row slot
  RowKernel kern = nullptr;
#define IB200_ROW(GG)                                                                                                 \
  if (c.g == GG)                                                                                                      \
    kern = c.w == 1 ? row_kernel<GG, false, 8> : c.nu == 8 ? row_kernel<(GG < 512 ? GG : 128), true, 8> : c.nu == 4 ? row_kernel<GG, true, 4> : row_kernel<GG, true, 2>;
  IB200_ROW(32) IB200_ROW(128) IB200_ROW(512)
#undef IB200_ROW
  if (RowKernel compiled = find_static(p, c.g, c.w, c.nu)) kern = compiled;
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
  kern<<<(int)(ctas < cap ? ctas : cap), c.threads, c.smem, s>>>(p, c.units, c.nbuf);
  return cudaPeekAtLastError() == cudaSuccess ? IB200_OK : cuda_fail(cudaGetLastError(), "row program launch");
}

}  // namespace ib200

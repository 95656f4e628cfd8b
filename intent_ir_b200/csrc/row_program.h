// A fused "row program": several steps of a plan that all work on the same [rows, cols]
// problem -- elementwise chains over the full tensor, reductions along the row, small
// computations on the per-row results, softmax -- executed by ONE kernel in which a group of
// threads owns a row from the first load to the last store.  Intermediates that the unfused
// plan would write to and read back from HBM (x*x before a row sum, the masked scores before
// a softmax, the residual sum before a normalisation) stay in shared memory or never exist.
//
// The program is a list of phases executed in order for every row:
//   FULL phase    an EwProgram-style chain over the row's `cols` elements.  Operands are row
//                 slots (shared memory, one row-long vector each), row scalars, immediates and
//                 the accumulator; results go to global memory, stay in a slot for a later
//                 phase, and / or are reduced along the row into a row scalar.
//   SCALAR phase  a chain over row scalars only (mean, variance, rstd ...), run by one thread.
// The reference has no counterpart: its generated kernels are one per op pattern
// (backends/cuda/codegen/intentir_to_cuda.py) and its interpreter materialises every op.
#pragma once
#include <stdint.h>

#include "ew_program.h"

namespace ib200 {

constexpr int kRowMaxPhases = 12;
constexpr int kRowMaxInputs = 24;
constexpr int kRowMaxLoads = 16;
constexpr int kRowMaxOutputs = 16;
constexpr int kRowMaxInstr = 128;
constexpr int kRowMaxSlots = 16;
constexpr int kRowMaxScalars = 32;
constexpr int kRowMaxSinks = 4;  // outputs of one phase

// operand codes on top of ew_program.h's: EW_ROWSCALAR + k names row scalar k
constexpr uint8_t EW_ROWSCALAR = 0x40;
constexpr uint8_t kRowNone = 0xFF;

enum RowDomain : uint8_t { ROW_FULL = 0, ROW_SCALAR = 1 };

struct RowInput {  // a global operand staged into a slot at the start of a FULL phase
  const void* ptr;
  int64_t row_stride;  // elements between consecutive rows (0: the same vector for every row)
  int32_t col_stride;  // elements between consecutive columns
  int32_t dtype;
  uint8_t kind;    // EwInputKind
  uint8_t slot;
  uint8_t once;    // row-invariant: staged once per CTA, before the first row, into a slot all its warps read
  uint8_t vec_ok;  // filled at launch: unit column stride, aligned base, row stride % 4 == 0
  int32_t pad;
};

struct RowScalarLoad {  // S[scalar] = ptr[row * row_stride]
  const void* ptr;
  int64_t row_stride;
  int32_t dtype;
  int32_t scalar;
};

struct RowOutput {
  void* ptr;           // global destination, or null when the value only feeds later phases
  int64_t row_stride;  // elements between consecutive rows of the destination
  int32_t dtype;
  uint8_t src;         // slot, EW_ROWSCALAR + k, or EW_ACC (the phase's last result)
  uint8_t reduce;      // 0, or IB200_REDUCE_* + 1: fold the row into row scalar `scalar`
  uint8_t scalar;      // FULL: destination of the reduction; SCALAR: where the value is kept (kRowNone: nowhere)
  uint8_t vec_ok;      // filled at launch
  float scale;         // reductions: result multiplied by this
  int32_t pad;
};

struct RowPhase {
  uint8_t domain, n_inputs, n_loads, n_outputs;
  uint16_t first_input, first_load, first_output, first_instr, n_instr, pad;
};

struct RowProgram {
  int64_t rows;
  int32_t cols;
  int32_t n_phases, n_scalars;
  int32_t n_row_slots, n_once_slots;  // slots 0 .. n_row_slots-1 are per row, the rest row-invariant (one copy per CTA)
  int32_t n_inputs, n_loads, n_outputs, n_instr;
  RowPhase phase[kRowMaxPhases];
  RowInput in[kRowMaxInputs];
  RowScalarLoad load[kRowMaxLoads];
  RowOutput out[kRowMaxOutputs];
  EwInstr instr[kRowMaxInstr];
};

// whether some launch shape holds that many slots of `cols` elements in shared memory
bool row_program_fits(int n_row_slots, int n_once_slots, int cols);

int launch_row_program(const RowProgram& prog, cudaStream_t s);

// whether the program is one of those whose phases are also compiled into the kernel as straight-line code
// (the same arithmetic, without the decoding); any other program runs decoded
bool row_program_compiled_in(const RowProgram& prog);

}  // namespace ib200

// The micro-op program a fused elementwise/broadcast chain is lowered to.  The planner
// (host) fills one EwProgram per fused group; elementwise.cu executes it in a single pass
// over the output: every external operand is read once, every intermediate lives in
// on-chip storage, every result is written once.
//
// Execution model: each thread owns 8 output elements.  Values live in "slots" (a register
// file kept in shared memory, one column per thread) or in the accumulator ACC (real
// registers holding the previous instruction's result), so a linear chain
// x -> op -> op -> ... -> y never touches the slot file after its operands are loaded.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace ib200 {

constexpr int kEwMaxInputs = 8;
constexpr int kEwMaxOutputs = 4;
constexpr int kEwMaxInstr = 64;
constexpr int kEwMaxRank = 5;
constexpr int kEwMaxSlots = 16;  // inputs occupy the first n_inputs slots

enum EwOp : uint8_t {
  EW_MOV = 0,  // acc = a
  EW_ADD, EW_SUB, EW_MUL, EW_DIV, EW_MAX, EW_MIN,            // numpy semantics: max/min propagate NaN
  EW_RELU, EW_EXP, EW_RSQRT, EW_ABS, EW_FLOOR,               // rsqrt = 1/sqrt(x), both IEEE-rounded
  EW_NE, EW_LT, EW_LE, EW_GT, EW_GE,                         // results are 1.0 / 0.0
  EW_AND, EW_OR, EW_NOT,                                     // operands are "!= 0"
  EW_WHERE,                                                  // acc = (a != 0) ? b : c
  EW_TO_BOOL, EW_TO_INT, EW_ROUND_BF16, EW_ROUND_F16,        // casts (to f32 is EW_MOV)
  EW_RSUB, EW_RDIV, EW_LOADB,                                // b - a, b / a, acc = b (register-path forms)
  EW_NUM_OPS
};

// operand codes: 0..kEwMaxSlots-1 = slot, EW_ACC = previous result, EW_IMM = instr.imm
constexpr uint8_t EW_ACC = 0x80;
constexpr uint8_t EW_IMM = 0x81;
constexpr uint8_t EW_NODST = 0xFF;

struct EwInstr {
  uint8_t op, a, b, c;
  uint8_t dst;  // slot to also store the result into, or EW_NODST
  uint8_t pad[3];
  float imm;
};

enum EwInputKind : int32_t {
  EW_IN_TENSOR = 0,  // value = ptr[offset]
  EW_IN_IOTA = 1,    // value = offset  (strides form a one-hot ramp along the iota axis)
};

enum EwStageMode : int32_t {  // how an operand reaches the slot file
  EW_STAGE_NONE = 0,
  EW_STAGE_ASYNC_F32X4,  // cp.async 16 bytes (4 contiguous f32)
  EW_STAGE_ASYNC_HALF4,  // cp.async 8 bytes (4 contiguous bf16 / f16), widened in place afterwards
  EW_STAGE_ASYNC_F32,    // cp.async 4 bytes (scalar mode)
  EW_STAGE_BROADCAST,    // one scalar load, replicated (inner stride 0)
  EW_STAGE_GATHER,       // scalar loads with the inner stride
  EW_STAGE_IOTA,         // value = offset
  EW_STAGE_BYTE4,        // one 32-bit load of 4 contiguous bool / u8 values, widened to 4 floats
};

struct EwInput {
  const void* ptr;
  int32_t dtype;
  int32_t kind;
  int64_t stride[kEwMaxRank];  // element strides over the collapsed output dims; 0 = broadcast
  int32_t vec_ok;              // inner stride 1, base 16-byte aligned, outer strides % 4 == 0
  int32_t mode;                // EwStageMode, filled by launch_elementwise
};

struct EwOutput {
  void* ptr;
  int32_t dtype;
  uint8_t src;  // slot or EW_ACC (only the last instruction's result may use EW_ACC)
  uint8_t pad[3];
};

struct EwProgram {
  int32_t rank;  // collapsed output rank (>= 1)
  int32_t n_inputs, n_outputs, n_instr, n_slots;
  int32_t vec;                // 1: inner extent % 4 == 0 and every output base 16-byte aligned
  uint32_t dim[kEwMaxRank];   // collapsed output extents, outermost first
  int64_t total;              // number of output elements
  EwInput in[kEwMaxInputs];
  EwOutput out[kEwMaxOutputs];
  EwInstr instr[kEwMaxInstr];
};

int launch_elementwise(const EwProgram& prog, cudaStream_t s);
// The register code a linear chain would run (assuming aligned operands) as a signature string, and whether that code
// is one of the programs compiled into the library as straight-line kernels; "" for programs on the slot-file path.
std::string ew_register_signature(const EwProgram& prog, bool* compiled_in);
// The same program with every value carried as a double: exact for f64 tensors and for integers up to 2^53, which
// the f32 lanes of the kernels above are not.  `imm` holds the kEwMaxInstr immediates at full precision.
int launch_elementwise_wide(const EwProgram& prog, const double* imm, cudaStream_t s);

}  // namespace ib200

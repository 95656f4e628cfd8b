/*
 * intentir_b200 — C ABI of the B200 (sm_100a) execution backend for IntentIR graphs.
 *
 * This is the boundary a host binds instead of the reference's CUDA backend:
 *   - planning replaces  backends/cuda/cpp_codegen/intentir_cuda_codegen.cpp:5855-5873
 *     (pybind `lower_from_json_str(intent_json, bindings_json) -> json`) and the Python
 *     dispatcher backends/cuda/codegen/intentir_to_cuda.py:2047-2201;
 *   - launching replaces the generated torch-extension wrapper of
 *     frontends/cuda/runtime.py:621-804 (`launch(*tensors, *scalars, grid, block, smem)`),
 *     with the kernels of backends/cuda/runtime/kernels/*.cuh replaced by the
 *     pre-compiled sm_100a kernels in this library.
 *
 * Conventions
 *   - Plain pointers and sizes only.  Every `const void*` / `void*` tensor argument is a
 *     DEVICE pointer to a dense row-major array owned by the caller and borrowed for the
 *     duration of the call.
 *   - `stream` is a `cudaStream_t` passed as `void*` (NULL = the legacy default stream).
 *     Calls only enqueue work: the library never synchronises and never allocates device
 *     memory; scratch memory, where needed, is passed in by the caller (`workspace`).
 *   - Functions return IB200_OK (0) or a negative status; `ib200_last_error()` returns a
 *     thread-local, human readable message for the last failure on the calling thread.
 *   - The device is the caller's current CUDA device.
 */
#ifndef INTENTIR_B200_H_
#define INTENTIR_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define IB200_API __attribute__((visibility("default")))
#else
#define IB200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------- */
#define IB200_OK 0
#define IB200_ERR_INVALID (-1)     /* bad argument (null pointer, negative extent, bad dtype)      */
#define IB200_ERR_UNSUPPORTED (-2) /* graph / shape / dtype outside what the kernels cover; the    */
                                   /* counterpart of CudaLoweringError, intentir_to_cuda.py:23-24  */
#define IB200_ERR_CUDA (-3)        /* a CUDA runtime / driver call failed (CudaRuntimeError,       */
                                   /* frontends/cuda/runtime.py:23-24)                             */
#define IB200_ERR_BUFFER (-4)      /* caller-provided output / workspace buffer too small          */
#define IB200_ERR_DEVICE_WAIT (-5) /* a bounded device-side wait ran out (see ib200_check_status)  */

/* ---- element types (the IntentIR dtype strings of intent_ir/ir/ir_types.py:38-64) ---- */
#define IB200_F32 0
#define IB200_BF16 1
#define IB200_F16 2
#define IB200_I32 3
#define IB200_I64 4
#define IB200_BOOL 5 /* "bool" and "i1": one byte, 0 or 1 */
#define IB200_U8 6
#define IB200_I8 7
#define IB200_I16 8
#define IB200_F64 9

/* ---- reduction kinds for ib200_reduce ------------------------------------------------- */
#define IB200_REDUCE_SUM 0 /* reduce_sum, verify/interpreter.py:478-488 (optional scale)        */
#define IB200_REDUCE_MAX 1 /* reduce_max, :495-500 (NaN propagates, like np.max)                */
#define IB200_REDUCE_ANY 2 /* reduce_any, :489-494 (element != 0; NaN counts as true)           */

/* ---- activation codes for ib200_gemm_bias_act ---------------------------------------- */
#define IB200_ACT_NONE 0
#define IB200_ACT_RELU 1
/* ---- flags for ib200_gemm_bias_act_ws ------------------------------------------------- */
#define IB200_GEMM_CTA_PAIRS 2  /* force the tensor-core product onto pairs of CTAs (tcgen05 cta_group::2, 256 x 256 tiles) */
#define IB200_GEMM_ONE_CTA 4    /* force the one-CTA kernel (128 x 256/192/128 tiles); default: pairs for large products */
#define IB200_GEMM_NARROW_TAIL 8 /* CTA pairs: the tiles of a mostly empty last round run as two 256 x 128 units each (default: whole) */
#define IB200_GEMM_ALLOW_TF32 1 /* f32 operands may be multiplied as TF32 on the tensor cores (the reference's
                                   ALLOW_TF32 binding, intentir_to_cuda.py:577-578); without it f32 stays exact FMA */

IB200_API const char* ib200_last_error(void);
IB200_API int ib200_version(void);

/* ======================================================================================
 * Planner + executor: IntentIR JSON in, a launchable plan out.
 * ====================================================================================== */

typedef struct ib200_plan ib200_plan_t;

/* Stateless: lower an IntentIR graph under concrete bindings and write the plan
 * description as JSON into `out` (NUL terminated).  Replaces
 * `lower_from_json_str(intent_json, bindings_json)` (intentir_cuda_codegen.cpp:5858).
 * The JSON mirrors the reference's lowered-kernel record
 * {kernel_name, cuda_src:"", io_spec{arg_names, tensors{name:{dtype,shape}}, scalars},
 *  launch{grid,block,shared_mem}, output_names, bindings} (intentir_to_cuda.py:2110-2125)
 * plus {"steps":[...], "buffers":[...], "workspace_bytes":N}.  A step names its kernel and extents and
 * either its micro-op program ("program" for elementwise steps, "row_program" for fused row steps:
 * operands with buffer ids, offsets and strides, instructions, stores) or, for the reduce / softmax /
 * normalisation / product / transpose kernels, "args": the buffer ids and options its launcher is given --
 * enough for a host to follow, or re-execute, what a launch will do without a device.  Non-finite numbers
 * are read and written as Python's json module does: NaN, Infinity, -Infinity.  Returns
 * IB200_ERR_BUFFER when `cap` is too small (the needed size is then reported by ib200_last_error). */
IB200_API int ib200_plan_json(const char* intent_json, const char* bindings_json, char* out, size_t cap);

/* Build a reusable plan object (same lowering as ib200_plan_json). */
IB200_API int ib200_plan_create(const char* intent_json, const char* bindings_json, ib200_plan_t** plan);
IB200_API void ib200_plan_destroy(ib200_plan_t* plan);
IB200_API int ib200_plan_describe(const ib200_plan_t* plan, char* out, size_t cap);
/* Number of tensor arguments (io_spec.arg_names order: external inputs, then outputs). */
IB200_API int ib200_plan_num_args(const ib200_plan_t* plan);
/* Scratch bytes the caller must provide to ib200_plan_launch (0 for single-kernel plans). */
IB200_API size_t ib200_plan_workspace_bytes(const ib200_plan_t* plan);
/* Number of kernel launches one ib200_plan_launch enqueues. */
IB200_API int ib200_plan_num_launches(const ib200_plan_t* plan);

/* Enqueue the plan.  `args[i]` is the device pointer of io_spec.arg_names[i].  `workspace`
 * must be 256-byte aligned and at least ib200_plan_workspace_bytes(plan) long (may be NULL
 * when that is 0).  ZERO-FILL THE WORKSPACE ONCE before its first use: plans whose kernels have
 * bounded device-side waits keep a status word in it that is only ever written when a wait
 * runs out, so garbage there reads as a failure.  Replaces `mod.launch(...)`
 * (frontends/cuda/runtime.py:723-746). */
IB200_API int ib200_plan_launch(const ib200_plan_t* plan, void* const* args, int n_args, void* workspace,
                      size_t workspace_bytes, void* stream);

/* After the plan's launches: synchronise `stream`, read the plan's status word out of
 * `workspace` and return IB200_ERR_DEVICE_WAIT if a bounded device-side wait ran out during
 * the plan (IB200_OK at once for plans without such kernels).  The word is left as found:
 * clear it (4 bytes at the offset "status_offset" of the plan description) before reusing
 * the workspace after a failure.  The reference has no counterpart: its kernels have no
 * device-side waits. */
IB200_API int ib200_plan_check_status(const ib200_plan_t* plan, const void* workspace, void* stream);

/* Same as ib200_plan_launch, for callers that cannot supply a workspace because they are not
 * allowed to allocate device memory (their memory belongs to another runtime's pool, or
 * their hot loop must never reach cudaMalloc).  The scratch is a fixed array of
 * ib200_noalloc_workspace_limit() bytes (32 MiB) built into the library image; a GPU holds
 * it from the moment the CUDA runtime loads the library's module there until the process
 * exits.  Plans needing more return IB200_ERR_BUFFER and launch nothing.  The array is
 * shared by all calls in the process: calls whose kernels could overlap on the GPU race on
 * it, so keep them ordered.  The first call on a device resolves the array's address; under
 * the runtime's lazy module loading (the default) that is also when the runtime backs the
 * 32 MiB, so make this first call early, while the device still has that much free, and
 * outside any stream capture.  The library itself never allocates.
 * This entry point has no counterpart in the reference: its runner always allocates through
 * torch (frontends/cuda/runtime.py:961-1008). */
IB200_API int ib200_plan_launch_noalloc(const ib200_plan_t* plan, void* const* args, int n_args, void* stream);
IB200_API size_t ib200_noalloc_workspace_limit(void);
/* ib200_plan_check_status for a plan launched through ib200_plan_launch_noalloc: reads the
 * status word out of the built-in array on the current device (synchronises `stream`).  Call
 * it before the next ib200_plan_launch_noalloc, which clears the word.  No counterpart in the
 * reference. */
IB200_API int ib200_plan_check_status_noalloc(const ib200_plan_t* plan, void* stream);
/* Failure injection from the host, for tests of the error path: writes `code` into the plan's
 * status word inside the built-in array, exactly where a kernel whose bounded wait ran out
 * would have written it (synchronises `stream`).  No GPU work is disturbed.  No counterpart
 * in the reference. */
IB200_API int ib200_noalloc_debug_poke_status(const ib200_plan_t* plan, int32_t code, void* stream);

/* ======================================================================================
 * Direct per-op entry points (the same kernels the plans launch).
 * ====================================================================================== */

/* out[o, i] = reduce over r of x[o, r, i]  — x viewed as [outer, reduce, inner], dense.
 * SUM: out = scale * sum (scale 1.0 for plain sums); MAX propagates NaN; ANY writes one
 * byte per output (x_dtype may be a float type or IB200_BOOL; out_dtype must be IB200_BOOL).
 * Replaces the generated reduce_sum / reduce_max / any_dim kernels
 * (intentir_to_cuda.py:1553-1776) and kernels/reduce.cuh. */
IB200_API int ib200_reduce(const void* x, void* out, int x_dtype, int out_dtype, int kind, int64_t outer,
                 int64_t reduce, int64_t inner, float scale, void* stream);

/* The same reduction with scratch memory, which lets shapes with too few independent results to fill
 * the GPU (a handful of very long rows, a whole-tensor sum, a reduction over the leading axis of a
 * narrow matrix) be split along the reduced axis: every CTA reduces one segment, and the CTA that
 * finishes last folds the partial results in segment order, so results do not vary from run to run.
 * ib200_reduce_scratch_bytes gives the amount for a shape (0: that shape is never split); `scratch`
 * is 256-byte aligned device memory in any state, not shared with a launch that may run at the
 * same time.  With too little scratch (or NULL) this is ib200_reduce. */
IB200_API size_t ib200_reduce_scratch_bytes(int64_t outer, int64_t reduce, int64_t inner);
IB200_API int ib200_reduce_ws(const void* x, void* out, int x_dtype, int out_dtype, int kind, int64_t outer,
                    int64_t reduce, int64_t inner, float scale, void* scratch, size_t scratch_bytes, void* stream);

/* The BASELINE any_kernel_dim case: out[m] = any_n(x[m, n] != 0), f32 in, one byte out. */
IB200_API int ib200_reduce_any_f32(const float* x, uint8_t* out, int64_t rows, int64_t cols, void* stream);

/* Row softmax over the last axis with max subtraction (verify/interpreter.py:501-506).
 * `row_max` / `row_sum` (f32[rows]) are optional extra outputs (NULL to skip): the row
 * maximum and the sum of exp(x - max), as the decomposed graph of
 * pipeline/cuda/core.py:453-493 exposes them.  Replaces kernels/softmax.cuh (no 1024
 * column limit). dtype: IB200_F32, IB200_BF16 or IB200_F16 (same for x and y). */
IB200_API int ib200_softmax(const void* x, void* y, float* row_max, float* row_sum, int dtype, int64_t rows,
                  int64_t cols, void* stream);

/* Same kernel with separate input and output types: y may be IB200_F32 for bf16 / f16 inputs
 * (a bf16 result above 0.5 cannot meet the verifier's 1e-3 tolerance, verify/tolerances.py:111-113). */
IB200_API int ib200_softmax_io(const void* x, void* y, float* row_max, float* row_sum, int in_dtype, int out_dtype,
                     int64_t rows, int64_t cols, void* stream);

/* Softmax / row normalisation with scratch memory (16-byte aligned, ib200_softmax_scratch_bytes /
 * ib200_norm_scratch_bytes bytes; 0 means the shape never uses it; contents irrelevant).  Rows
 * longer than the resident kernels hold (16 Ki elements; 128 Ki for the normalisation's cluster
 * kernels) that are too few to fill the GPU one CTA per row, or too large for L2, are cut into
 * segments of 8 Ki .. 64 Ki elements, one CTA each: pass 1 leaves (max, sum) or (mean, squared
 * deviations) per segment in the scratch, pass 2 folds them in a fixed order and writes the
 * segment.  Without scratch these shapes run one streaming CTA per row.  Same arithmetic as
 * ib200_softmax_io / ib200_norm_rows; no counterpart in the reference (its softmax stops at
 * 1024 columns, kernels/softmax.cuh). */
IB200_API int ib200_softmax_ws(const void* x, void* y, float* row_max, float* row_sum, int in_dtype, int out_dtype,
                     int64_t rows, int64_t cols, void* scratch, size_t scratch_bytes, void* stream);
IB200_API size_t ib200_softmax_scratch_bytes(int dtype, int64_t rows, int64_t cols);
IB200_API int ib200_norm_rows_ws(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                       int dtype, int affine_dtype, int64_t rows, int64_t cols, int64_t affine_inner,
                       int64_t affine_period, float eps, void* scratch, size_t scratch_bytes, void* stream);
IB200_API size_t ib200_norm_scratch_bytes(int dtype, int64_t rows, int64_t cols);

/* softmax(where(mask, x, fill)) over f32 rows of at most 16384 elements, the mask applied as each row
 * is loaded (the masked scores are never written): mask holds one byte per element (0 = replace by
 * `fill`), row r starting at mask + r * mask_row_stride, so 0 shares one mask vector between all rows
 * and `cols` gives every row its own.  The graph form is where -> softmax,
 * pipeline/tilelang/core.py:1050-1076; the plan builder folds it into this kernel by itself. */
IB200_API int ib200_softmax_masked(const void* x, const void* mask, int64_t mask_row_stride, float fill, void* y,
                         float* row_max, float* row_sum, int64_t rows, int64_t cols, void* stream);

/* Normalisation over contiguous rows of `cols` elements with centred (two-pass) variance:
 *   mean = sum(x)/cols; var = sum((x-mean)^2)/cols; rstd = 1/sqrt(var+eps);
 *   y[r, j] = (x[r, j]-mean)*rstd * w[widx] + b[widx],  widx = ((r*cols + j) / affine_inner) % affine_period
 * layernorm: affine_inner = 1, affine_period = cols.  groupnorm over X[N,C,HW] with G groups:
 * rows = N*G, cols = (C/G)*HW, affine_inner = HW, affine_period = C.  w / b may be NULL
 * (identity affine).  mean / rstd (f32[rows]) may be NULL.  x, y share `dtype`; w, b share
 * `affine_dtype`.  Replaces kernels/layernorm.cuh (which uses E[x^2]-mean^2); groupnorm has
 * no counterpart in the reference CUDA backend (oracle: pipeline/tilelang/core.py:187-232). */
IB200_API int ib200_norm_rows(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                    int dtype, int affine_dtype, int64_t rows, int64_t cols, int64_t affine_inner,
                    int64_t affine_period, float eps, void* stream);

IB200_API int ib200_layernorm(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                    int dtype, int64_t rows, int64_t cols, float eps, void* stream);

IB200_API int ib200_groupnorm(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                    int dtype, int64_t n, int64_t c, int64_t hw, int64_t groups, float eps,
                    void* stream);

/* C[M,N] = act(A[M,K] · B + bias[N]); fp32 accumulation.  B is [K,N] row-major, or [N,K]
 * when transpose_b != 0.  bias may be NULL.  in_dtype (A and B) is IB200_BF16, IB200_F16 or
 * IB200_F32; out_dtype (C) is in_dtype or IB200_F32; bias has out_dtype.  16-bit inputs whose K
 * and N are multiples of 8 run on the tcgen05 / TMEM tensor-core path; everything else runs on a
 * tiled fp32 FMA kernel.
 * `status` is a caller-provided device int32 (zero it once); the tensor-core kernel sets it
 * non-zero if one of its bounded waits runs out (read it with ib200_check_status).  May be
 * NULL for the FMA path only.  Replaces kernels/wmma_matmul.cuh and matmul_fallback.cuh. */
IB200_API int ib200_gemm_bias_act(const void* a, const void* b, const void* bias, void* c, int in_dtype,
                        int out_dtype, int64_t m, int64_t n, int64_t k, int transpose_b, int act,
                        int32_t* status, void* stream);

/* The same product with options and scratch memory.  `flags`: IB200_GEMM_ALLOW_TF32 sends f32
 * operands (K, N multiples of 8) to the tensor cores as TF32, which is what the reference's
 * opt-in wmma kernel does (kernels/wmma_matmul.cuh:124-563); products then carry 10-bit
 * mantissas, inside the verifier's matmul tolerance for inputs of moderate dynamic range.
 * Large products (M >= 256, tiles for at least half the SM pairs) run on pairs of CTAs sharing
 * 256 x 256 tiles (tcgen05 cta_group::2); IB200_GEMM_CTA_PAIRS / IB200_GEMM_ONE_CTA force either form, and
 * IB200_GEMM_NARROW_TAIL lets the pair kernel run the tiles of a short last round as 256 x 128 units.
 * `scratch` (256-byte aligned, ib200_gemm_scratch_bytes(...) bytes, contents irrelevant) lets the
 * one-CTA kernel cut the tiles of a last, mostly empty round of tiles along K and add the
 * slices up in a fixed order; with scratch == NULL every tile runs whole, as in
 * ib200_gemm_bias_act.  A TF32 product whose B is [K,N] transposes B into the scratch first
 * (the tensor-core kernel takes 32-bit operands K-major only) and stays on the FMA kernel
 * when the scratch is too small for that.  Plans take the scratch from their workspace. */
IB200_API int ib200_gemm_bias_act_ws(const void* a, const void* b, const void* bias, void* c, int in_dtype,
                           int out_dtype, int64_t m, int64_t n, int64_t k, int transpose_b, int act, int flags,
                           void* scratch, size_t scratch_bytes, int32_t* status, void* stream);
IB200_API size_t ib200_gemm_scratch_bytes(int in_dtype, int out_dtype, int64_t m, int64_t n, int64_t k, int transpose_b, int flags);

/* Copy the device status word to the host (this call DOES synchronise `stream`) and map a
 * non-zero word to IB200_ERR_DEVICE_WAIT.  With status == NULL it checks the library's own word,
 * which the direct normalisation entry points use for their bounded waits on staged rows. */
IB200_API int ib200_check_status(const int32_t* status, void* stream);

/* out[i, j] = x[j, i] for a dense [rows, cols] matrix of 2- or 4-byte elements.
 * Replaces the generated transpose2d kernel (intentir_to_cuda.py:1487-1550). */
IB200_API int ib200_transpose2d(const void* x, void* out, int elem_bytes, int64_t rows, int64_t cols,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INTENTIR_B200_H_ */

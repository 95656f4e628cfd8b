// The extern "C" surface declared in include/intentir_b200.h: argument checks, the
// thread-local error message, and forwarding to the per-file launchers.
#include <string>

#include "common.cuh"

namespace ib200 {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}
int cuda_fail(cudaError_t err, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorName(err) + " (" + cudaGetErrorString(err) + ")";
  return IB200_ERR_CUDA;
}

}  // namespace ib200

using namespace ib200;

extern "C" {

const char* ib200_last_error(void) { return g_last_error.c_str(); }
int ib200_version(void) { return 100; }

int ib200_reduce(const void* x, void* out, int x_dtype, int out_dtype, int kind, int64_t outer, int64_t reduce, int64_t inner,
                 float scale, void* stream) {
  return launch_reduce(x, out, x_dtype, out_dtype, kind, outer, reduce, inner, scale, static_cast<cudaStream_t>(stream));
}

size_t ib200_reduce_scratch_bytes(int64_t outer, int64_t reduce, int64_t inner) { return reduce_scratch_bytes(outer, reduce, inner); }

int ib200_reduce_ws(const void* x, void* out, int x_dtype, int out_dtype, int kind, int64_t outer, int64_t reduce, int64_t inner,
                    float scale, void* scratch, size_t scratch_bytes, void* stream) {
  if (scratch && (reinterpret_cast<uintptr_t>(scratch) & 255u)) return fail(IB200_ERR_INVALID, "reduce_ws: scratch must be 256-byte aligned");
  return launch_reduce(x, out, x_dtype, out_dtype, kind, outer, reduce, inner, scale, static_cast<cudaStream_t>(stream), scratch, scratch_bytes);
}

int ib200_reduce_any_f32(const float* x, uint8_t* out, int64_t rows, int64_t cols, void* stream) {
  return launch_reduce(x, out, IB200_F32, IB200_BOOL, IB200_REDUCE_ANY, rows, cols, 1, 1.0f, static_cast<cudaStream_t>(stream));
}

int ib200_softmax(const void* x, void* y, float* row_max, float* row_sum, int dtype, int64_t rows, int64_t cols, void* stream) {
  return launch_softmax(x, y, row_max, row_sum, dtype, rows, cols, static_cast<cudaStream_t>(stream));
}

int ib200_softmax_io(const void* x, void* y, float* row_max, float* row_sum, int in_dtype, int out_dtype, int64_t rows, int64_t cols,
                     void* stream) {
  return launch_softmax(x, y, row_max, row_sum, in_dtype, rows, cols, static_cast<cudaStream_t>(stream), out_dtype);
}

int ib200_softmax_masked(const void* x, const void* mask, int64_t mask_row_stride, float fill, void* y, float* row_max, float* row_sum,
                         int64_t rows, int64_t cols, void* stream) {
  if (!mask) return fail(IB200_ERR_INVALID, "softmax_masked: mask is null");
  if (mask_row_stride < 0 || (mask_row_stride > 0 && rows > 0 && beyond_any_device(rows, mask_row_stride)))
    return fail(IB200_ERR_INVALID, "softmax_masked: the mask's row stride must be 0 (one vector for all rows) or positive");
  const SoftmaxMask mk{static_cast<const uint8_t*>(mask), mask_row_stride, fill, 0};
  return launch_softmax(x, y, row_max, row_sum, IB200_F32, rows, cols, static_cast<cudaStream_t>(stream), IB200_F32, &mk);
}

int ib200_softmax_ws(const void* x, void* y, float* row_max, float* row_sum, int in_dtype, int out_dtype, int64_t rows, int64_t cols,
                     void* scratch, size_t scratch_bytes, void* stream) {
  if (scratch && (reinterpret_cast<uintptr_t>(scratch) & 15u)) return fail(IB200_ERR_INVALID, "softmax_ws: scratch must be 16-byte aligned");
  return launch_softmax(x, y, row_max, row_sum, in_dtype, rows, cols, static_cast<cudaStream_t>(stream), out_dtype, nullptr, scratch, scratch_bytes);
}
size_t ib200_softmax_scratch_bytes(int dtype, int64_t rows, int64_t cols) { return softmax_scratch_bytes(rows, cols, dtype == IB200_F32 ? 4 : 2); }

int ib200_norm_rows_ws(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int dtype, int affine_dtype,
                       int64_t rows, int64_t cols, int64_t affine_inner, int64_t affine_period, float eps, void* scratch,
                       size_t scratch_bytes, void* stream) {
  if (scratch && (reinterpret_cast<uintptr_t>(scratch) & 15u)) return fail(IB200_ERR_INVALID, "norm_rows_ws: scratch must be 16-byte aligned");
  return launch_norm_rows(x, w, b, y, mean, rstd, dtype, affine_dtype, rows, cols, affine_inner, affine_period, eps,
                          static_cast<cudaStream_t>(stream), nullptr, true, nullptr, nullptr, scratch, scratch_bytes);
}
size_t ib200_norm_scratch_bytes(int dtype, int64_t rows, int64_t cols) { return norm_scratch_bytes(rows, cols, dtype == IB200_F32 ? 4 : 2); }

int ib200_norm_rows(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int dtype, int affine_dtype,
                    int64_t rows, int64_t cols, int64_t affine_inner, int64_t affine_period, float eps, void* stream) {
  return launch_norm_rows(x, w, b, y, mean, rstd, dtype, affine_dtype, rows, cols, affine_inner, affine_period, eps,
                          static_cast<cudaStream_t>(stream));
}

int ib200_layernorm(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int dtype, int64_t rows,
                    int64_t cols, float eps, void* stream) {
  return launch_norm_rows(x, w, b, y, mean, rstd, dtype, dtype, rows, cols, 1, cols, eps, static_cast<cudaStream_t>(stream));
}

int ib200_groupnorm(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int dtype, int64_t n,
                    int64_t c, int64_t hw, int64_t groups, float eps, void* stream) {
  if (groups <= 0 || c < 0 || n < 0 || hw < 0) return fail(IB200_ERR_INVALID, "groupnorm: bad extents");
  if (beyond_any_device(n, c > 0 ? c : 1, hw > 0 ? hw : 1)) return fail(IB200_ERR_INVALID, "groupnorm: more than 2^40 elements");
  if (c % groups != 0) return fail(IB200_ERR_INVALID, "groupnorm: C must be a multiple of the group count");
  return launch_norm_rows(x, w, b, y, mean, rstd, dtype, dtype, n * groups, (c / groups) * hw, hw > 0 ? hw : 1, c > 0 ? c : 1,
                          eps, static_cast<cudaStream_t>(stream));
}

int ib200_gemm_bias_act(const void* a, const void* b, const void* bias, void* c, int in_dtype, int out_dtype, int64_t m,
                        int64_t n, int64_t k, int transpose_b, int act, int32_t* status, void* stream) {
  return launch_gemm(a, b, bias, c, in_dtype, out_dtype, m, n, k, transpose_b, act, status, static_cast<cudaStream_t>(stream));
}

int ib200_gemm_bias_act_ws(const void* a, const void* b, const void* bias, void* c, int in_dtype, int out_dtype, int64_t m,
                           int64_t n, int64_t k, int transpose_b, int act, int flags, void* scratch, size_t scratch_bytes,
                           int32_t* status, void* stream) {
  if (scratch && (reinterpret_cast<uintptr_t>(scratch) & 255u)) return fail(IB200_ERR_INVALID, "gemm_bias_act_ws: scratch must be 256-byte aligned");
  return launch_gemm(a, b, bias, c, in_dtype, out_dtype, m, n, k, transpose_b, act, status, static_cast<cudaStream_t>(stream), flags,
                     scratch, scratch_bytes);
}

size_t ib200_gemm_scratch_bytes(int in_dtype, int out_dtype, int64_t m, int64_t n, int64_t k, int transpose_b, int flags) {
  return gemm_scratch_bytes(in_dtype, out_dtype, m, n, k, flags, transpose_b);
}

int ib200_check_status(const int32_t* status, void* stream) {
  if (!status) status = norm_default_status();  // the word used by the direct normalisation entry points
  if (!status) return fail(IB200_ERR_CUDA, "check_status: no status word on this device");
  int32_t host = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  IB200_CUDA_OK(cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, s));
  IB200_CUDA_OK(cudaStreamSynchronize(s));
  if (host != 0) {
    static const char* where[] = {"", "producer waiting for a free ring stage", "MMA issuer waiting for a drained accumulator",
                                  "MMA issuer waiting for a TMA stage", "epilogue waiting for a finished accumulator",
                                  "normalisation waiting for a staged row segment", "normalisation waiting for its cluster's statistics",
                                  "long-row kernel waiting for the other segments of its row"};
    return fail(IB200_ERR_DEVICE_WAIT, std::string("bounded device wait expired (") +
                                           (host > 0 && host < 8 ? where[host] : "unknown site") + ")");
  }
  return IB200_OK;
}

int ib200_transpose2d(const void* x, void* out, int elem_bytes, int64_t rows, int64_t cols, void* stream) {
  return launch_transpose2d(x, out, elem_bytes, rows, cols, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ib200_plan_launch_noalloc: run a plan without the caller providing (or anyone allocating)
// a workspace.
//
// Who needs this: hosts that are allowed to launch work on the GPU but not to allocate on
// it.  Two examples are a verification worker living inside a process whose device memory is
// entirely owned by another framework's pool, and a latency-critical loop that must never
// reach cudaMalloc (which can synchronise the whole device and takes an unpredictable time).
// Such a host cannot hand ib200_plan_launch the scratch buffer that multi-kernel plans need
// for their intermediates.
//
// What it does instead: the scratch lives in a fixed array in device global memory that is
// part of this library's image (IB200_NOALLOC_WORKSPACE_BYTES, 32 MiB).  A GPU carries the
// array from the moment the CUDA runtime loads this translation unit's module on it until the
// process exits.  When that moment is depends on the runtime's module loading mode: with eager
// loading it is context creation, whether or not this entry point is ever called; with lazy
// loading (the default of current CUDA releases, CUDA_MODULE_LOADING=LAZY) it is the first call
// of this entry point on that device, whose address lookup makes the runtime load the module
// and back the 32 MiB — measured on a B200: free device memory drops by 32 MiB (plus the
// module's code) across that first call and stays flat across later ones.  Plans that need
// more are refused with IB200_ERR_BUFFER; nothing is launched in that case.
//
// Rules for callers
//   * The first call on each device looks up the array's device address.  This library
//     allocates nothing for it, but under lazy module loading the runtime materialises the
//     array at that moment, so it can fail with an out-of-memory status if the device is
//     already full: make the first call early (a plan that needs no scratch will do), and
//     outside of any stream capture.
//   * The array is shared by every call in the process.  Its contents after a call are
//     whatever that plan left there; the one region a plan expects to start at zero (the
//     status word of the tensor-core GEMM) is cleared on the stream at the start of each
//     call.  Two calls whose kernels can overlap on the GPU (different streams, no ordering
//     between them) would both write the array: do not do that, order them.
//   * No cudaMalloc / cudaFree / allocating library routine is reached from here; inputs and
//     outputs are still the caller's buffers, as for ib200_plan_launch.
#include <mutex>

#include "common.cuh"

#define IB200_NOALLOC_WORKSPACE_BYTES (32u << 20)

namespace ib200 {
long plan_status_offset(const ib200_plan* plan);  // plan.cu: byte offset of the status word, or -1
}

namespace {

// Device-side storage.  In host code this name is only a handle for the runtime: the
// address kernels must be given comes from cudaGetSymbolAddress, below.
static __device__ __align__(256) unsigned char g_noalloc_workspace[IB200_NOALLOC_WORKSPACE_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_workspace_addr[kMaxDevices] = {};

// Once per device, with that device current: resolve the array's device address.
int workspace_for_current_device(void** out) {
  int dev = -1;
  IB200_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ib200::fail(IB200_ERR_UNSUPPORTED, "plan_launch_noalloc: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_workspace_addr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_workspace);
    if (e != cudaSuccess) return ib200::cuda_fail(e, "cudaGetSymbolAddress(noalloc workspace)");
    if (!p) return ib200::fail(IB200_ERR_CUDA, "plan_launch_noalloc: the workspace symbol has no device address");
    g_workspace_addr[dev] = p;
  }
  *out = g_workspace_addr[dev];
  return IB200_OK;
}

}  // namespace

extern "C" {

size_t ib200_noalloc_workspace_limit(void) { return IB200_NOALLOC_WORKSPACE_BYTES; }

int ib200_plan_check_status_noalloc(const ib200_plan_t* plan, void* stream) {
  if (!plan) return ib200::fail(IB200_ERR_INVALID, "plan_check_status_noalloc: null plan");
  if (ib200::plan_status_offset(plan) < 0) return IB200_OK;
  void* ws = nullptr;
  if (int rc = workspace_for_current_device(&ws)) return rc;
  return ib200_plan_check_status(plan, ws, stream);
}

int ib200_noalloc_debug_poke_status(const ib200_plan_t* plan, int32_t code, void* stream) {
  if (!plan) return ib200::fail(IB200_ERR_INVALID, "noalloc_debug_poke_status: null plan");
  const long status = ib200::plan_status_offset(plan);
  if (status < 0) return ib200::fail(IB200_ERR_INVALID, "noalloc_debug_poke_status: this plan has no status word");
  void* ws = nullptr;
  if (int rc = workspace_for_current_device(&ws)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  IB200_CUDA_OK(cudaMemcpyAsync(static_cast<char*>(ws) + status, &code, sizeof(code), cudaMemcpyHostToDevice, s));
  IB200_CUDA_OK(cudaStreamSynchronize(s));  // `code` is a stack variable
  return IB200_OK;
}

int ib200_plan_launch_noalloc(const ib200_plan_t* plan, void* const* args, int n_args, void* stream) {
  if (!plan) return ib200::fail(IB200_ERR_INVALID, "plan_launch_noalloc: null plan");
  const size_t need = ib200_plan_workspace_bytes(plan);
  if (need > IB200_NOALLOC_WORKSPACE_BYTES)
    return ib200::fail(IB200_ERR_BUFFER, "plan_launch_noalloc: this plan needs " + std::to_string(need) +
                                             " bytes of scratch, the built-in workspace holds " +
                                             std::to_string((size_t)IB200_NOALLOC_WORKSPACE_BYTES) +
                                             "; use ib200_plan_launch with a caller-provided workspace");
  void* ws = nullptr;
  if (int rc = workspace_for_current_device(&ws)) return rc;
  const long status = ib200::plan_status_offset(plan);
  if (status >= 0)  // the previous user of the array may have left anything here
    IB200_CUDA_OK(cudaMemsetAsync(static_cast<char*>(ws) + status, 0, 256, static_cast<cudaStream_t>(stream)));
  return ib200_plan_launch(plan, args, n_args, ws, IB200_NOALLOC_WORKSPACE_BYTES, stream);
}

}  // extern "C"

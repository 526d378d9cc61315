// trifast_backward_static_scratch: the whole backward with its scratch memory in
// a fixed device array owned by the library, for callers that must not allocate.
//
// Who needs this: code that runs where device allocation is off limits -- an
// inference or training runtime that handed the whole GPU to its own memory
// pool at start-up (so a late cudaMalloc fails or fragments the pool), a plugin
// whose enqueue callback is forbidden to allocate, or a latency-critical loop
// that cannot afford the implicit synchronisation of cudaMalloc / cudaFree.
// Such callers can still pass their inputs and outputs, but have nowhere to get
// the backward's workspace (delta, fully-masked-row flags, the fp32 bias
// gradient and its row-split partials) from.  Here that workspace lives in
// g_scratch below, so the call allocates nothing.

#include <mutex>

#include "kernels.h"

namespace trifast {
namespace {

// Upper bound of the scratch this entry point serves.  Every GPU that loads the
// library keeps this much device memory reserved until the process exits.
constexpr size_t kStaticScratchBytes = TRIFAST_STATIC_SCRATCH_BYTES;  // 16 MiB

// The scratch itself.  In host code this name is only a handle for the runtime:
// it is not a device address and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned char g_scratch[kStaticScratchBytes];

constexpr int kMaxDev = 64;
void* g_scratch_ptr[kMaxDev];
cudaError_t g_scratch_err[kMaxDev];
std::once_flag g_scratch_once[kMaxDev];

// Device address of g_scratch on the current device, resolved once per device
// with that device current.
int scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return TRIFAST_ERR_LAUNCH;
  std::call_once(g_scratch_once[dev], [dev] {
    void* p = nullptr;
    g_scratch_err[dev] = cudaGetSymbolAddress(&p, g_scratch);
    g_scratch_ptr[dev] = (g_scratch_err[dev] == cudaSuccess) ? p : nullptr;
  });
  if (g_scratch_err[dev] != cudaSuccess || !g_scratch_ptr[dev]) return TRIFAST_ERR_LAUNCH;
  *out = g_scratch_ptr[dev];
  return TRIFAST_OK;
}

}  // namespace
}  // namespace trifast

extern "C" {

int trifast_backward_static_scratch(const trifast_shape* shape, const trifast_t5* d_o,
                                    const trifast_t5* q, const trifast_t5* k, const trifast_t5* v,
                                    const trifast_t4* bias, const trifast_mask* mask,
                                    const trifast_t5* o, const float* lse, const trifast_t5* dq,
                                    const trifast_t5* dk, const trifast_t5* dv,
                                    const trifast_t4* db, void* stream) {
  if (!shape) return TRIFAST_ERR_NULL;
  const size_t need = trifast_backward_workspace_bytes(shape);
  if (need == 0) {  // invalid shape: let the common validation name the reason
    trifast_plan plan;
    const int rc = trifast_pick_plan(shape, &plan);
    return rc ? rc : TRIFAST_ERR_SHAPE;
  }
  if (need > trifast::kStaticScratchBytes) return TRIFAST_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = trifast::scratch_address(&scratch);
  if (rc) return rc;
  // Nothing in the scratch has to start at zero: delta, the row flags, the fp32
  // bias gradient and every partial are written in full by this call before
  // anything reads them, so the previous call's contents are simply overwritten.
  return trifast_backward(shape, d_o, q, k, v, bias, mask, o, lse, dq, dk, dv, db, scratch,
                          trifast::kStaticScratchBytes, stream);
}

}  // extern "C"

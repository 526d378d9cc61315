// A kernel whose only job is to let one bounded wait run out, so that the path
// "wait gives up -> status word -> host error" can be exercised without making
// any real kernel misbehave.  One warp waits on an mbarrier that nobody ever
// arrives on, with the limit passed as an argument; when the limit is reached the
// wait returns false (it does not trap or spin on), the kernel ORs its bit into
// the device status word and exits normally.

#include "kernels.h"
#include "tc_common.cuh"

namespace trifast {
namespace {
using namespace tc;

__global__ void wait_probe_kernel(long long limit_cycles, unsigned int* status) {
  __shared__ __align__(8) unsigned long long barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&barrier), 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  (void)mbar_wait_limit(smem_u32(&barrier), 0, &abort_flag, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag) atomicOr(status, (unsigned int)kStatusTimeoutProbe);
}

}  // namespace

cudaError_t wait_probe(long long limit_cycles, unsigned int* status, cudaStream_t s) {
  wait_probe_kernel<<<1, 32, 0, s>>>(limit_cycles, status);
  return cudaGetLastError();
}

}  // namespace trifast

// Self-test of the bounded mbarrier wait every kernel of this library relies on.
//
// All device-side waits go through mbar_wait (ptx.cuh): a spin on mbarrier.try_wait with an iteration
// limit, after which the waiting code stores a DeviceStatus code in the caller's status word and leaves
// its loop, so a protocol mistake ends a kernel instead of hanging the GPU.  In a correct run no wait
// ever expires, so that path would otherwise never execute.  The kernel below runs it on purpose in the
// only harmless way: one thread waits, with a short limit, on a barrier that nobody arrives at; the wait
// gives up, the thread stores kWaitMiscTimeout and the kernel returns normally.  Nothing traps and the
// context stays usable.  The reference's precedent for a bounded wait is
// _tma_mbarrier_try_wait_parity(ptr, phase, time_limit) (src/nvidia/flash_attn/sm120/attention_cutedsl.py:2434).
#include "atrex_fa_sm100.h"
#include "fa_kernels.cuh"
#include "ptx.cuh"

namespace atrex_sm100 {
namespace {

__global__ void atrex_sm100_selftest_bounded_wait_kernel(int32_t* status, int32_t* result, uint32_t limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool arrived = mbar_spin(&bar, 0, limit);   // phase 0 never completes: there is no arrival
    if (!arrived && status != nullptr) atomicExch(status, (int)kWaitMiscTimeout);
    if (result != nullptr) *result = arrived ? 1 : 0;
  }
}

}  // namespace
}  // namespace atrex_sm100

extern "C" int atrex_fa_sm100_selftest_bounded_wait(int32_t* device_status, int32_t* result, uint32_t spin_limit,
                                                    void* stream) {
  using namespace atrex_sm100;
  if (result == nullptr || spin_limit == 0 || spin_limit > (1u << 16)) return ATREX_FA_INVALID_VALUE;
  const cudaError_t e = launch_kernel(atrex_sm100_selftest_bounded_wait_kernel, dim3(1), dim3(32), 0,
                                      static_cast<cudaStream_t>(stream), device_status, result, spin_limit);
  return e == cudaSuccess ? ATREX_FA_OK : ATREX_FA_CUDA_ERROR;
}

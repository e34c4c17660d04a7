// Self-test of the bounded barrier wait (sm_100a).
//
// The attention kernels never spin without a limit: tc::mbar_wait gives up after a
// time limit, the CTA records a status bit and returns, and the host raises from the
// status word.  This file exercises exactly that routine on a hardware barrier that
// nothing arrives at, with a limit of the caller's choosing (milliseconds instead of
// the kernels' 2 s), so the abort path can be tested without faulting, trapping or
// hanging the GPU.  No counterpart in the reference.
#include "tc.cuh"

namespace ulm {
namespace {

__global__ void __launch_bounds__(64)
wait_timeout_kernel(uint64_t limit_ns, uint32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  __shared__ uint32_t fail_bits;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
    fail_bits = 0;
    tc::fence_mbar_init();
  }
  __syncthreads();
  // warp 0: lane 0 waits for a phase that never completes; warp 1 waits too and must leave as soon
  // as warp 0 has raised the abort flag (or on its own limit)
  if ((threadIdx.x & 31) == 0) {
    if (!tc::mbar_wait(&bar, 0, &abort_flag, limit_ns)) atomicOr(&fail_bits, (uint32_t)ULM_STATUS_TIMEOUT_LOAD);
  }
  __syncthreads();
  if (threadIdx.x == 0 && fail_bits && status) atomicOr(status, fail_bits);
}

}  // namespace
}  // namespace ulm

extern "C" int ulm_selftest_wait_timeout(uint64_t limit_ns, uint32_t* status_dev, void* stream) {
  using namespace ulm;
  if (limit_ns < 1 || limit_ns > 100000000ull) return fail(ULM_ERR_ARG, "ulm_selftest_wait_timeout: limit_ns must be in [1, 100000000]");
  if (!status_dev) return fail(ULM_ERR_ARG, "ulm_selftest_wait_timeout: null status word");
  wait_timeout_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(limit_ns, status_dev);
  return check_launch("ulm_selftest_wait_timeout");
}

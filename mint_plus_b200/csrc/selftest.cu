// Self-test of the bounded-wait error path: a kernel with the set-up of the tensor-core kernels (mbarrier, TMEM
// allocation, role split) whose consumer waits on a barrier that no one ever completes.  The wait gives up after the
// limit the caller names, records its code in *dev_status, the roles unwind, TMEM is released and the kernel returns:
// the very path a lost copy or a missed arrival would take in the attention and GEMM kernels, exercised without one.
#include "common.cuh"
#include "ptx.cuh"

namespace mintb {

using namespace ptx;

constexpr int kSelftestCode = 0x901;

__global__ void __launch_bounds__(64) selftest_wait_kernel(unsigned long long limit_ns, int* status, int* trail) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, 32); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_slot;
  bool ok = true;
  if (warp == 0 && lane == 0) {
    ok = mbar_wait_limit(&bar, 0, status, kSelftestCode, limit_ns);   // phase 0 never completes: nothing arrives on `bar`
    if (trail != nullptr) trail[0] = ok ? 1 : 2;                      // 2: the wait gave up and the role went on to unwind
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, 32);
    if (lane == 0 && trail != nullptr) trail[1] = 1;                  // TMEM was released after the failed wait
  }
}

}  // namespace mintb

extern "C" int mintb_selftest_wait(unsigned long long limit_ns, int* dev_status, int* trail, void* stream) {
  using namespace mintb;
  if (dev_status == nullptr || limit_ns == 0 || limit_ns > 1000000000ull) {
    set_error("mintb_selftest_wait: dev_status is required and the limit must lie in (0, 1e9] ns");
    return MINTB_EINVAL;
  }
  selftest_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, dev_status, trail);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("selftest launch: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  return MINTB_OK;
}

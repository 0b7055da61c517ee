// Self-test of the bounded-wait protocol the tcgen05 kernels in this directory share: a wait on an
// mbarrier whose last arrival never comes must give up after its cycle limit, record where it gave up
// in the caller's status word, raise the CTA's abort flag, and let every warp reach the common
// teardown, where the tensor memory the CTA holds is freed. Nothing here faults or spins without
// bound: the kernel returns by itself after at most `limit_cycles` (plus the teardown).
#include "cab_common.cuh"
#include "sm100_primitives.cuh"

namespace {

constexpr int kSelftestWhere = 901;   // the code a timed-out wait of this kernel leaves in *status

__global__ void __launch_bounds__(96, 1) wait_selftest_kernel(int* status, long long limit_cycles, int withhold) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 2);          // two arrivals complete the phase
    abort_flag = 0;
    sm100::mbar_fence_init();
  }
  if (warp == 2) {                      // hold some tensor memory, as the real kernels do
    sm100::tmem_alloc(&tmem_base, 32);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before_sync();
  __syncthreads();
  sm100::tc_fence_after_sync();
  if (warp == 0 && lane == 0) {
    sm100::mbar_arrive(&bar);                       // first arrival
    if (!withhold) sm100::mbar_arrive(&bar);        // the second one is what the test withholds
  } else if (warp == 1) {
    // every lane waits, as the epilogue warps of the GEMM do; on a time-out all of them leave
    sm100::mbar_wait_limited(&bar, 0, &abort_flag, status, kSelftestWhere, limit_cycles);
  }
  // common teardown: reached by every warp whether or not the wait completed
  sm100::tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    sm100::tc_fence_after_sync();
    sm100::tmem_dealloc(tmem_base, 32);
  }
}

}  // namespace

extern "C" int cab_wait_selftest(int* status, long long limit_cycles, int withhold, cudaStream_t stream) {
  if (!status) return CAB_ERR_BAD_ARGUMENT;
  // the limit stays far below anything a watchdog could notice: at most about half a second
  if (limit_cycles <= 0 || limit_cycles > 1000000000LL) return CAB_ERR_BAD_ARGUMENT;
  if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) return CAB_ERR_LAUNCH;
  wait_selftest_kernel<<<1, 96, 0, stream>>>(status, limit_cycles, withhold);
  return cab::launch_status();
}

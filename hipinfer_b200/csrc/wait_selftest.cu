// A kernel whose only work is to let a bounded wait run out, so that the path every tensor-core
// kernel here takes when a wait gives up can be exercised without a fault: a block with the same
// set-up as those kernels (an mbarrier, a tensor-memory allocation, an abort flag in shared
// memory) arms its barrier for bytes that no copy ever delivers, waits with a limit of a few
// thousand polls through the same hb_mbar_wait(), finds the limit reached, raises the status
// word, frees its tensor memory and returns. Nothing is in flight when the block ends. The
// reference's counterpart is the error return of its argument checks (src/api.cu:1827-1839) and
// HI_CHECK (src/hip_compat.h:95-97); it has no bounded waits because it has no asynchronous pipelines.
#include "tc_common.cuh"

__global__ void __launch_bounds__(64) wait_selftest_kernel(int* status, uint32_t polls, int* out) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    hb_mbar_init(&bar, 1);
    hb_fence_barrier_init();
  }
  if (warp == 0) {
    hb_tmem_alloc(&tmem_slot, 32);
    hb_tmem_relinquish();
  }
  __syncthreads();
  if (threadIdx.x == 0) hb_mbar_expect_tx(&bar, 64);      // 64 bytes that nothing will ever bring
  bool ok = true;
  if (threadIdx.x == 32) ok = hb_mbar_wait(&bar, 0, abort_flag, polls);
  __syncthreads();
  if (threadIdx.x == 32) out[0] = ok ? 1 : 0;
  if (threadIdx.x == 0) {
    out[1] = *abort_flag;
    if (*abort_flag) atomicExch(status, 1);
  }
  hb_tc_fence_before();
  __syncthreads();
  if (warp == 0) hb_tmem_dealloc(tmem_slot, 32);
}

// out (2 ints on the device): out[0] = 1 if the wait completed (it cannot), out[1] = the block's abort flag.
HB_EXPORT int hb_wait_selftest(int* status, int polls, int* out, cudaStream_t s) {
  if (!status || !out || polls < 1 || polls > (1 << 16)) HB_FAIL("hb_wait_selftest: status, out and 1 <= polls <= 65536 are needed");
  wait_selftest_kernel<<<1, 64, 0, s>>>(status, (uint32_t)polls, out);
  HB_CHECK_LAUNCH("hb_wait_selftest");
  return 0;
}

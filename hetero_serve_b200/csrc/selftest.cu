// A self-test of the bounded wait every TMA/tcgen05 pipeline of this library relies on.
//
// hs_selftest_wait_timeout launches one warp that initialises an mbarrier nobody will ever
// arrive on and waits on it with `mbar_wait` (the function the kernels use) under a small
// poll limit.  No copy or MMA is in flight, so running out is harmless: the wait gives up,
// ORs HS_STATUS_PIPELINE_TIMEOUT into the status word and the kernel returns; the context
// stays usable.  It shows, without hanging or faulting anything, the path a wrong expect-tx
// count or a lost arrive would take in the real kernels.
#include "tcgen05.cuh"

namespace hs {

__global__ void selftest_wait_kernel(int* status, int* gave_up, uint32_t limit) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(&bar, 0, status, limit);
    *gave_up = ok ? 0 : 1;
  }
}

}  // namespace hs

// status: the engine's status word; gave_up: one int that receives 1 when the wait ran out;
// limit: polls before giving up (1 .. 1,000,000: this is a test of the path, not a timer).
HS_EXPORT int hs_selftest_wait_timeout(int* status, int* gave_up, int limit, void* stream) {
  if (!status || !gave_up) return HS_ERR_ARGUMENT;
  if (limit < 1 || limit > 1000000) return HS_ERR_UNSUPPORTED;
  hs::selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, gave_up, (uint32_t)limit);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

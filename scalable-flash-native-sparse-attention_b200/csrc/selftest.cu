// Self-test of the bounded-wait path shared by the tcgen05 / TMA kernels.
//
// Every pipeline wait in those kernels goes through tc::mbar_wait, which polls a shared-memory barrier a limited number of
// times, then gives up: the kernel ORs a bit into the caller's status word, shortens its later waits and still runs to its
// end.  A healthy pipeline never takes that path, so this entry point exercises it on purpose and safely: one warp waits,
// with a small poll limit, on a barrier that nobody arrives on.  Nothing else is in flight (no bulk copy, no MMA, no tensor
// memory), so the kernel simply returns after `polls` polls with the bit set and the context stays usable.
#include "tc_common.cuh"

namespace nsa {

__global__ void wait_timeout_selftest_kernel(int32_t* status, int polls, int32_t* waits_failed) {
  using namespace tc;
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  int budget = polls;
  int failed = 0;
  if (threadIdx.x == 0) {
    // first wait: runs out after `polls` polls; the second one must then give up after the shortened budget
    if (!mbar_wait(bar, 0, &budget)) ++failed;
    if (!mbar_wait(bar, 0, &budget)) ++failed;
    if (failed && status) atomicOr(status, 512);
    if (waits_failed) *waits_failed = failed * 1000 + budget;
  }
}

}  // namespace nsa

extern "C" int nsa_selftest_wait_timeout(int32_t* status, int32_t polls, int32_t* waits_failed, void* stream) {
  NSA_REQUIRE(status != nullptr, NSA_ERR_BAD_ARG, "selftest_wait_timeout: status word is required");
  NSA_REQUIRE(polls >= 1 && polls <= (1 << 20), NSA_ERR_BAD_ARG, "selftest_wait_timeout: polls=%d out of range [1, 2^20]", polls);
  nsa::wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, polls, waits_failed);
  return nsa::check_launch("selftest_wait_timeout");
}

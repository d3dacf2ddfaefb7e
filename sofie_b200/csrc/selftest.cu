// Self test of the bounded waits every tensor-core kernel of this library is built from.
//
// One CTA allocates tensor memory, initialises an mbarrier that nothing ever arrives on and lets two
// warps wait for it with the same helper the contraction kernels use (umma::mbar_wait), but with a cycle
// limit chosen by the caller instead of the library's one second. The first waiter whose limit runs out
// raises the CTA's abort flag and stores a code in the status word of the stream's context; the second
// waiter leaves through the abort flag; every thread then reaches the common exit, where the tensor
// memory is released. The kernel therefore ends by itself after `limit_cycles` SM clocks, nothing
// faults, and the context stays usable: exactly the path a contraction kernel takes when a copy it
// waits for never completes.
#include "umma.cuh"

namespace sofie {
namespace {

using namespace umma;

constexpr uint32_t kStatusSelfTest = 0x1ff;

__global__ void __launch_bounds__(96, 1) wait_timeout_kernel(uint32_t *status, long long limit_cycles, uint32_t *reached_exit)
{
   __shared__ uint64_t never_bar;
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;
   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   if (threadIdx.x == 0) {
      mbar_init(&never_bar, 1);
      abort_flag = 0;
      fence_mbar_init();
   }
   if (warp == 1) {
      tmem_alloc(&tmem_base_holder, 32);
      tmem_relinquish();
   }
   tc_fence_before();
   __syncthreads();
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;
   if (warp == 0 && lane == 0) {
      // the role whose wait runs out
      (void)mbar_wait(&never_bar, 0, &abort_flag, status, kStatusSelfTest, 0x7e57, limit_cycles);
   } else if (warp == 2 && lane == 0) {
      // a role with the library's own (one second) limit: it leaves because the CTA was aborted
      (void)mbar_wait(&never_bar, 0, &abort_flag, nullptr, kStatusSelfTest, 0x7e58);
   }
   tc_fence_before();
   __syncthreads();
   if (warp == 1) {
      __syncwarp();
      tc_fence_after();
      tmem_dealloc(tmem_base, 32);
   }
   if (threadIdx.x == 0 && reached_exit) *reached_exit = 1u;
}

} // namespace
} // namespace sofie

extern "C" int sofie_cuda_selftest_wait_timeout(void *stream, int64_t limit_cycles, uint32_t *reached_exit_device)
{
   using namespace sofie;
   SOFIE_REQUIRE(limit_cycles > 0 && limit_cycles <= 200000000LL, "limit_cycles must be in (0, 2e8]: this is a test of a short wait");
   cudaStream_t s = as_stream(stream);
   uint32_t *status = device_status_word(s);
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot obtain the status word");
   wait_timeout_kernel<<<1, 96, 0, s>>>(status, (long long)limit_cycles, reached_exit_device);
   SOFIE_LAUNCH_CHECK("wait_timeout_kernel");
   return SOFIE_CUDA_OK;
}

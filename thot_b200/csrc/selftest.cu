// Self-test of the bounded wait that every bulk-async kernel in this library relies on.
//
// A one-CTA kernel waits, with the same mbar_wait_bounded the norm and gather kernels use, on a
// shared-memory barrier that nothing ever completes.  The wait must give up after `cycle_limit`
// SM cycles (about a millisecond in the test), record a code in the device status word and let
// the kernel return normally, which is what turns a mis-programmed copy into an error code
// instead of a hung GPU.  Nothing here faults, traps or spins without a limit.
#include "launchers.h"

namespace nb2 {

__global__ void __launch_bounds__(64)
bounded_wait_selftest_kernel(unsigned int* status, long long cycle_limit, long long* waited_cycles) {
    __shared__ uint64_t never_completes;
    __shared__ int gave_up;
    if (threadIdx.x == 0) {
        mbar_init(&never_completes, 1);          // one arrival is expected and none will come
        gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long t0 = clock64();
    const bool arrived = mbar_wait_bounded(&never_completes, 0u, &gave_up, kStatusSelfTest, status, cycle_limit);
    if (threadIdx.x == 0 && waited_cycles != nullptr) *waited_cycles = arrived ? -1 : clock64() - t0;
}

}  // namespace nb2

using namespace nb2;

extern "C" int nb2_selftest_bounded_wait(int64_t cycle_limit, int64_t* waited_cycles, void* stream) {
    NB2_REQUIRE(cycle_limit > 0 && cycle_limit <= 2000000000LL, NB2_ERR_SHAPE,
                "bounded-wait self-test: cycle_limit=%lld must be in (0, 2e9]", (long long)cycle_limit);
    unsigned int* status = device_status_ptr();
    if (status == nullptr) return cuda_status(cudaGetLastError(), "device status word lookup");
    bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, (long long)cycle_limit, (long long*)waited_cycles);
    return cuda_status(cudaGetLastError(), "bounded-wait self-test launch");
}

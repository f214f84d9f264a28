// Self-test of the bounded-wait convention the pipelined kernels rely on: a one-warp kernel waits on an
// mbarrier that nothing ever arrives on, with a short limit; the wait gives up, the site code lands in the
// host-visible error word, the kernel returns normally and the next synchronising call reports it. Nothing
// faults, traps or hangs: the context stays usable.
#include "common.h"
#include "ptx_utils.cuh"
#include "tma_utils.cuh"

namespace kutacc {
namespace dev {
namespace {

__global__ void wait_timeout_kernel(int *err, long long limit_clocks, int code)
{
    __shared__ uint64_t bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_barrier_init();
    }
    __syncthreads();
    // phase 0 never completes: nobody arrives
    mbar_wait_limit(b, 0u, err, code, limit_clocks);
}

}  // namespace
}  // namespace dev
}  // namespace kutacc

extern "C" int kutacc_b200_selftest_wait_timeout(int64_t limit_microseconds)
{
    using namespace kutacc;
    if (limit_microseconds < 1) limit_microseconds = 1;
    if (limit_microseconds > 100000) limit_microseconds = 100000;      // never more than 0.1 s
    dev::KernelErrorWord &ew = dev::kernel_error_word();
    if (ew.device == nullptr) return -1;
    dev::wait_timeout_kernel<<<1, 32, 0, (cudaStream_t)runtime().stream>>>(ew.device, limit_microseconds * 2000LL, 0x5e1f);
    count_launch();
    end_of_call();               // synchronous mode: reports "a device-side wait ran out of time (site 24095)"
    return 0;
}

// Self-test of the path by which a kernel reports that one of its bounded waits ran out.
//
// Every wait of the tcgen05 kernels on an mbarrier is bounded: after a fixed number of polls the waiting
// role raises the library's error word, lets go of what it holds and returns, and the host finds the word
// set when it reads the step's results (tma_host.cu: tff_error_word_to_host_async, tff_kernel_error).  In a
// correct run that never happens, so nothing would ever exercise the path from the word to the caller.
// This launcher runs the same wait (tc5::mbar_wait_limit) on a barrier of its own: with ``arrive`` = 1 one
// arrival completes the phase and the wait returns at once; with ``arrive`` = 0 nothing ever arrives, the
// wait gives up after ``max_polls`` polls (a few thousand: some tens of microseconds) and raises the word.
// The kernel always returns; it holds no tensor memory and has no copies in flight.
#include "tcgen05.cuh"

namespace {
__global__ void bounded_wait_selftest_kernel(int* error_flag, unsigned max_polls, int arrive) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = tc5::smem_u32(&bar);
    if (threadIdx.x == 0) {
        tc5::mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (arrive) tc5::mbar_arrive(b);
        tc5::mbar_wait_limit(b, 0, error_flag, max_polls);
    }
}
}  // namespace

// max_polls is clamped to [1, 2^20] so that the launch ends within a fraction of a second whatever it is given.
TFF_API int tff_selftest_bounded_wait(int arrive, int max_polls, cudaStream_t stream) {
    int* flag = tff_device_error_flag();
    if (!flag) return TFF_ERR_LAUNCH;
    unsigned polls = max_polls < 1 ? 1u : (max_polls > (1 << 20) ? (1u << 20) : (unsigned)max_polls);
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(flag, polls, arrive ? 1 : 0);
    return tff_launch_status();
}

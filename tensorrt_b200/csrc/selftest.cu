// Self-test of the bounded device wait that every tensor-core kernel of this library relies on: one CTA waits, with
// the product's own wait routine, on an mbarrier that nothing ever arrives at. The wait has to give up after the given
// time, record its code, and the kernel has to take the same way out as the product kernels (abort flag, drain,
// status word) and return - leaving the context usable for the next launch. Nothing here traps, faults or spins
// without a limit.
#include "sm100.cuh"

namespace b200
{
namespace
{

__global__ void __launch_bounds__(64, 1) waitExpiryKernel(uint64_t const limitNs, uint32_t* statusWord, uint32_t* polled)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abortWord;
    volatile uint32_t* abortFlag = &abortWord;
    if (threadIdx.x == 0)
    {
        mbarInit(&bar, 1);
        *abortFlag = 0;
        fenceBarrierInit();
    }
    __syncthreads();
    if (threadIdx.x == 0)
    {
        // the barrier's first phase never completes: no thread arrives and no copy is bound to it
        bool const ok = mbarWaitSlow(smemAddr(&bar), 0, abortFlag, kWaitTmaFull, limitNs);
        if (polled)
            *polled = ok ? 1u : 0u;
    }
    else if (threadIdx.x == 32)
    {
        // a second waiter, as in the product kernels: it sees the abort flag set by the first and returns early
        mbarWaitSlow(smemAddr(&bar), 0, abortFlag, kWaitStageFree, limitNs * 4);
    }
    __syncthreads();
    uint32_t const aborted = *abortFlag;
    if (aborted != 0)
    {
        uint64_t const t0 = globalTimerNs();
        while (globalTimerNs() - t0 < 100000ull)
            __nanosleep(1000);
        if (threadIdx.x == 0 && statusWord)
            atomicMax(statusWord, aborted);
    }
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int32_t bert_b200_selftest_wait_expiry(void* stream, int64_t limit_ns, uint32_t* status_word, uint32_t* completed)
{
    B200_REQUIRE(status_word != nullptr, "selftest_wait_expiry: null status word");
    B200_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ll, "selftest_wait_expiry: limit must be between 1 ns and 100 ms, got %lld",
        static_cast<long long>(limit_ns));
    waitExpiryKernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint64_t>(limit_ns), status_word, completed);
    return checkLaunch("waitExpiryKernel");
}

// Measures what the tensor pipe of this GPU sustains for the MMA shape the FC kernels issue: every SM pair runs a
// chain of tcgen05.mma.cta_group::2 (256 x 256 x 32 bytes of K, INT8 or FP16) on operands that already sit in shared
// memory, with no loads, no epilogue and no other warps competing for issue slots. The result is the denominator of the
// INT8 roofline (no vendor library routine is involved, and no nominal figure).
#include "sm100.cuh"

namespace b200
{
namespace
{

constexpr int kProbeThreads = 128;
constexpr int kTileBytes = 128 * 128; // 128 rows of 128 bytes: this CTA's half of A, and its half of B
constexpr int kProbeSmem = 2 * kTileBytes + 64 + 1024;

template <bool kInt8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kProbeThreads, 1) mmaRateProbeKernel(int32_t const groups, uint32_t* statusWord)
{
    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + kTileBytes;
    uint64_t* done = reinterpret_cast<uint64_t*>(smem + 2 * kTileBytes);
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(done + 1);
    volatile uint32_t* abortFlag = tmemSlot + 1;
    int const warp = threadIdx.x >> 5;
    bool const leader = clusterCtaRank() == 0;

    // operands: a fixed pattern of small values (FP16: finite numbers around one; INT8: bytes), not zeros - an idle
    // datapath would flatter the clock under the power limit
    for (int i = threadIdx.x; i < 2 * kTileBytes / 4; i += kProbeThreads)
    {
        uint32_t const h = static_cast<uint32_t>(i) * 2654435761u + blockIdx.x;
        reinterpret_cast<uint32_t*>(smem)[i] = kInt8 ? h : (0x3c003c00u | (h & 0x03ff03ffu));
    }
    if (threadIdx.x == 0)
    {
        mbarInit(done, 1);
        *abortFlag = 0;
        fenceBarrierInit();
    }
    fenceProxyAsync();
    if (warp == 1)
        tmemAllocPair(tmemSlot, 256);
    tcFenceBefore();
    __syncthreads();
    clusterSync();
    tcFenceAfter();
    uint32_t const tmemBase = *tmemSlot;

    if (leader && threadIdx.x == 0)
    {
        constexpr uint32_t kIdesc = makeInstrDesc(kInt8 ? 2u : 1u, kInt8 ? 1u : 0u, 0u, 0u, 256u, 256u);
        uint64_t const desc = makeSmemDesc(0, 16, 1024, kSwizzle128B);
        uint32_t const hi = static_cast<uint32_t>(desc >> 32);
        uint32_t const aLo = static_cast<uint32_t>(desc) + (smemAddr(sA) >> 4);
        uint32_t const bLo = static_cast<uint32_t>(desc) + (smemAddr(sB) >> 4);
        mmaPairLoHi<kInt8, false>(tmemBase, aLo, bLo, hi, kIdesc);
        for (int32_t g = 0; g < groups; ++g)
        {
            // one 128-byte K block = four MMAs of 32 bytes of K each, as in the FC kernels' inner loop
            mmaPairLoHi<kInt8, true>(tmemBase, aLo, bLo, hi, kIdesc);
            mmaPairLoHi<kInt8, true>(tmemBase, aLo + 2, bLo + 2, hi, kIdesc);
            mmaPairLoHi<kInt8, true>(tmemBase, aLo + 4, bLo + 4, hi, kIdesc);
            mmaPairLoHi<kInt8, true>(tmemBase, aLo + 6, bLo + 6, hi, kIdesc);
        }
        tcCommitPair(done, 3); // one arrival in each CTA of the pair once every MMA has completed
    }
    if (threadIdx.x == 0)
    {
        if (!mbarWait(done, 0, abortFlag, kWaitAccFull) && statusWord)
            atomicMax(statusWord, kWaitAccFull);
    }
    __syncthreads();
    tcFenceBefore();
    clusterSync();
    if (warp == 1)
    {
        __syncwarp();
        tcFenceAfter();
        tmemFreePair(tmemBase, 256);
    }
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int32_t bert_b200_probe_mma_rate(void* stream, int32_t type_id, int32_t k_blocks, uint32_t* status_word, float* tera_ops_host)
{
    B200_REQUIRE(tera_ops_host != nullptr, "probe_mma_rate: null result pointer");
    B200_REQUIRE(type_id == BERT_B200_FP16 || type_id == BERT_B200_INT8, "probe_mma_rate: type_id %d", type_id);
    B200_REQUIRE(k_blocks > 0 && k_blocks <= (1 << 22), "probe_mma_rate: k_blocks %d", k_blocks);
    auto s = static_cast<cudaStream_t>(stream);
    int const pairs = smCount() / 2;
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "probe_mma_rate: cudaEventCreate failed");
    auto launch = [&](int32_t groups) -> cudaError_t {
        if (type_id == BERT_B200_INT8)
        {
            cudaFuncSetAttribute(mmaRateProbeKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem);
            mmaRateProbeKernel<true><<<2 * pairs, kProbeThreads, kProbeSmem, s>>>(groups, status_word);
        }
        else
        {
            cudaFuncSetAttribute(mmaRateProbeKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem);
            mmaRateProbeKernel<false><<<2 * pairs, kProbeThreads, kProbeSmem, s>>>(groups, status_word);
        }
        return cudaPeekAtLastError();
    };
    cudaError_t e = launch(k_blocks / 8 + 1); // warm-up (module load, clocks)
    if (e == cudaSuccess)
        e = cudaEventRecord(e0, s);
    if (e == cudaSuccess)
        e = launch(k_blocks);
    if (e == cudaSuccess)
        e = cudaEventRecord(e1, s);
    if (e == cudaSuccess)
        e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess)
        e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "probe_mma_rate: %s", cudaGetErrorString(e));
    // per MMA: 2 x 256 x 256 x K operations, K = 32 (INT8) or 16 (FP16) elements
    double const perMma = 2.0 * 256 * 256 * (type_id == BERT_B200_INT8 ? 32 : 16);
    *tera_ops_host = static_cast<float>(perMma * 4.0 * k_blocks * pairs / (ms * 1e-3) / 1e12);
    return BERT_B200_OK;
}

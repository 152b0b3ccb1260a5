// Fully connected layer on the sm_100a tensor cores: C = epilogue(A * Wt^T).
//
// Replaces the cublasLtMatmul call of the reference FC plugin (plugin/fcPlugin/fcPlugin.cpp:551-610)
// and the separate bias / GELU / quantise layers that follow it in the reference graph.
//
// Design (one persistent CTA per SM, 18 warps, warp specialised):
//   warp 0  : TMA producer - A[128 x 128B] and Wt[BLOCK_N x 128B] tiles, 128-byte swizzle, into a
//             STAGES-deep shared-memory ring guarded by full/empty mbarriers.
//   warp 1  : allocates all 512 TMEM columns, then one lane issues tcgen05.mma (UMMA 128 x BLOCK_N x 16
//             for FP16 / x 32 for INT8) with the accumulator in TMEM; tcgen05.commit releases ring
//             stages and publishes finished accumulators.
//   warps 2-17: epilogue (four warps per TMEM lane quadrant, each owning every fourth 32-column chunk) -
//             tcgen05.ld the accumulator (double buffered, so tile i+1's main loop overlaps tile i's
//             epilogue), scale / bias / erf-GELU / quantise, 128-bit stores.
// Every mbarrier wait is bounded (see sm100.cuh); on expiry the CTA drains, frees TMEM and exits,
// and the status word tells the host.
#include "sm100.cuh"

#include <mutex>

namespace b200
{

int32_t fcF32(bert_b200_fc_params const& p, cudaStream_t stream);

namespace
{

constexpr int kBlockM = 128;
constexpr int kRowBytes = 128; // one swizzle span = BLOCK_K * sizeof(In)
constexpr int kTmemCols = 512;
constexpr int kEpilogueWarps = 16;
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kFcThreads = 64 + kEpilogueThreads;

struct FcArgs
{
    int64_t M, N, K;
    void* C;
    int64_t ldc;
    float const* bias;
    int32_t act;
    float alpha;
    float outScale;
    uint32_t* statusWord;
    float qLo, qHi; // clamp bounds -128 / outScale and 127 / outScale for quantised results
};

template <int BLOCK_N>
struct FcSmem
{
    static constexpr int kStages = BLOCK_N == 256 ? 4 : 6;
    static constexpr int kABytes = kBlockM * kRowBytes;
    static constexpr int kBBytes = BLOCK_N * kRowBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierOff = kStages * kStageBytes;
    // full[kStages], empty[kStages], accFull[2], accEmpty[2], tmem base, abort flag
    static constexpr int kTotal = kBarrierOff + (2 * kStages + 4) * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024; // slack for 1024-byte alignment of the ring
};

// erf-GELU through a fitted tanh form: gelu(x) = x/2 * (1 + tanh(x * (c1 + c3 x^2 + c5 x^4))), x^2 clamped at 64.
// The three coefficients are a minimax fit against 0.5 x (1 + erf(x / sqrt 2)) on [-9, 9]: |error| <= 2.6e-5
// (the classic 0.044715 cubic form is off by 4.7e-4). On top comes the error of the hardware tanh.approx
// (about 2^-11 relative), i.e. at most ~2.5e-4 |x| absolute - below FP16 resolution of the result and about
// 1 % of an INT8 step. Cost: 5 FMA-pipe operations and one MUFU operation per value.
constexpr float kGeluC1 = 7.97507884e-01f;
constexpr float kGeluC3 = 3.70056460e-02f;
constexpr float kGeluC5 = -3.51516788e-04f;

__device__ __forceinline__ float geluInner(float x)
{
    float const x2 = fminf(x * x, 64.f);
    return x * fmaf(fmaf(kGeluC5, x2, kGeluC3), x2, kGeluC1);
}

__device__ __forceinline__ float tanhApprox(float x)
{
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// scale * gelu(x); `halfScale` = scale / 2
__device__ __forceinline__ float geluErf(float x, float halfScale)
{
    float const h = x * halfScale;
    return fmaf(h, tanhApprox(geluInner(x)), h);
}

// Two values at once for results that are quantised to INT8 right away: the whole tanh argument is formed in packed
// FP16 with the classic cubic x * (0.79788456 + 0.035677408 x^2) (|error| of that GELU form <= 4.7e-4, FP16 argument
// and tanh.approx.f16x2 add about 3e-4 |x|), together a few hundredths of an INT8 step at most; the product with x
// stays in FP32. 5.5 instructions per value instead of 9, and one MUFU operation per pair.
__device__ __forceinline__ void geluErfPair(float& a, float& b, float halfScale)
{
    uint32_t x, t;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(x) : "f"(b), "f"(a));
    __half2 const xh = *reinterpret_cast<__half2 const*>(&x);
    __half2 const poly = __hfma2(__hmul2(xh, xh), __float2half2_rn(0.035677408f), __float2half2_rn(0.79788456f));
    __half2 const u = __hmul2(xh, poly);
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(t) : "r"(*reinterpret_cast<uint32_t const*>(&u)));
    float2 const tf = __half22float2(*reinterpret_cast<__half2 const*>(&t));
    float const ha = a * halfScale, hb = b * halfScale;
    a = fmaf(ha, tf.x, ha);
    b = fmaf(hb, tf.y, hb);
}

// What is left to do to a value when it is quantised: multiply by s, with the clamp done before at [lo, hi].
struct QuantStep
{
    float s, lo, hi;
    bool useConvert; // round with cvt.rni.sat (conversion unit) instead of clamp + FMA
    bool unitScale;  // s == 1: the values are already scaled
};

template <typename Out>
__device__ __forceinline__ void storeChunk32(Out* dst, float const (&v)[32], QuantStep const& q, int validCols);

template <>
__device__ __forceinline__ void storeChunk32<__half>(__half* dst, float const (&v)[32], QuantStep const&, int validCols)
{
#pragma unroll
    for (int g = 0; g < 4; ++g)
    {
        if (g * 8 < validCols)
        {
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                f[j] = v[g * 8 + j];
            *reinterpret_cast<uint4*>(dst + g * 8) = packHalf8(f);
        }
    }
}

template <>
__device__ __forceinline__ void storeChunk32<int8_t>(int8_t* dst, float const (&v)[32], QuantStep const& q, int validCols)
{
#pragma unroll
    for (int g = 0; g < 2; ++g)
    {
        if (g * 16 < validCols)
        {
            uint4 o;
            uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                w[j] = packChar4Scaled(v[g * 16 + 4 * j], v[g * 16 + 4 * j + 1], v[g * 16 + 4 * j + 2], v[g * 16 + 4 * j + 3], q.s, q.lo, q.hi);
            *reinterpret_cast<uint4*>(dst + g * 16) = o;
        }
    }
}

// alpha / bias / activation for 32 accumulator columns of one row. Returns what the quantising store still has to do:
// after GELU the values are already multiplied by out_scale (it rides on the 1/2 of the GELU), otherwise the scale is
// left to the store, which folds it into its rounding FMA.
template <bool kInt8, typename Out>
__device__ __forceinline__ QuantStep fcEpilogueMath(uint32_t const (&r)[32], float (&v)[32], FcArgs const& args, int64_t col, int validCols)
{
    constexpr bool kQuant = sizeof(Out) == 1;
    bool const foldScale = kQuant && args.bias == nullptr && args.act != BERT_B200_ACT_GELU_ERF;
    if (args.bias)
    {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
        {
            float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
            if (j < validCols)
                b = __ldg(reinterpret_cast<float4 const*>(args.bias + col + j));
            float const bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                float const a = kInt8 ? static_cast<float>(static_cast<int32_t>(r[j + i])) : __uint_as_float(r[j + i]);
                v[j + i] = fmaf(a, args.alpha, bb[i]);
            }
        }
    }
    else
    {
        // nothing between the accumulator and the quantisation: one multiply by alpha * out_scale
        float const a1 = foldScale ? args.alpha * args.outScale : args.alpha;
#pragma unroll
        for (int j = 0; j < 32; ++j)
        {
            float const a = kInt8 ? static_cast<float>(static_cast<int32_t>(r[j])) : __uint_as_float(r[j]);
            v[j] = a * a1;
        }
    }
    if (args.act == BERT_B200_ACT_GELU_ERF)
    {
        if (kQuant)
        {
            float const halfScale = 0.5f * args.outScale;
#pragma unroll
            for (int j = 0; j < 32; j += 2)
                geluErfPair(v[j], v[j + 1], halfScale);
        }
        else
        {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                v[j] = geluErf(v[j], 0.5f);
        }
        return QuantStep{1.f, -128.f, 127.f, false, true};
    }
    if (foldScale)
        return QuantStep{1.f, -128.f, 127.f, true, true};
    return QuantStep{args.outScale, args.qLo, args.qHi, true, false};
}

// ... then 128-bit stores straight from the registers of the row's thread (one-CTA kernel).
template <bool kInt8, typename Out>
__device__ __forceinline__ void fcEpilogueChunk(uint32_t const (&r)[32], FcArgs const& args, Out* C, int64_t row, int64_t col,
    int validCols)
{
    float v[32];
    QuantStep const q = fcEpilogueMath<kInt8, Out>(r, v, args, col, validCols);
    if (row < args.M)
        storeChunk32<Out>(C + row * args.ldc + col, v, q, validCols);
}

// ... or into a [32 rows x 32 columns] staging tile in shared memory, laid out the way a TMA store with the 32-byte
// (INT8) or 64-byte (FP16) swizzle expects it: row `lane`, 16-byte piece c at (c ^ f(lane)) - which also spreads the
// 32 lanes' 128-bit stores over all banks.
template <typename Out>
__device__ __forceinline__ void stageChunk32(uint8_t* tile, int lane, float const (&v)[32], QuantStep const& q);

template <>
__device__ __forceinline__ void stageChunk32<__half>(uint8_t* tile, int lane, float const (&v)[32], QuantStep const&)
{
    uint8_t* const rowPtr = tile + lane * 64;
    int const x = (lane >> 1) & 3;
#pragma unroll
    for (int g = 0; g < 4; ++g)
    {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            f[j] = v[g * 8 + j];
        *reinterpret_cast<uint4*>(rowPtr + ((g ^ x) << 4)) = packHalf8(f);
    }
}

template <>
__device__ __forceinline__ void stageChunk32<int8_t>(uint8_t* tile, int lane, float const (&v)[32], QuantStep const& q)
{
    uint8_t* const rowPtr = tile + lane * 32;
    int const x = (lane >> 2) & 1;
#pragma unroll
    for (int g = 0; g < 2; ++g)
    {
        uint4 o;
        uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            // Without GELU the conversion unit is idle and issue slots are scarce: multiply + saturating convert.
            // With GELU the unit is busy with tanh: clamp + rounding FMA on the FMA pipe instead. Same results.
            w[j] = q.useConvert
                ? (q.unitScale ? packChar4Cvt(v[g * 16 + 4 * j], v[g * 16 + 4 * j + 1], v[g * 16 + 4 * j + 2], v[g * 16 + 4 * j + 3])
                               : packChar4Cvt(v[g * 16 + 4 * j], v[g * 16 + 4 * j + 1], v[g * 16 + 4 * j + 2], v[g * 16 + 4 * j + 3], q.s))
                : packChar4Scaled(v[g * 16 + 4 * j], v[g * 16 + 4 * j + 1], v[g * 16 + 4 * j + 2], v[g * 16 + 4 * j + 3], q.s, q.lo, q.hi);
        }
        *reinterpret_cast<uint4*>(rowPtr + ((g ^ x) << 4)) = o;
    }
}

template <typename In, int BLOCK_N, typename Out>
__global__ void __launch_bounds__(kFcThreads, 1)
    fcTcgen05Kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, FcArgs const args)
{
    using L = FcSmem<BLOCK_N>;
    constexpr bool kInt8 = sizeof(In) == 1;
    constexpr int kBlockK = kRowBytes / sizeof(In);
    constexpr int kUmmaKBytes = 32; // UMMA K = 16 halves or 32 bytes
    constexpr uint32_t kIdesc
        = makeInstrDesc(kInt8 ? 2u : 1u, kInt8 ? 1u : 0u, 0u, 0u, static_cast<uint32_t>(kBlockM), static_cast<uint32_t>(BLOCK_N));

    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + L::kStages * L::kABytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarrierOff);
    uint64_t* empty = full + L::kStages;
    uint64_t* accFull = empty + L::kStages;
    uint64_t* accEmpty = accFull + 2;
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(accEmpty + 2);
    volatile uint32_t* abortFlag = tmemSlot + 1;

    int const warp = threadIdx.x >> 5;
    int const lane = threadIdx.x & 31;

    if (threadIdx.x == 0)
    {
        for (int i = 0; i < L::kStages; ++i)
        {
            mbarInit(&full[i], 1);
            mbarInit(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i)
        {
            mbarInit(&accFull[i], 1);
            mbarInit(&accEmpty[i], kEpilogueThreads);
        }
        *abortFlag = 0;
        fenceBarrierInit();
        prefetchTensorMap(&mapA);
        prefetchTensorMap(&mapB);
    }
    if (warp == 1)
        tmemAlloc(tmemSlot, kTmemCols);
    tcFenceBefore();
    __syncthreads();
    tcFenceAfter();
    uint32_t const tmemBase = *tmemSlot;

    int64_t const mBlocks = (args.M + kBlockM - 1) / kBlockM;
    int64_t const nBlocks = (args.N + BLOCK_N - 1) / BLOCK_N;
    int64_t const numTiles = mBlocks * nBlocks;
    int const kBlocks = static_cast<int>((args.K + kBlockK - 1) / kBlockK);

    if (warp == 0)
    {
        if (lane == 0)
        {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < numTiles && ok; tile += gridDim.x)
            {
                int32_t const m0 = static_cast<int32_t>(tile / nBlocks) * kBlockM;
                int32_t const n0 = static_cast<int32_t>(tile % nBlocks) * BLOCK_N;
                for (int kb = 0; kb < kBlocks; ++kb)
                {
                    if (!mbarWait(&empty[stage], phase ^ 1u, abortFlag, kWaitStageFree))
                    {
                        ok = false;
                        break;
                    }
                    mbarArriveExpectTx(&full[stage], L::kStageBytes);
                    tmaLoad2d(sA + stage * L::kABytes, &mapA, &full[stage], kb * kBlockK, m0);
                    tmaLoad2d(sB + stage * L::kBBytes, &mapB, &full[stage], kb * kBlockK, n0);
                    if (++stage == L::kStages)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            // Tail: wait until the MMA side has released every stage, so that no tcgen05.commit
            // arrival is still in flight towards this CTA's shared memory when it exits.
            for (int i = 0; i < L::kStages && ok; ++i)
            {
                ok = mbarWait(&empty[stage], phase ^ 1u, abortFlag, kWaitStageFree);
                if (++stage == L::kStages)
                {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    }
    else if (warp == 1)
    {
        if (lane == 0)
        {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t accPhase = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < numTiles && ok; tile += gridDim.x)
            {
                if (!mbarWait(&accEmpty[acc], accPhase ^ 1u, abortFlag, kWaitAccFree))
                    break;
                tcFenceAfter();
                uint32_t const dTmem = tmemBase + static_cast<uint32_t>(acc * BLOCK_N);
                for (int kb = 0; kb < kBlocks; ++kb)
                {
                    if (!mbarWait(&full[stage], phase, abortFlag, kWaitTmaFull))
                    {
                        ok = false;
                        break;
                    }
                    tcFenceAfter();
                    uint32_t const aBase = smemAddr(sA + stage * L::kABytes);
                    uint32_t const bBase = smemAddr(sB + stage * L::kBBytes);
#pragma unroll
                    for (int k = 0; k < kRowBytes / kUmmaKBytes; ++k)
                    {
                        uint64_t const aDesc = makeSmemDesc(aBase + k * kUmmaKBytes, 16, 1024, kSwizzle128B);
                        uint64_t const bDesc = makeSmemDesc(bBase + k * kUmmaKBytes, 16, 1024, kSwizzle128B);
                        if (kInt8)
                            mmaI8(dTmem, aDesc, bDesc, kIdesc, (kb | k) != 0);
                        else
                            mmaF16(dTmem, aDesc, bDesc, kIdesc, (kb | k) != 0);
                    }
                    tcCommit(&empty[stage]);
                    if (++stage == L::kStages)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
                tcCommit(&accFull[acc]);
                acc ^= 1;
                if (acc == 0)
                    accPhase ^= 1u;
            }
        }
    }
    else
    {
        int const quad = warp & 3;        // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
        int const part = (warp - 2) >> 2; // four warps share a quadrant; each takes every fourth 32-column chunk
        int acc = 0;
        uint32_t accPhase = 0;
        Out* const C = static_cast<Out*>(args.C);
        for (int64_t tile = blockIdx.x; tile < numTiles; tile += gridDim.x)
        {
            int64_t const m0 = (tile / nBlocks) * kBlockM;
            int64_t const n0 = (tile % nBlocks) * BLOCK_N;
            if (!mbarWait(&accFull[acc], accPhase, abortFlag, kWaitAccFull))
                break;
            tcFenceAfter();
            int64_t const row = m0 + quad * 32 + lane;
            uint32_t const taddr = tmemBase + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll 1
            for (int c = part; c < BLOCK_N / 32; c += kEpilogueWarps / 4) // this warp's 32-column chunks of the tile
            {
                uint32_t r[32];
                tmemLoad32(taddr + c * 32, r);
                tmemLoadWait32(r);
                int64_t const col = n0 + c * 32;
                int const validCols = static_cast<int>(args.N - col < 32 ? args.N - col : 32);
                if (validCols > 0) // warp-uniform
                    fcEpilogueChunk<kInt8, Out>(r, args, C, row, col, validCols);
            }
            tcFenceBefore();
            mbarArrive(&accEmpty[acc]);
            acc ^= 1;
            if (acc == 0)
                accPhase ^= 1u;
        }
    }

    __syncthreads();
    uint32_t const aborted = *abortFlag;
    if (aborted != 0)
    {
        // Give copies / MMAs still in flight a bounded time to land before shared memory and TMEM go away.
        uint64_t const t0 = globalTimerNs();
        while (globalTimerNs() - t0 < 1000000ull)
            __nanosleep(1000);
        if (threadIdx.x == 0 && args.statusWord)
            atomicMax(args.statusWord, aborted);
        __syncthreads();
    }
    if (warp == 1)
    {
        __syncwarp();
        tcFenceAfter();
        tmemFree(tmemBase, kTmemCols);
    }
}

template <typename In, int BLOCK_N, typename Out>
int32_t launchFc(bert_b200_fc_params const& p, cudaStream_t stream)
{
    using L = FcSmem<BLOCK_N>;
    constexpr int kBlockK = kRowBytes / sizeof(In);
    CUtensorMapDataType const dt = sizeof(In) == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mapA, mapB;
    {
        uint64_t const dims[2] = {static_cast<uint64_t>(p.k), static_cast<uint64_t>(p.m)};
        uint64_t const strides[1] = {static_cast<uint64_t>(p.lda) * sizeof(In)};
        uint32_t const box[2] = {static_cast<uint32_t>(kBlockK), static_cast<uint32_t>(kBlockM)};
        int32_t const st = makeTensorMap(&mapA, dt, 2, p.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != BERT_B200_OK)
            return st;
    }
    {
        uint64_t const dims[2] = {static_cast<uint64_t>(p.k), static_cast<uint64_t>(p.n)};
        uint64_t const strides[1] = {static_cast<uint64_t>(p.k) * sizeof(In)};
        uint32_t const box[2] = {static_cast<uint32_t>(kBlockK), static_cast<uint32_t>(BLOCK_N)};
        int32_t const st = makeTensorMap(&mapB, dt, 2, p.wt, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != BERT_B200_OK)
            return st;
    }
    auto kernel = fcTcgen05Kernel<In, BLOCK_N, Out>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "fc: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    int64_t const tiles = ((p.m + kBlockM - 1) / kBlockM) * ((p.n + BLOCK_N - 1) / BLOCK_N);
    int const grid = static_cast<int>(tiles < smCount() ? tiles : smCount());
    FcArgs args{p.m, p.n, p.k, p.c, p.ldc, p.bias, p.activation, p.alpha, p.out_scale, p.status_word,
        p.out_scale > 0.f ? -128.f / p.out_scale : 0.f, p.out_scale > 0.f ? 127.f / p.out_scale : 0.f};
    kernel<<<grid, kFcThreads, L::kDynamic, stream>>>(mapA, mapB, args);
    return checkLaunch("fcTcgen05Kernel");
}


// ------------------------------------------------------------------------------------------------
// Two-CTA variant: a cluster of two CTAs (neighbouring SMs) computes one 256 x BLOCK_N tile with
// tcgen05.mma.cta_group::2. Each CTA loads its own 128 rows of A and its own BLOCK_N/2 rows of Wt, so a pair
// moves (256 + BLOCK_N) rows per k-block instead of 2 x (128 + BLOCK_N): the shared-memory fill bandwidth per SM,
// which bounds the one-CTA kernel, drops by a third and the ring gets deeper (6-8 stages).
//   Leader (cluster rank 0): its MMA lane issues every MMA; its "full" barriers collect the TMA bytes of both
//   CTAs; its "accEmpty" barriers collect the epilogue arrivals of both CTAs. tcgen05.commit multicasts the
//   "stage free" and "accumulator ready" arrivals to both CTAs.
// ------------------------------------------------------------------------------------------------
template <int BLOCK_N>
struct FcPairSmem
{
    static constexpr int kABytes = kBlockM * kRowBytes;            // this CTA's 128 rows of A
    static constexpr int kBBytes = (BLOCK_N / 2) * kRowBytes;      // this CTA's half of the Wt rows
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = BLOCK_N == 256 ? 6 : 8;
    static constexpr int kOutOff = kStages * kStageBytes;          // epilogue staging: kOutWarpBytes per epilogue warp
    static constexpr int kOutWarpBytes = 2048;                     // one FP16 or two INT8 [32 x 32] chunks
    static constexpr int kBarrierOff = kOutOff + kEpilogueWarps * kOutWarpBytes;
    static constexpr int kTotal = kBarrierOff + (2 * kStages + 4) * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
    static_assert(kDynamic <= 232448, "shared memory budget of one CTA");
};

template <typename In, int BLOCK_N, typename Out>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFcThreads, 1)
    fcTcgen05PairKernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
        const __grid_constant__ CUtensorMap mapC, FcArgs const args)
{
    using L = FcPairSmem<BLOCK_N>;
    constexpr bool kInt8 = sizeof(In) == 1;
    constexpr int kBlockK = kRowBytes / sizeof(In);
    constexpr int kUmmaKBytes = 32;
    constexpr int kPairM = 2 * kBlockM;
    constexpr uint32_t kIdesc
        = makeInstrDesc(kInt8 ? 2u : 1u, kInt8 ? 1u : 0u, 0u, 0u, static_cast<uint32_t>(kPairM), static_cast<uint32_t>(BLOCK_N));

    extern __shared__ uint8_t smemRaw[];
    // the dynamic shared memory window starts at the same offset in both CTAs, so this rounding agrees too
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + L::kStages * L::kABytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarrierOff);
    uint64_t* empty = full + L::kStages;
    uint64_t* accFull = empty + L::kStages;
    uint64_t* accEmpty = accFull + 2;
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(accEmpty + 2);
    volatile uint32_t* abortFlag = tmemSlot + 1;

    int const warp = threadIdx.x >> 5;
    int const lane = threadIdx.x & 31;
    uint32_t const rank = clusterCtaRank();
    bool const leader = rank == 0;

    if (threadIdx.x == 0)
    {
        for (int i = 0; i < L::kStages; ++i)
        {
            mbarInit(&full[i], 1);  // the leader's producer arrives (with the byte count of both CTAs)
            mbarInit(&empty[i], 1); // one multicast commit from the leader
        }
        for (int i = 0; i < 2; ++i)
        {
            mbarInit(&accFull[i], 1);
            mbarInit(&accEmpty[i], 2 * kEpilogueWarps); // one lane per epilogue warp of both CTAs (used in the leader only)
        }
        *abortFlag = 0;
        fenceBarrierInit();
        prefetchTensorMap(&mapA);
        prefetchTensorMap(&mapB);
        prefetchTensorMap(&mapC);
    }
    if (warp == 1)
        tmemAllocPair(tmemSlot, kTmemCols);
    tcFenceBefore();
    __syncthreads();
    clusterSync(); // both CTAs' barriers are initialised before any remote arrival or TMA signal
    tcFenceAfter();
    uint32_t const tmemBase = *tmemSlot;
    // set-up done: the next kernel of the stream may start its own; the operands of this one must be complete
    gridDependencyLaunch();
    gridDependencyWait();

    int64_t const mBlocks = (args.M + kPairM - 1) / kPairM;
    int64_t const nBlocks = (args.N + BLOCK_N - 1) / BLOCK_N;
    int64_t const numTiles = mBlocks * nBlocks;
    int const kBlocks = static_cast<int>((args.K + kBlockK - 1) / kBlockK);
    int64_t const firstTile = blockIdx.x / 2;
    int64_t const tileStride = gridDim.x / 2;

    if (warp == 0)
    {
        if (lane == 0)
        {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // running shared-memory addresses of the stage being filled (see mmaPairLoHi for why)
            uint32_t const fullAddr0 = smemAddr(full), emptyAddr0 = smemAddr(empty);
            uint32_t const fullLeader0 = mapaShared(full, 0);
            uint32_t const aAddr0 = smemAddr(sA), bAddr0 = smemAddr(sB);
            uint32_t off8 = 0, aAddr = aAddr0, bAddr = bAddr0;
            for (int64_t tile = firstTile; tile < numTiles && ok; tile += tileStride)
            {
                int32_t const m0 = static_cast<int32_t>(tile / nBlocks) * kPairM + static_cast<int32_t>(rank) * kBlockM;
                int32_t const n0 = static_cast<int32_t>(tile % nBlocks) * BLOCK_N + static_cast<int32_t>(rank) * (BLOCK_N / 2);
                for (int kb = 0; kb < kBlocks; ++kb)
                {
                    if (!mbarWaitAddr(emptyAddr0 + off8, phase ^ 1u, abortFlag, kWaitStageFree))
                    {
                        ok = false;
                        break;
                    }
                    if (leader)
                        mbarArriveExpectTxAddr(fullAddr0 + off8, 2 * L::kStageBytes);
                    tmaLoad2dPairAddr(aAddr, &mapA, fullLeader0 + off8, kb * kBlockK, m0);
                    tmaLoad2dPairAddr(bAddr, &mapB, fullLeader0 + off8, kb * kBlockK, n0);
                    off8 += 8;
                    aAddr += L::kABytes;
                    bAddr += L::kBBytes;
                    if (++stage == L::kStages)
                    {
                        stage = 0;
                        phase ^= 1u;
                        off8 = 0;
                        aAddr = aAddr0;
                        bAddr = bAddr0;
                    }
                }
            }
            // Tail: every stage released, i.e. no commit arrival is still on its way to this CTA.
            for (int i = 0; i < L::kStages && ok; ++i)
            {
                ok = mbarWait(&empty[stage], phase ^ 1u, abortFlag, kWaitStageFree);
                if (++stage == L::kStages)
                {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    }
    else if (warp == 1)
    {
        if (lane == 0 && leader)
        {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t accPhase = 0;
            bool ok = true;
            // descriptor words and barrier addresses of the stage being consumed, kept running (see mmaPairLoHi)
            uint64_t const descZero = makeSmemDesc(0, 16, 1024, kSwizzle128B);
            uint32_t const descHi = static_cast<uint32_t>(descZero >> 32);
            uint32_t const aLo0 = static_cast<uint32_t>(descZero) + (smemAddr(sA) >> 4);
            uint32_t const bLo0 = static_cast<uint32_t>(descZero) + (smemAddr(sB) >> 4);
            uint32_t const fullAddr0 = smemAddr(full), emptyAddr0 = smemAddr(empty);
            uint32_t off8 = 0, aLo = aLo0, bLo = bLo0;
            constexpr uint32_t kStep = kUmmaKBytes >> 4; // descriptor units per UMMA K step
            static_assert(kRowBytes / kUmmaKBytes == 4, "four MMAs per k-block");
            for (int64_t tile = firstTile; tile < numTiles && ok; tile += tileStride)
            {
                if (!mbarWait(&accEmpty[acc], accPhase ^ 1u, abortFlag, kWaitAccFree))
                    break;
                tcFenceAfter();
                uint32_t const dTmem = tmemBase + static_cast<uint32_t>(acc * BLOCK_N);
                for (int kb = 0; kb < kBlocks; ++kb)
                {
                    if (!mbarWaitAddr(fullAddr0 + off8, phase, abortFlag, kWaitTmaFull))
                    {
                        ok = false;
                        break;
                    }
                    tcFenceAfter();
                    if (kb == 0)
                        mmaPairLoHi<kInt8, false>(dTmem, aLo, bLo, descHi, kIdesc);
                    else
                        mmaPairLoHi<kInt8, true>(dTmem, aLo, bLo, descHi, kIdesc);
                    mmaPairLoHi<kInt8, true>(dTmem, aLo + kStep, bLo + kStep, descHi, kIdesc);
                    mmaPairLoHi<kInt8, true>(dTmem, aLo + 2 * kStep, bLo + 2 * kStep, descHi, kIdesc);
                    mmaPairLoHi<kInt8, true>(dTmem, aLo + 3 * kStep, bLo + 3 * kStep, descHi, kIdesc);
                    tcCommitPairAddr(emptyAddr0 + off8, 3);
                    off8 += 8;
                    aLo += L::kABytes >> 4;
                    bLo += L::kBBytes >> 4;
                    if (++stage == L::kStages)
                    {
                        stage = 0;
                        phase ^= 1u;
                        off8 = 0;
                        aLo = aLo0;
                        bLo = bLo0;
                    }
                }
                if (!ok)
                    break;
                tcCommitPair(&accFull[acc], 3);
                acc ^= 1;
                if (acc == 0)
                    accPhase ^= 1u;
            }
        }
    }
    else
    {
        int const quad = warp & 3;
        int const part = (warp - 2) >> 2;
        constexpr int kChunksPerWarp = BLOCK_N / 32 / (kEpilogueWarps / 4);
        constexpr int kChunkBytes = 32 * 32 * static_cast<int>(sizeof(Out));
        constexpr int kBufs = L::kOutWarpBytes / kChunkBytes; // staging tiles of this warp: 2 (INT8) or 1 (FP16)
        uint8_t* const stage0 = smem + L::kOutOff + (warp - 2) * L::kOutWarpBytes;
        int buf = 0;
        int acc = 0;
        uint32_t accPhase = 0;
        for (int64_t tile = firstTile; tile < numTiles; tile += tileStride)
        {
            int64_t const rowBase = (tile / nBlocks) * kPairM + static_cast<int64_t>(rank) * kBlockM + quad * 32;
            int64_t const n0 = (tile % nBlocks) * BLOCK_N;
            if (!mbarWait(&accFull[acc], accPhase, abortFlag, kWaitAccFull))
                break;
            tcFenceAfter();
            uint32_t const taddr = tmemBase + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll
            for (int i = 0; i < kChunksPerWarp; ++i) // this warp's 32-column chunks of the tile
            {
                int const c = part + i * (kEpilogueWarps / 4);
                uint32_t r[32];
                tmemLoad32(taddr + c * 32, r);
                tmemLoadWait32(r);
                if (i == kChunksPerWarp - 1)
                {
                    // The accumulator is in registers: hand the TMEM buffer back before the arithmetic and the store.
                    tcFenceBefore();
                    __syncwarp();
                    if (lane == 0)
                        mbarArriveCluster(mapaShared(&accEmpty[acc], 0)); // the leader's barrier counts both CTAs
                }
                int64_t const col = n0 + c * 32;
                if (col < args.N && rowBase < args.M) // warp-uniform
                {
                    int const validCols = static_cast<int>(args.N - col < 32 ? args.N - col : 32);
                    float v[32];
                    QuantStep const q = fcEpilogueMath<kInt8, Out>(r, v, args, col, validCols);
                    uint8_t* const tileBuf = stage0 + buf * kChunkBytes;
                    if (lane == 0)
                        bulkWaitGroupRead<kBufs - 1>(); // the store that last used this staging tile has read it
                    __syncwarp();
                    stageChunk32<Out>(tileBuf, lane, v, q);
                    fenceProxyAsync();
                    __syncwarp();
                    if (lane == 0)
                    {
                        // rows >= M and columns >= N of the box are clipped by the TMA unit
                        tmaStore2d(&mapC, tileBuf, static_cast<int32_t>(col), static_cast<int32_t>(rowBase));
                        bulkCommitGroup();
                    }
                    buf = buf + 1 == kBufs ? 0 : buf + 1;
                }
            }
            acc ^= 1;
            if (acc == 0)
                accPhase ^= 1u;
        }
        if (lane == 0)
            bulkWaitGroup<0>(); // every store of this warp has left shared memory and reached global memory
    }

    __syncthreads();
    uint32_t const aborted = *abortFlag;
    if (aborted != 0)
    {
        uint64_t const t0 = globalTimerNs();
        while (globalTimerNs() - t0 < 1000000ull)
            __nanosleep(1000);
        if (threadIdx.x == 0 && args.statusWord)
            atomicMax(args.statusWord, aborted);
        __syncthreads();
    }
    tcFenceBefore();
    clusterSync(); // the peer no longer signals barriers of, or reads operands from, this CTA's shared memory
    if (warp == 1)
    {
        __syncwarp();
        tcFenceAfter();
        tmemFreePair(tmemBase, kTmemCols);
    }
}

template <typename In, int BLOCK_N, typename Out>
int32_t launchFcPair(bert_b200_fc_params const& p, cudaStream_t stream)
{
    using L = FcPairSmem<BLOCK_N>;
    constexpr int kBlockK = kRowBytes / sizeof(In);
    CUtensorMapDataType const dt = sizeof(In) == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mapA, mapB;
    {
        uint64_t const dims[2] = {static_cast<uint64_t>(p.k), static_cast<uint64_t>(p.m)};
        uint64_t const strides[1] = {static_cast<uint64_t>(p.lda) * sizeof(In)};
        uint32_t const box[2] = {static_cast<uint32_t>(kBlockK), static_cast<uint32_t>(kBlockM)};
        int32_t const st = makeTensorMap(&mapA, dt, 2, p.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != BERT_B200_OK)
            return st;
    }
    {
        uint64_t const dims[2] = {static_cast<uint64_t>(p.k), static_cast<uint64_t>(p.n)};
        uint64_t const strides[1] = {static_cast<uint64_t>(p.k) * sizeof(In)};
        uint32_t const box[2] = {static_cast<uint32_t>(kBlockK), static_cast<uint32_t>(BLOCK_N / 2)};
        int32_t const st = makeTensorMap(&mapB, dt, 2, p.wt, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != BERT_B200_OK)
            return st;
    }
    CUtensorMap mapC;
    {
        uint64_t const dims[2] = {static_cast<uint64_t>(p.n), static_cast<uint64_t>(p.m)};
        uint64_t const strides[1] = {static_cast<uint64_t>(p.ldc) * sizeof(Out)};
        uint32_t const box[2] = {32u, 32u};
        int32_t const st = makeTensorMap(&mapC, sizeof(Out) == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
            p.c, dims, strides, box, sizeof(Out) == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B);
        if (st != BERT_B200_OK)
            return st;
    }
    auto kernel = fcTcgen05PairKernel<In, BLOCK_N, Out>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "fc: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    int64_t const tiles = ((p.m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((p.n + BLOCK_N - 1) / BLOCK_N);
    int64_t const pairs = smCount() / 2;
    int const grid = static_cast<int>(2 * (tiles < pairs ? tiles : pairs));
    FcArgs args{p.m, p.n, p.k, p.c, p.ldc, p.bias, p.activation, p.alpha, p.out_scale, p.status_word,
        p.out_scale > 0.f ? -128.f / p.out_scale : 0.f, p.out_scale > 0.f ? 127.f / p.out_scale : 0.f};
    cudaError_t const le = launchDependent(kernel, dim3(grid), dim3(kFcThreads), L::kDynamic, stream, mapA, mapB, mapC, args);
    if (le != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "fcTcgen05PairKernel: %s", cudaGetErrorString(le));
    return checkLaunch("fcTcgen05PairKernel");
}

// Tiles of 128 x BLOCK_N over the SMs: pick the BLOCK_N that wastes less of the last wave.
int pickBlockN(int64_t m, int64_t n)
{
    if (n <= 128)
        return 128;
    int const sms = smCount();
    auto cost = [&](int bn) {
        int64_t const tiles = ((m + kBlockM - 1) / kBlockM) * ((n + bn - 1) / bn);
        int64_t const waves = (tiles + sms - 1) / sms;
        // time ~ waves * tile work; 128-wide tiles run the tensor pipe a little less efficiently
        return static_cast<double>(waves) * bn * (bn == 128 ? 1.06 : 1.0);
    };
    return cost(128) < cost(256) ? 128 : 256;
}

// Same for 256 x BLOCK_N pair tiles over the SM pairs.
int pickBlockNPair(int64_t m, int64_t n)
{
    if (n <= 128)
        return 128;
    int const pairs = smCount() / 2;
    auto cost = [&](int bn) {
        int64_t const tiles = ((m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((n + bn - 1) / bn);
        int64_t const waves = (tiles + pairs - 1) / pairs;
        // measured: 256 x 128 pair tiles reach about two thirds of the rate of 256 x 256 tiles (1.43 against 2.16 POP/s)
        return static_cast<double>(waves) * bn * (bn == 128 ? 1.5 : 1.0);
    };
    return cost(128) < cost(256) ? 128 : 256;
}

} // namespace

EncodeTiledFn getEncodeTiled()
{
    static std::mutex mtx;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lock(mtx);
    if (!fn)
    {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int32_t makeTensorMap(CUtensorMap* map, CUtensorMapDataType type, int rank, void const* base, uint64_t const* dims,
    uint64_t const* stridesBytes, uint32_t const* box, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn const fn = getEncodeTiled();
    if (!fn)
        B200_FAIL(BERT_B200_NOT_INITIALIZED, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t d[5];
    cuuint64_t s[4];
    cuuint32_t b[5];
    cuuint32_t es[5];
    for (int i = 0; i < rank; ++i)
    {
        d[i] = dims[i];
        b[i] = box[i];
        es[i] = 1;
        if (i > 0)
            s[i - 1] = stridesBytes[i - 1];
    }
    CUresult const r = fn(map, type, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s, b, es,
        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        B200_FAIL(BERT_B200_BAD_PARAM, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    return BERT_B200_OK;
}

} // namespace b200

using namespace b200;

extern "C" int32_t bert_b200_fc(bert_b200_fc_params const* params, void* stream)
{
    B200_REQUIRE(params != nullptr, "fc: null params");
    bert_b200_fc_params const& p = *params;
    B200_REQUIRE(p.m >= 0 && p.n > 0 && p.k > 0, "fc: bad sizes m=%lld n=%lld k=%lld", static_cast<long long>(p.m),
        static_cast<long long>(p.n), static_cast<long long>(p.k));
    B200_REQUIRE(p.a && p.wt && p.c, "fc: null pointer");
    B200_REQUIRE(p.lda >= p.k && p.ldc >= p.n, "fc: lda/ldc smaller than the row length");
    B200_REQUIRE(p.activation == BERT_B200_ACT_NONE || p.activation == BERT_B200_ACT_GELU_ERF, "fc: unknown activation %d",
        p.activation);
    if (p.m == 0)
        return BERT_B200_OK;
    auto s = static_cast<cudaStream_t>(stream);
    if (p.type_id == BERT_B200_FP32)
    {
        B200_REQUIRE(p.out_type_id == BERT_B200_FP32, "fc: FP32 input needs FP32 output");
        return fcF32(p, s);
    }
    B200_REQUIRE(p.type_id == BERT_B200_FP16 || p.type_id == BERT_B200_INT8, "fc: type_id %d", p.type_id);
    B200_REQUIRE(p.out_type_id != BERT_B200_INT8 || p.out_scale > 0.f, "fc: INT8 output needs out_scale > 0");
    B200_REQUIRE(p.m < (1ll << 31) && p.n < (1ll << 31) && p.k < (1ll << 31), "fc: sizes exceed the 32-bit TMA coordinates");
    int const elem = p.type_id == BERT_B200_FP16 ? 2 : 1;
    B200_REQUIRE((p.k * elem) % 16 == 0 && (p.lda * elem) % 16 == 0, "fc: row bytes of A / Wt must be a multiple of 16");
    B200_REQUIRE(aligned16(p.a) && aligned16(p.wt) && aligned16(p.c), "fc: A, Wt and C must be 16-byte aligned");
    B200_REQUIRE(p.n % 16 == 0, "fc: n=%lld must be a multiple of 16", static_cast<long long>(p.n));
    B200_REQUIRE(!p.bias || aligned16(p.bias), "fc: bias must be 16-byte aligned");
    int const outElem = p.out_type_id == BERT_B200_FP16 ? 2 : 1;
    B200_REQUIRE((p.ldc * outElem) % 16 == 0, "fc: row bytes of C must be a multiple of 16");
    // More than one 128-row block: two-CTA tiles of 256 rows; a single block would leave the peer CTA idle.
    bool const pair = p.m > kBlockM;
    int const bn = pair ? pickBlockNPair(p.m, p.n) : pickBlockN(p.m, p.n);
#define B200_FC_DISPATCH(IN, OUT)                                                                                      \
    return pair ? (bn == 128 ? launchFcPair<IN, 128, OUT>(p, s) : launchFcPair<IN, 256, OUT>(p, s))                     \
                : (bn == 128 ? launchFc<IN, 128, OUT>(p, s) : launchFc<IN, 256, OUT>(p, s))
    if (p.type_id == BERT_B200_FP16)
    {
        B200_REQUIRE(p.out_type_id == BERT_B200_FP16, "fc: FP16 input needs FP16 output");
        B200_FC_DISPATCH(__half, __half);
    }
    if (p.out_type_id == BERT_B200_INT8)
    {
        B200_FC_DISPATCH(int8_t, int8_t);
    }
    B200_REQUIRE(p.out_type_id == BERT_B200_FP16, "fc: INT8 input needs INT8 or FP16 output");
    B200_FC_DISPATCH(int8_t, __half);
#undef B200_FC_DISPATCH
}

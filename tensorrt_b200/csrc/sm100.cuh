// Thin inline-PTX layer for the Blackwell (sm_100a) data path used by the tensor-core kernels:
// mbarriers with bounded waits, TMA tiled loads (never multicast), tcgen05 MMA / TMEM access,
// shared-memory matrix descriptors and the host-side tensor-map encoder.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace b200
{

// Status codes written to the caller's status word when a bounded device wait expires.
enum : uint32_t
{
    kWaitOk = 0,
    kWaitTmaFull = 1,   // consumer waited for a TMA tile
    kWaitStageFree = 2, // producer waited for a free pipeline stage
    kWaitAccFull = 3,   // epilogue waited for an accumulator
    kWaitAccFree = 4,   // MMA issuer waited for a drained accumulator
    kWaitSoftmax = 5    // MMA issuer waited for softmax output / softmax waited for scores
};

// ---- host: tensor maps ----------------------------------------------------------------------
// cuTensorMapEncodeTiled is fetched through the runtime so the library does not link libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, cuuint64_t const*,
    cuuint64_t const*, cuuint32_t const*, cuuint32_t const*, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn getEncodeTiled();

// rank-`rank` tensor of `elemBytes`-byte elements; dims[0] is the contiguous one; strides in bytes for dims 1...
int32_t makeTensorMap(CUtensorMap* map, CUtensorMapDataType type, int rank, void const* base, uint64_t const* dims,
    uint64_t const* stridesBytes, uint32_t const* box, CUtensorMapSwizzle swizzle);

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smemAddr(void const* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globalTimerNs()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbarInit(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fenceBarrierInit()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA / tcgen05.mma operands).
__device__ __forceinline__ void fenceProxyAsync()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbarArrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}

__device__ __forceinline__ void mbarArriveExpectTx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}

// `barAddr` is a shared::cta address (smemAddr); the loops of the single-thread producer / MMA roles keep such
// addresses in registers so that a wait costs no address arithmetic.
__device__ __forceinline__ bool mbarTryWaitAddr(uint32_t barAddr, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(barAddr), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking form: mbarrier.try_wait may suspend the thread for a system-dependent time before it reports an
// incomplete phase; a thread that polls several barriers in turn (and must not sleep on one while another completes)
// uses test_wait, which returns at once.
__device__ __forceinline__ bool mbarTestWaitAddr(uint32_t barAddr, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(barAddr), "r"(parity)
        : "memory");
    return ok != 0;
}

// Every spin in these kernels is bounded: after kWaitLimitNs without progress the waiter records
// `code` in *abortFlag (shared memory; every later wait in the CTA returns immediately) and
// returns false. The kernel then drains, frees its TMEM and exits; the host sees the status word.
constexpr uint64_t kWaitLimitNs = 2000000000ull; // 2 s

// The polling loop is one out-of-line copy per kernel image: inlined at every wait it was a sizeable part of the
// code of the persistent kernels, whose single-thread roles are sensitive to instruction-cache misses.
static __device__ __noinline__ bool mbarWaitSlow(
    uint32_t barAddr, uint32_t parity, volatile uint32_t* abortFlag, uint32_t code, uint64_t limitNs = kWaitLimitNs)
{
    // The clock is only consulted every 256 failed polls (a read of %globaltimer costs far more than a poll, and most
    // waits end within a few polls), so the common case is nothing but try_wait.
    uint64_t t0 = 0;
    uint32_t polls = 0;
    while (true)
    {
        if (mbarTryWaitAddr(barAddr, parity))
            return true;
        if ((++polls & 255u) == 0)
        {
            if (*abortFlag != 0)
                return false;
            uint64_t const now = globalTimerNs();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > limitNs)
            {
                *abortFlag = code;
                return false;
            }
        }
    }
}

__device__ __forceinline__ bool mbarWaitAddr(uint32_t barAddr, uint32_t parity, volatile uint32_t* abortFlag, uint32_t code)
{
    if (mbarTryWaitAddr(barAddr, parity))
        return true;
    return mbarWaitSlow(barAddr, parity, abortFlag, code);
}

__device__ __forceinline__ bool mbarWait(uint64_t* bar, uint32_t parity, volatile uint32_t* abortFlag, uint32_t code)
{
    return mbarWaitAddr(smemAddr(bar), parity, abortFlag, code);
}

// ---- TMA ------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetchTensorMap(CUtensorMap const* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Tiled loads into this CTA's shared memory, completion on an mbarrier of this CTA. No multicast.
__device__ __forceinline__ void tmaLoad2d(void* dst, CUtensorMap const* map, uint64_t* bar, int32_t c0, int32_t c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smemAddr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smemAddr(bar)), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tmaLoad4d(
    void* dst, CUtensorMap const* map, uint64_t* bar, int32_t c0, int32_t c1, int32_t c2, int32_t c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smemAddr(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smemAddr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Tiled store from this CTA's shared memory (bulk async-group completion). The writer makes its shared-memory
// writes visible to the async proxy first (fenceProxyAsync by every writing thread, then a barrier); the issuing
// thread must see its groups complete (bulkWaitGroup<0>) before the CTA exits. The innermost coordinate times the
// element size is a multiple of 16 bytes at every call site; elements outside the tensor are not written.
__device__ __forceinline__ void tmaStore2d(CUtensorMap const* map, void const* src, int32_t c0, int32_t c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smemAddr(src)), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void bulkCommitGroup()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// At most N of this thread's most recent bulk groups may still be reading their shared-memory source.
template <int N>
__device__ __forceinline__ void bulkWaitGroupRead()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// At most N of this thread's most recent bulk groups may still be incomplete.
template <int N>
__device__ __forceinline__ void bulkWaitGroup()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tcgen05 / TMEM -------------------------------------------------------------------------
// Executed by one full warp. Writes the TMEM base address to *dst (shared memory).
__device__ __forceinline__ void tmemAlloc(uint32_t* dst, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(dst)), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmemFree(uint32_t addr, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcFenceBefore()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcFenceAfter()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// The mbarrier receives one arrival when all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tcCommit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar))
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; issued by a single thread.
__device__ __forceinline__ void mmaF16(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t iDesc, bool accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(dTmem),
        "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}

__device__ __forceinline__ void mmaI8(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t iDesc, bool accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(dTmem),
        "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}

// The same with the 64-bit descriptors assembled inside the asm block from their 32-bit halves: a thread that issues
// many small MMAs keeps one low word per operand tile (start address in bits 0-13; + bytes >> 4 moves it) and one
// constant high word per operand kind in registers instead of rebuilding or holding dozens of 64-bit descriptors.
template <bool kInt8>
__device__ __forceinline__ void mmaLoHi(
    uint32_t dTmem, uint32_t aLo, uint32_t aHi, uint32_t bLo, uint32_t bHi, uint32_t iDesc, bool accumulate)
{
    if constexpr (kInt8)
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            ".reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %6, 0;\n\t"
            "mov.b64 da, {%1, %2};\n\t"
            "mov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t"
            "}" ::"r"(dTmem),
            "r"(aLo), "r"(aHi), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(static_cast<uint32_t>(accumulate))
            : "memory");
    else
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            ".reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %6, 0;\n\t"
            "mov.b64 da, {%1, %2};\n\t"
            "mov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
            "}" ::"r"(dTmem),
            "r"(aLo), "r"(aHi), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(static_cast<uint32_t>(accumulate))
            : "memory");
}

// Lane l of the warp receives TMEM lane (base lane + l), 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmemLoad32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmemLoad16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// tcgen05.ld is asynchronous: its destination registers may only be read after tcgen05.wait::ld. Passing the
// registers through the wait as read-write operands makes every later use depend on it, so the compiler cannot
// schedule arithmetic on them ahead of the wait (needed when a load is left in flight across other work).
__device__ __forceinline__ void tmemLoadWait32(uint32_t (&r)[32])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                 "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

__device__ __forceinline__ void tmemLoadWait16(uint32_t (&r)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}

// ---- two-CTA (cta_group::2) variants ---------------------------------------------------------
// A cluster of two CTAs on neighbouring SMs issues one MMA of M = 256: each CTA supplies its own 128 rows of A and its
// own half of the B rows from its own shared memory and keeps its own 128 accumulator rows in its own TMEM. Only
// the even ("leader") CTA issues MMAs and commits. None of the loads below uses multicast.
__device__ __forceinline__ uint32_t clusterCtaRank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void clusterSync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapaShared(void const* localPtr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr(localPtr)), "r"(rank));
    return r;
}

__device__ __forceinline__ void mbarArriveCluster(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}

// Executed by the same warp index in both CTAs of the pair.
__device__ __forceinline__ void tmemAllocPair(uint32_t* dst, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(dst)), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmemFreePair(uint32_t addr, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}

// One arrival on the mbarrier at the same shared-memory offset in every CTA of `ctaMask`, once all MMAs issued
// so far have completed.
__device__ __forceinline__ void tcCommitPair(uint64_t* bar, uint16_t ctaMask)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smemAddr(bar)),
        "h"(ctaMask)
        : "memory");
}

// Lean forms for the inner loops of the single-thread roles. Those threads share a warp scheduler with busy epilogue
// warps, so every instruction they need per k-block costs tensor-pipe time: shared-memory addresses and the descriptor
// words are kept in registers, the 64-bit descriptors are assembled inside the asm block from a running low word
// (start-address field in bits 0-13, + bytes >> 4 to advance) and the constant high word, and the accumulate flag is
// a compile-time constant where it can be.
template <bool kInt8, bool kAcc>
__device__ __forceinline__ void mmaPairLoHi(uint32_t dTmem, uint32_t aLo, uint32_t bLo, uint32_t descHi, uint32_t iDesc)
{
    if constexpr (kInt8)
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            ".reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %5, 0;\n\t"
            "mov.b64 da, {%1, %3};\n\t"
            "mov.b64 db, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %4, p;\n\t"
            "}" ::"r"(dTmem),
            "r"(aLo), "r"(bLo), "r"(descHi), "r"(iDesc), "n"(kAcc ? 1 : 0)
            : "memory");
    else
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            ".reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %5, 0;\n\t"
            "mov.b64 da, {%1, %3};\n\t"
            "mov.b64 db, {%2, %3};\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t"
            "}" ::"r"(dTmem),
            "r"(aLo), "r"(bLo), "r"(descHi), "r"(iDesc), "n"(kAcc ? 1 : 0)
            : "memory");
}

__device__ __forceinline__ void tcCommitPairAddr(uint32_t barAddr, uint16_t ctaMask)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(barAddr),
        "h"(ctaMask)
        : "memory");
}

// Tile into this CTA's shared memory (`dstAddr`, a shared::cta address); the transaction bytes are counted on the
// mbarrier at `barClusterAddr`, which may live in the peer CTA (the leader's "full" barrier collects both CTAs' loads).
__device__ __forceinline__ void tmaLoad2dPairAddr(uint32_t dstAddr, CUtensorMap const* map, uint32_t barClusterAddr, int32_t c0, int32_t c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dstAddr), "l"(reinterpret_cast<uint64_t>(map)), "r"(barClusterAddr), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void mbarArriveExpectTxAddr(uint32_t barAddr, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barAddr), "r"(bytes) : "memory");
}

// ---- descriptors ----------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address, leading / stride byte offsets (all >> 4),
// descriptor version 1 (Blackwell) in bits 46-47 and the swizzle mode in bits 61-63.
enum : uint64_t
{
    kSwizzleNone = 0,
    kSwizzle128B = 2,
    kSwizzle64B = 4,
    kSwizzle32B = 6
};

__device__ __forceinline__ uint64_t makeSmemDesc(uint32_t saddr, uint32_t lboBytes, uint32_t sboBytes, uint64_t swizzle)
{
    return static_cast<uint64_t>((saddr >> 4) & 0x3fffu) | (static_cast<uint64_t>((lboBytes >> 4) & 0x3fffu) << 16)
        | (static_cast<uint64_t>((sboBytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (swizzle << 61);
}

// Instruction descriptor (32 bit) for kind::f16 / kind::i8, dense, no negate, no saturate.
//   cFormat: 1 = F32, 2 = S32.  abFormat: kind::f16 -> 0 = F16, 1 = BF16; kind::i8 -> 1 = signed 8 bit.
//   aMajor / bMajor: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t makeInstrDesc(
    uint32_t cFormat, uint32_t abFormat, uint32_t aMajor, uint32_t bMajor, uint32_t m, uint32_t n)
{
    return (cFormat << 4) | (abFormat << 7) | (abFormat << 10) | (aMajor << 15) | (bMajor << 16) | ((n >> 3) << 17)
        | ((m >> 4) << 24);
}

#endif // __CUDACC__

} // namespace b200

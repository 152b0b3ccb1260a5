// FP16 fused multi-head attention on the sm_100a tensor cores with a key-block-wise online softmax
// (head sizes 16, 32, 48, 64; any sequence length), fixed [S,B,N,3,d], packed [total,N,3,d] and separate
// [B,N,S,d] layouts.
//
// Replaces, for FP16, the precompiled fused attention kernels the reference launches through
// FusedMHARunnerFP16[v2]::run (plugin/bertQKVToContextPlugin/mhaRunner.cu:835-860, 1127-1265) and its unfused
// cuBLAS + softmax path (mhaRunner.cu:533-601) for the sequence lengths those kernels do not cover.
//
// One persistent CTA per SM keeps TWO 128-query tiles in flight (streams 0 and 1). The tiles of the CTA's work
// list are dealt alternately to the two streams, across the boundaries of (sequence, head) items, so an odd number
// of tiles per item (S = 384) leaves no stream idle. 12 warps:
//   warps 0-3 / 4-7 : softmax of stream 0 / 1, ONE THREAD PER QUERY ROW (the 32x32b TMEM load hands lane = row):
//                     no cross-thread reduction, no barrier among softmax threads. Per key block: load the 128
//                     scores into registers (their TMEM columns are then free for the next block's scores), block
//                     maximum, lazy rescale (below), p = exp2(x*scale*log2e - m), row sum, P as FP16 pairs into 64
//                     TMEM columns of its own. The normalising epilogue of a tile is deferred into the first block of
//                     the stream's next tile, so its wait for the last context product costs nothing.
//   warp 8          : one lane loads the Q tiles (two slots, one per stream).
//   warp 9          : one lane loads K / V blocks (128 keys x 64 channels, 16 KB) into a ring of 12 stages. The
//                     blocks of an item stay resident for all its query tiles when they fit (S <= 768); longer
//                     sequences stream their blocks once per pair of query tiles.
//   warps 10 / 11   : one lane each, the MMA thread of stream 0 / 1. It issues the stream's scores  S = Q K_j^T
//                     (128 x 128, FP32, TMEM columns 128*stream ..) as soon as the softmax threads hold the previous
//                     block in registers - the first block of the stream's NEXT tile right behind the last block of
//                     this one -, and the context products  O (+)= P_j V_j  (128 x 64, A operand = P straight from TMEM
//                     columns 256 + 64*stream .., accumulator in columns 384 + 64*stream ..) as soon as P_j is stored.
//                     (Every tcgen05.mma / commit keeps its issuing thread busy for 50-120 cycles: the twelve MMAs and
//                     four commits of a block are a thread's work of its own per stream.) A thread per stream may block
//                     on its stream's barriers; one thread serving both streams must not - an operand that a loader
//                     delivers only after the OTHER stream has been served would never arrive.
// Online softmax: the running maximum m only moves when the block maximum exceeds it by more than 8 in the log2
// domain (P then stays below 2^8, far inside FP16); when it moves, the softmax threads scale the row sum and the
// context accumulator in TMEM themselves (after the previous P V product has completed). The final context is
// O / rowsum. Compared with a softmax over the exact row maximum this changes nothing but the rounding of P.
// Every wait is bounded (sm100.cuh); on expiry the CTA drains, frees TMEM and reports through the status word.
#include "sm100.cuh"

namespace b200
{

namespace
{

#ifdef MHA_TRACE
// timeline of CTA 0: (role, event code, cycle) triples, 512 events per role, roles 0/1 softmax, 2/3 MMA threads
#define TR_DECL(role) uint32_t trN = 0; uint32_t* const trBuf = (blockIdx.x == 0 && args.statusWord) ? args.statusWord + 16 + (role) * 1024 : nullptr
#define TR_EVT(code) do { if (trBuf && trN < 512) { trBuf[2 * trN] = (code); trBuf[2 * trN + 1] = static_cast<uint32_t>(clock64()); ++trN; } } while (0)
#else
#define TR_DECL(role)
#define TR_EVT(code)
#endif

constexpr int kTile = 128;       // query rows per tile = keys per block
constexpr int kHeadSize = 64;    // channels per tile row (smaller heads are zero-filled by the TMA unit)
constexpr int kStages = 12;      // K / V ring
constexpr int kStageBytes = kTile * kHeadSize * 2; // 16 KB: one Q tile, one K block, one V block
constexpr int kThreads = 384;    // 8 softmax warps, Q loader, K/V loader, two MMA issuers
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kPColumn = 256; // P blocks (FP16 pairs): 64 columns per stream
constexpr uint32_t kOColumn = 384; // context accumulators: 64 columns per stream
constexpr float kRescaleLog2 = 8.f;

struct OnlineArgs
{
    int32_t B, S, N, total;
    int32_t d;
    int32_t fixedLayout;
    void* out;
    int32_t const* cu;
    int32_t const* maskIdx;
    float scaleBmm1;
    uint32_t* statusWord;
    int32_t tilesPerUnit, chunks; // a work unit = (sequence, head, chunk of tilesPerUnit query tiles)
    int32_t stepChunk, stepHead, stepB; // gridDim.x = stepChunk + chunks * (stepHead + N * stepB)
};

// [ Q slot 0 ][ Q slot 1 ][ 12 K/V stages ][ barriers ]
constexpr int kSmemQ = 0;
constexpr int kSmemKv = 2 * kStageBytes;
constexpr int kSmemBars = kSmemKv + kStages * kStageBytes;
// full[12] empty[12] qFull[2] qFree[2] sFull[2] sFree[2] pReady[2] pvDone[2], tmem slot, abort flag
constexpr int kNumBars = 2 * kStages + 12;
constexpr int kGeoEntries = 128; // geometry words of the CTA's first work units, read once from global memory
constexpr int kSmemGeo = kSmemBars + kNumBars * 8 + 16;
constexpr int kSmemBytes = kSmemGeo + kGeoEntries * 8 + 1024;

__device__ __forceinline__ float ex2Approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fmax3(float a, float b, float c)
{
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (P, FP16, two keys per 32-bit column, lane = query row) is read from
// tensor memory. The 64-bit B descriptor is assembled from its halves inside the asm block.
__device__ __forceinline__ void mmaF16TmemA(uint32_t dTmem, uint32_t aTmem, uint32_t bLo, uint32_t bHi, uint32_t iDesc, bool accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
        "}" ::"r"(dTmem),
        "r"(aTmem), "r"(bLo), "r"(bHi), "r"(iDesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}

__device__ __forceinline__ void tmemStore16(uint32_t taddr, uint32_t const (&r)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tmemStoreWait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t packHalf2(float lo, float hi)
{
    __half2 const h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t const*>(&h);
}

// Geometry of one work unit; identical in every role (derived from the arguments and two words of global memory).
struct Unit
{
    int32_t b, head, rowBase, rows, len, nb, tBegin, tEnd;
};

// The CTA's list of query tiles in processing order. Tile number n (counted per CTA) belongs to stream n & 1.
// A "sub-item" is the run of tiles that shares one load of the K / V blocks: all tiles of a unit when its blocks fit
// the ring, otherwise pairs of tiles (one per stream). `loadBase` is the number of K / V blocks loaded before it:
// block j of the sub-item is load number loadBase + 2j (K) and loadBase + 2j + 1 (V); a load number L lives in ring
// stage L % kStages and is the (L / kStages)-th fill of that stage.
struct Walker
{
    OnlineArgs const* ap;
    int32_t numUnits;
    int32_t unit;
    Unit g;
    int32_t t;        // query tile inside the (sequence, head)
    int32_t subEnd;   // one past the last tile of the sub-item
    int32_t subTiles; // tiles in the sub-item = uses of each of its stages
    uint32_t loadBase;
    uint32_t n;
    // (row base, end) or mask length of the CTA's k-th unit for k < kGeoEntries, staged in shared memory by the kernel's
    // prologue: a load from global memory at every change of unit (under streaming traffic often a DRAM access) would
    // sit on the critical path of every role
    int2 const* geo;

    __device__ __forceinline__ Walker(OnlineArgs const& args, int2 const* geoTable)
        : ap(&args)
        , numUnits(args.B * args.N * args.chunks)
        , geo(geoTable)
    {
    }

    __device__ __forceinline__ static void fetch(OnlineArgs const& a, int32_t u, int32_t& wa, int32_t& wb)
    {
        int32_t const b = (u / a.chunks) / a.N;
        wa = 0;
        wb = 0;
        if (a.fixedLayout)
        {
            if (a.maskIdx)
                wb = __ldg(a.maskIdx + b);
        }
        else
        {
            wa = __ldg(a.cu + b);
            wb = __ldg(a.cu + b + 1);
        }
    }

    // The CTA's k-th unit is unit number blockIdx.x + k * gridDim.x = (sequence cb, head ch, chunk cc). Going to the
    // next one adds the launch's precomputed decomposition of gridDim.x (no division on the way).
    int32_t k, cb, ch, cc;

    __device__ __forceinline__ void firstUnit()
    {
        unit = static_cast<int32_t>(blockIdx.x);
        k = 0;
        cc = unit % ap->chunks;
        int32_t const i = unit / ap->chunks;
        cb = i / ap->N;
        ch = i - cb * ap->N;
    }

    __device__ __forceinline__ void stepUnit()
    {
        unit += static_cast<int32_t>(gridDim.x);
        ++k;
        cc += ap->stepChunk;
        if (cc >= ap->chunks)
        {
            cc -= ap->chunks;
            ++ch;
        }
        ch += ap->stepHead;
        if (ch >= ap->N)
        {
            ch -= ap->N;
            ++cb;
        }
        cb += ap->stepB;
    }

    // geometry of the current unit; returns whether it has work for the tensor pipeline (a query row and a valid key)
    __device__ __forceinline__ bool geometry(Unit& o) const
    {
        int32_t wa, wb;
        if (k < kGeoEntries)
        {
            int2 const e = geo[k];
            wa = e.x;
            wb = e.y;
        }
        else
            fetch(*ap, unit, wa, wb);
        o.b = cb;
        o.head = ch;
        if (ap->fixedLayout)
        {
            o.rowBase = 0;
            o.rows = ap->S;
            o.len = ap->maskIdx ? min(max(wb, 0), ap->S) : ap->S;
        }
        else
        {
            o.rowBase = wa;
            o.len = min(max(wb - wa, 0), ap->S);
            o.rows = o.len;
        }
        o.nb = (o.len + kTile - 1) / kTile;
        int32_t const nq = (o.rows + kTile - 1) / kTile;
        o.tBegin = cc * ap->tilesPerUnit;
        o.tEnd = min(nq, o.tBegin + ap->tilesPerUnit);
        return o.len > 0 && o.tBegin < o.tEnd;
    }

    // settles on the current unit or the first one after it that has work
    __device__ __forceinline__ bool seek()
    {
        while (unit < numUnits && !geometry(g))
            stepUnit();
        if (unit >= numUnits)
            return false;
        t = g.tBegin;
        setSub();
        return true;
    }

    __device__ __forceinline__ bool resident() const
    {
        return 2 * g.nb <= kStages;
    }

    __device__ __forceinline__ void setSub()
    {
        subTiles = resident() ? g.tEnd - t : min(2, g.tEnd - t);
        subEnd = t + subTiles;
    }

    __device__ __forceinline__ bool begin()
    {
        n = 0;
        loadBase = 0;
        firstUnit();
        return seek();
    }

    __device__ __forceinline__ bool next()
    {
        ++t;
        ++n;
        if (t == subEnd)
        {
            loadBase += 2u * static_cast<uint32_t>(g.nb);
            if (t == g.tEnd)
            {
                stepUnit();
                return seek();
            }
            setSub();
        }
        return true;
    }

    __device__ __forceinline__ bool firstOfSub() const
    {
        return t == subEnd - subTiles;
    }
};

// The loads [first, last) of a ring of kStages stages, in load order, for a thread that reads none of them: wait until
// each block has landed, hand its stage back. Out of line: it runs once per tile at most and the kernel is sensitive to
// the size of its hot code.
static __device__ __noinline__ bool passThroughLoads(
    uint32_t fullAddr, uint32_t emptyAddr, uint32_t first, uint32_t last, volatile uint32_t* abortFlag)
{
    for (uint32_t L = first; L < last; ++L)
    {
        uint32_t const stage = L % kStages;
        if (!mbarWaitAddr(fullAddr + 8 * stage, (L / kStages) & 1u, abortFlag, kWaitTmaFull))
            return false;
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(emptyAddr + 8 * stage) : "memory");
    }
    return true;
}

template <bool BNSD>
__global__ void __maxnreg__(168)
    mhaOnlineF16Kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
        const __grid_constant__ CUtensorMap mapV, OnlineArgs const args)
{
    constexpr uint32_t kIdescQk = makeInstrDesc(1u, 0u, 0u, 0u, 128u, 128u);
    constexpr uint32_t kIdescPv = makeInstrDesc(1u, 0u, 0u, 1u, 128u, 64u);

    int const warp = threadIdx.x >> 5;
    int const lane = threadIdx.x & 31;

    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sQ = smem + kSmemQ;
    uint8_t* sKv = smem + kSmemKv;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemBars);
    uint64_t* full = bars;                    // [12] K / V block landed
    uint64_t* empty = bars + kStages;         // [12] every MMA that reads the stage has completed
    uint64_t* qFull = bars + 2 * kStages;     // [2]  Q tile of the stream landed
    uint64_t* qFree = qFull + 2;              // [2]  all score MMAs of the stream's tile have completed
    uint64_t* sFull = qFree + 2;              // [2]  scores of a key block complete               (once per block)
    uint64_t* sFree = sFull + 2;              // [2]  scores are in registers, 4 arrivals           (once per block)
    uint64_t* pReady = sFree + 2;             // [2]  P block written, 4 arrivals                   (once per block)
    uint64_t* pvDone = pReady + 2;            // [2]  context product of a block complete           (once per block)
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(pvDone + 2);
    volatile uint32_t* abortFlag = tmemSlot + 1;
    int2* geoTable = reinterpret_cast<int2*>(smem + kSmemGeo);

    if (threadIdx.x == 0)
    {
        for (int i = 0; i < kStages; ++i)
        {
            mbarInit(&full[i], 1);
            mbarInit(&empty[i], 2); // one arrival per stream (see the MMA threads)
        }
        for (int i = 0; i < 2; ++i)
        {
            mbarInit(&qFull[i], 1);
            mbarInit(&qFree[i], 1);
            mbarInit(&sFull[i], 1);
            mbarInit(&sFree[i], 4); // one arrival per softmax warp of the stream
            mbarInit(&pReady[i], 4);
            mbarInit(&pvDone[i], 1);
        }
        *abortFlag = 0;
        fenceBarrierInit();
        prefetchTensorMap(&mapQ);
        if (BNSD)
        {
            prefetchTensorMap(&mapK);
            prefetchTensorMap(&mapV);
        }
    }
    if (warp == 8)
        tmemAlloc(tmemSlot, kTmemCols);
    tcFenceBefore();
    __syncthreads();
    tcFenceAfter();
    uint32_t const tmemBase = *tmemSlot;
    gridDependencyLaunch();
    gridDependencyWait();
    {
        int32_t const numUnits = args.B * args.N * args.chunks;
        int32_t const u = static_cast<int32_t>(blockIdx.x) + static_cast<int32_t>(threadIdx.x) * static_cast<int32_t>(gridDim.x);
        if (threadIdx.x < kGeoEntries && u < numUnits)
        {
            int32_t wa, wb;
            Walker::fetch(args, u, wa, wb);
            geoTable[threadIdx.x] = make_int2(wa, wb);
        }
        __syncthreads();
    }

    // which: 0 = Q, 1 = K, 2 = V; row = first token of the box inside the (packed or per-sequence) tensor
    auto load = [&](uint8_t* dst, uint64_t* bar, int which, Unit const& g, int32_t row) {
        if (BNSD) // (channel, position, head, sequence)
            tmaLoad4d(dst, which == 0 ? &mapQ : (which == 1 ? &mapK : &mapV), bar, 0, row, g.head, g.b);
        else // (channel, which of [N][3], batch, row)
            tmaLoad4d(dst, &mapQ, bar, 0, g.head * 3 + which, args.fixedLayout ? g.b : 0, row);
    };

    if (warp == 8)
    {
        // ---- Q tiles: slot n & 1, refilled when the score MMAs of the stream's previous tile have completed ----
        if (lane == 0)
        {
            Walker w(args, geoTable);
            bool ok = true;
            for (bool more = w.begin(); more && ok; more = w.next())
            {
                uint32_t const slot = w.n & 1u;
                if (w.n >= 2)
                    ok = mbarWait(&qFree[slot], ((w.n >> 1) - 1) & 1u, abortFlag, kWaitStageFree);
                if (!ok)
                    break;
                mbarArriveExpectTx(&qFull[slot], kStageBytes);
                load(sQ + slot * kStageBytes, &qFull[slot], 0, w.g, (args.fixedLayout ? 0 : w.g.rowBase) + w.t * kTile);
            }
        }
    }
    else if (warp == 9)
    {
        // ---- K / V blocks of every sub-item, in the order the MMA threads consume them ----
        if (lane == 0)
        {
            Walker w(args, geoTable);
            bool ok = true;
            for (bool more = w.begin(); more && ok; more = w.next())
            {
                if (!w.firstOfSub())
                    continue;
                int32_t const rowK = args.fixedLayout ? 0 : w.g.rowBase;
                for (int j = 0; j < w.g.nb && ok; ++j)
                {
                    for (int kv = 0; kv < 2 && ok; ++kv)
                    {
                        uint32_t const L = w.loadBase + 2u * j + kv;
                        uint32_t const s = L % kStages;
                        uint32_t const fill = L / kStages;
                        if (fill > 0)
                            ok = mbarWait(&empty[s], (fill - 1) & 1u, abortFlag, kWaitStageFree);
                        if (!ok)
                            break;
                        mbarArriveExpectTx(&full[s], kStageBytes);
                        load(sKv + s * kStageBytes, &full[s], 1 + kv, w.g, rowK + j * kTile);
                    }
                }
            }
        }
    }
    else if (warp == 10 || warp == 11)
    {
        // ---- MMA issue: warp 10 owns stream 0, warp 11 stream 1 ----
        // The events of one stream come in a fixed order - scores of block j in registers (sFree), P_j written
        // (pReady), scores of block j+1 in registers, ... - so its thread simply waits for them in turn: after sFree it
        // issues the next scores (of this tile or of the stream's next one), after pReady the context product.
        if (lane == 0)
        {
            uint32_t const s = static_cast<uint32_t>(warp - 10);
            // K-major Q / K tiles (128-byte rows, 128-byte swizzle): SBO = 8 rows = 1024 B. V is MN-major (the head
            // dimension contiguous): one MMA consumes 16 key rows = 2048 B.
            uint64_t const dQk = makeSmemDesc(0, 16, 1024, kSwizzle128B);
            uint64_t const dV = makeSmemDesc(0, 1024, 1024, kSwizzle128B);
            uint32_t const hiQk = static_cast<uint32_t>(dQk >> 32), hiV = static_cast<uint32_t>(dV >> 32);
            uint32_t const qLo = static_cast<uint32_t>(dQk) + (smemAddr(sQ) >> 4) + s * (kStageBytes >> 4);
            uint32_t const kLo = static_cast<uint32_t>(dQk) + (smemAddr(sKv) >> 4);
            uint32_t const vLo = static_cast<uint32_t>(dV) + (smemAddr(sKv) >> 4);
            constexpr uint32_t kStage16 = kStageBytes >> 4;
            uint32_t const fullAddr = smemAddr(full), emptyAddr = smemAddr(empty);
            uint32_t const sFullAddr = smemAddr(&sFull[s]), sFreeAddr = smemAddr(&sFree[s]), pReadyAddr = smemAddr(&pReady[s]);
            uint32_t const pvDoneAddr = smemAddr(&pvDone[s]), qFullAddr = smemAddr(&qFull[s]), qFreeAddr = smemAddr(&qFree[s]);
            uint32_t const tS = tmemBase + s * kTile, tP = tmemBase + kPColumn + s * kHeadSize, tO = tmemBase + kOColumn + s * kHeadSize;
            bool ok = true;
            auto commitAddr = [](uint32_t barAddr) {
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barAddr) : "memory");
            };
            // A ring stage goes back to the loader when BOTH streams' MMA threads are done with it: each commits once, with
            // its last tile of the sub-item. A sub-item of a single tile is read by one stream only; the other stream's
            // thread still takes part in every one of its loads (passThrough below).
            auto release = [&](uint32_t stage, Walker const& w) {
                if (w.t >= w.subEnd - 2)
                    commitAddr(emptyAddr + 8 * stage);
            };
            // The loads of a single-tile sub-item of the OTHER stream, in load order: wait until the block has landed, hand
            // the stage back. A parity wait on an mbarrier is only valid for the barrier's NEXT phase, so a thread that
            // waits on the `full` barrier of a ring stage has to have seen every earlier fill of that stage - also the
            // fills whose data it never reads. (Skipping them - the other stream's thread adding the second arrival - let
            // a thread that came back to a stage two fills later see "complete" at once and multiply blocks that had not
            // landed: with many long sequences per CTA the attention hung until the waits expired.)
            auto passThrough = [&](Walker const& w) {
                ok = ok && passThroughLoads(fullAddr, emptyAddr, w.loadBase, w.loadBase + 2u * static_cast<uint32_t>(w.g.nb), abortFlag);
            };
            // scores of key block j of the tile `w` stands on
            auto issueQk = [&](Walker const& w, int32_t j) {
                uint32_t const L = w.loadBase + 2u * j;
                uint32_t const stage = L % kStages;
                ok = ok && mbarWaitAddr(fullAddr + 8 * stage, (L / kStages) & 1u, abortFlag, kWaitTmaFull);
                if (!ok)
                    return;
                tcFenceAfter();
                uint32_t const b = kLo + stage * kStage16;
#pragma unroll
                for (int k = 0; k < 4; ++k) // head size 64 = 4 x 16
                    mmaLoHi<false>(tS, qLo + 2 * k, hiQk, b + 2 * k, hiQk, kIdescQk, k != 0);
                commitAddr(sFullAddr);
                release(stage, w);
                if (j == w.g.nb - 1)
                    commitAddr(qFreeAddr);
            };
            auto issuePv = [&](Walker const& w, int32_t j) {
                uint32_t const L = w.loadBase + 2u * j + 1u;
                uint32_t const stage = L % kStages;
                ok = ok && mbarWaitAddr(fullAddr + 8 * stage, (L / kStages) & 1u, abortFlag, kWaitTmaFull);
                if (!ok)
                    return;
                tcFenceAfter();
                uint32_t const b = vLo + stage * kStage16;
#pragma unroll
                for (int k = 0; k < 8; ++k) // 128 keys = 8 x 16; P: 8 TMEM columns per 16 keys
                    mmaF16TmemA(tO, tP + 8 * k, b + k * 128u, hiV, kIdescPv, (j | k) != 0);
                commitAddr(pvDoneAddr);
                release(stage, w);
            };

            TR_DECL(2 + s);
            Walker cur(args, geoTable);
            bool active = cur.begin();
            if (s == 1 && active)
            {
                // tile 0 is stream 0's
                if (cur.subTiles == 1)
                    passThrough(cur);
                active = cur.next();
            }
            uint32_t qk = 0, pv = 0; // groups of score / context MMAs issued so far
            if (active && ok)
            {
                ok = mbarWaitAddr(qFullAddr, (cur.n >> 1) & 1u, abortFlag, kWaitTmaFull);
                if (ok)
                    issueQk(cur, 0);
                qk = 1;
            }
            while (active && ok)
            {
                // the other stream's tile that follows this one, then this stream's next tile
                Walker nxt = cur;
                bool const hasMid = nxt.next();
                bool const midAlone = hasMid && nxt.subTiles == 1; // a sub-item this thread reads nothing of
                uint32_t const midFirst = nxt.loadBase, midBlocks = static_cast<uint32_t>(nxt.g.nb);
                bool const hasNext = hasMid && nxt.next();
                for (int j = 0; j < cur.g.nb && ok; ++j)
                {
                    // Two things to issue per block: the scores that follow block j - block j + 1, or the first block of the
                    // stream's next tile - and the context product of block j. The scores go first, so that the tensor pipe
                    // has them done when the softmax threads come for them. Across a tile boundary the wait for their
                    // operands then holds back the product whose completion frees this tile's last V stage, and the loader
                    // works in load order: that is safe only while fewer than eleven loads lie between that V block and the
                    // next tile's first K block (none when the tiles share sub-items; the 2 nb loads of the other stream's
                    // tile when that is a sub-item of its own). With more, the loader would need the stage of that very V
                    // block first - a cycle - and the product goes first. (One call site each for the two MMA groups: the
                    // kernel is sensitive to the size of its code.)
                    bool const lastBlock = j + 1 == cur.g.nb;
                    bool qkPending = !lastBlock || hasNext, pvPending = true;
                    bool const qkFirst = !lastBlock || !midAlone || midBlocks <= 5;
                    bool midPending = lastBlock && midAlone;
                    if (qkPending)
                        ok = mbarWaitAddr(sFreeAddr, (qk - 1) & 1u, abortFlag, kWaitAccFree);
                    TR_EVT(1);
#pragma unroll 1
                    while ((qkPending || pvPending) && ok)
                    {
                        if (qkPending && (qkFirst || !pvPending))
                        {
                            if (lastBlock)
                            {
                                if (midPending)
                                    ok = passThroughLoads(fullAddr, emptyAddr, midFirst, midFirst + 2u * midBlocks, abortFlag);
                                midPending = false;
                                ok = ok && mbarWaitAddr(qFullAddr, (nxt.n >> 1) & 1u, abortFlag, kWaitTmaFull);
                            }
                            if (ok)
                                issueQk(lastBlock ? nxt : cur, lastBlock ? 0 : j + 1);
                            TR_EVT(2);
                            ++qk;
                            qkPending = false;
                        }
                        else
                        {
                            ok = mbarWaitAddr(pReadyAddr, pv & 1u, abortFlag, kWaitSoftmax);
                            TR_EVT(3);
                            if (ok)
                                issuePv(cur, j);
                            TR_EVT(4);
                            ++pv;
                            pvPending = false;
                        }
                    }
                    // the other stream's last tile, when this stream has none after it
                    if (midPending && ok)
                        ok = passThroughLoads(fullAddr, emptyAddr, midFirst, midFirst + 2u * midBlocks, abortFlag);
                }
                cur = nxt;
                active = hasNext;
            }
        }
    }
    else
    {
        // ---- softmax: stream = warp / 4, query row = TMEM lane ----
        uint32_t const s = static_cast<uint32_t>(warp >> 2);
        int const r = (warp & 3) * 32 + lane;
        uint32_t const tRow = tmemBase + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        uint32_t const tS = tRow + s * kTile;
        uint32_t const tP = tRow + kPColumn + s * kHeadSize;
        uint32_t const tO = tRow + kOColumn + s * kHeadSize;
        float const sl2 = args.scaleBmm1 * 1.4426950408889634f;
        float const thrRaw = kRescaleLog2 / sl2; // the same threshold on the unscaled scores
        bool ok = true;

        if (s == 0 && args.fixedLayout)
        {
            // sequences without a valid key: every probability is zero and so is the context row
            Walker z(args, geoTable);
            Unit g;
            int const chunks16 = args.d / 8;
            for (z.firstUnit(); z.unit < z.numUnits; z.stepUnit())
            {
                z.geometry(g);
                if (g.len > 0 || g.tBegin >= g.tEnd)
                    continue;
                int const q0 = g.tBegin * kTile, q1 = min(g.rows, g.tEnd * kTile);
                for (int i = threadIdx.x; i < (q1 - q0) * chunks16; i += kTile)
                {
                    int const q = q0 + i / chunks16, c = i % chunks16;
                    __half* row = BNSD
                        ? static_cast<__half*>(args.out) + ((static_cast<int64_t>(g.b) * args.N + g.head) * args.S + q) * args.d
                        : static_cast<__half*>(args.out) + (static_cast<int64_t>(q) * args.B + g.b) * args.N * args.d + g.head * args.d;
                    reinterpret_cast<uint4*>(row)[c] = make_uint4(0, 0, 0, 0);
                }
            }
        }

        TR_DECL(lane == 0 && (warp & 3) == 0 ? s : 7);
        Walker w(args, geoTable);
        bool active = w.begin() && (s == 0 || w.next());
        uint32_t blocks = 0; // key blocks this stream has completed: parity of sFull / pvDone
        // the tile whose context still has to be normalised and stored (null: none, or a row beyond the sequence)
        bool pending = false;
        __half* pendDst = nullptr;
        float pendInv = 0.f;
        // context of the stream's previous tile: wait for its last product, O / rowsum -> FP16
        auto epilogue = [&]() {
            ok = ok && mbarWait(&pvDone[s], (blocks - 1) & 1u, abortFlag, kWaitAccFull);
            tcFenceAfter();
#pragma unroll 1
            for (int c = 0; c < kHeadSize; c += 16) // 16 columns at a time: the block's scores stay in registers
            {
                uint32_t o[16];
                tmemLoad16(tO + c, o);
                tmemLoadWait16(o);
                if (pendDst != nullptr && ok && c < args.d)
                {
                    float f[8];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                    {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            f[i] = __uint_as_float(o[8 * h + i]) * pendInv;
                        reinterpret_cast<uint4*>(pendDst + c)[h] = packHalf8(f);
                    }
                }
            }
            tcFenceBefore();
            pending = false;
        };
        // Keys at or beyond `limit` (counted from the chunk's first column) take no part: -inf scores, zero probabilities.
        auto maskChunk = [](uint32_t(&x)[32], int limit) {
            if (limit < 32)
            {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i >= limit)
                        x[i] = 0xff800000u;
            }
        };
        while (active)
        {
            Unit const g = w.g;
            float mRun = -INFINITY, l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll 1
            for (int j = 0; j < g.nb; ++j)
            {
                TR_EVT(10);
                ok = ok && mbarWait(&sFull[s], blocks & 1u, abortFlag, kWaitSoftmax);
                tcFenceAfter();
                TR_EVT(11);
                int const limit = g.len - j * kTile;
                // All 128 scores of the row go to registers at once; their TMEM columns are free for the next block's
                // scores from here on, so the tensor pipe works on S_{j+1} during this block's exponentials.
                uint32_t x0[32], x1[32], x2[32], x3[32];
                tmemLoad32(tS, x0);
                tmemLoad32(tS + 32, x1);
                tmemLoad32(tS + 64, x2);
                tmemLoad32(tS + 96, x3);
                tmemLoadWait32(x0);
                tmemLoadWait32(x1);
                tmemLoadWait32(x2);
                tmemLoadWait32(x3);
                tcFenceBefore();
                __syncwarp();
                if (lane == 0)
                    mbarArrive(&sFree[s]);
                TR_EVT(12);
                // eight independent chains: the block maximum costs the latency of eight dependent maxima, not thirty-two
                float mA = -INFINITY, mB = -INFINITY, mC = -INFINITY, mD = -INFINITY;
                float mE = -INFINITY, mF = -INFINITY, mG = -INFINITY, mH = -INFINITY;
                maskChunk(x0, limit);
                maskChunk(x1, limit - 32);
                maskChunk(x2, limit - 64);
                maskChunk(x3, limit - 96);
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                {
                    mA = fmax3(mA, __uint_as_float(x0[i]), __uint_as_float(x0[i + 1]));
                    mB = fmax3(mB, __uint_as_float(x0[i + 2]), __uint_as_float(x0[i + 3]));
                    mC = fmax3(mC, __uint_as_float(x1[i]), __uint_as_float(x1[i + 1]));
                    mD = fmax3(mD, __uint_as_float(x1[i + 2]), __uint_as_float(x1[i + 3]));
                    mE = fmax3(mE, __uint_as_float(x2[i]), __uint_as_float(x2[i + 1]));
                    mF = fmax3(mF, __uint_as_float(x2[i + 2]), __uint_as_float(x2[i + 3]));
                    mG = fmax3(mG, __uint_as_float(x3[i]), __uint_as_float(x3[i + 1]));
                    mH = fmax3(mH, __uint_as_float(x3[i + 2]), __uint_as_float(x3[i + 3]));
                }
                mA = fmax3(mA, mB, mC);
                mD = fmax3(mD, mE, mF);
                mG = fmaxf(mG, mH);
                float const mBlk = fmax3(mA, mD, mG);
                if (j == 0)
                    mRun = mBlk;
                else
                {
                    // The running maximum moves only when this block exceeds it by more than 2^8 after scaling.
                    bool const move = mBlk > mRun + thrRaw;
                    if (__any_sync(0xffffffffu, move))
                    {
                        float const f = move ? ex2Approx((mRun - mBlk) * sl2) : 1.f;
                        if (move)
                            mRun = mBlk;
                        l0 *= f;
                        l1 *= f;
                        l2 *= f;
                        l3 *= f;
                        // the context so far, once the previous block's product has completed
                        ok = ok && mbarWait(&pvDone[s], (blocks - 1) & 1u, abortFlag, kWaitAccFull);
                        tcFenceAfter();
#pragma unroll 1
                        for (int c = 0; c < kHeadSize; c += 16)
                        {
                            uint32_t o[16];
                            tmemLoad16(tO + c, o);
                            tmemLoadWait16(o);
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                            tmemStore16(tO + c, o);
                        }
                    }
                }
                float const negM = -mRun * sl2;

                // p = exp2(x * scale * log2e - m), row sum, P as FP16 pairs (32 keys -> 16 columns)
                auto expChunk = [&](uint32_t(&x)[32], uint32_t(&p)[16]) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                    {
                        float const e0 = ex2Approx(fmaf(__uint_as_float(x[i]), sl2, negM));
                        float const e1 = ex2Approx(fmaf(__uint_as_float(x[i + 1]), sl2, negM));
                        float const e2 = ex2Approx(fmaf(__uint_as_float(x[i + 2]), sl2, negM));
                        float const e3 = ex2Approx(fmaf(__uint_as_float(x[i + 3]), sl2, negM));
                        l0 += e0;
                        l1 += e1;
                        l2 += e2;
                        l3 += e3;
                        p[i / 2] = packHalf2(e0, e1);
                        p[i / 2 + 1] = packHalf2(e2, e3);
                    }
                };
                {
                    uint32_t pa[16], pb[16];
                    TR_EVT(13);
                    expChunk(x0, pa);
                    expChunk(x1, pb);
                    TR_EVT(14);
                    // The P columns are read by the previous block's product and the context accumulator by the previous
                    // tile's epilogue: half a block of exponentials later both are long done.
                    if (pending)
                        epilogue();
                    else if (blocks > 0)
                        ok = ok && mbarWait(&pvDone[s], (blocks - 1) & 1u, abortFlag, kWaitAccFull);
                    TR_EVT(15);
                    tmemStore16(tP, pa);
                    tmemStore16(tP + 16, pb);
                    expChunk(x2, pa);
                    tmemStore16(tP + 32, pa);
                    expChunk(x3, pb);
                    tmemStore16(tP + 48, pb);
                    TR_EVT(16);
                }
                tmemStoreWait();
                tcFenceBefore();
                __syncwarp();
                if (lane == 0)
                    mbarArrive(&pReady[s]);
                TR_EVT(17);
                ++blocks;
            }
            int const q = w.t * kTile + r;
            pending = true;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(pendInv) : "f"((l0 + l1) + (l2 + l3)));
            pendDst = nullptr;
            if (q < g.rows)
            {
                if (BNSD)
                    pendDst = static_cast<__half*>(args.out) + ((static_cast<int64_t>(g.b) * args.N + g.head) * args.S + q) * args.d;
                else
                {
                    int64_t const rr = args.fixedLayout ? static_cast<int64_t>(q) * args.B + g.b : static_cast<int64_t>(g.rowBase) + q;
                    pendDst = static_cast<__half*>(args.out) + rr * args.N * args.d + g.head * args.d;
                }
            }
            active = w.next() && w.next();
        }
        if (pending)
            epilogue();
        tcFenceBefore();
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
    if (warp == 8)
    {
        __syncwarp();
        tcFenceAfter();
        tmemFree(tmemBase, kTmemCols);
    }
}

// Query tiles per work unit: all tiles of a (sequence, head) share one load of K / V, so whole items are the
// cheapest units; they are cut into smaller ones only when that shortens the longest CTA's list.
int32_t chooseTilesPerUnit(int64_t items, int32_t nqMax, int32_t sms)
{
    int32_t best = nqMax;
    int64_t bestCost = ((items + sms - 1) / sms) * nqMax;
    for (int32_t tpu = nqMax - 1; tpu >= 1; --tpu)
    {
        int64_t const chunks = (nqMax + tpu - 1) / tpu;
        int64_t const cost = ((items * chunks + sms - 1) / sms) * tpu;
        if (cost < bestCost)
        {
            bestCost = cost;
            best = tpu;
        }
    }
    return best;
}

template <bool BNSD>
int32_t launchOnline(CUtensorMap const (&maps)[3], OnlineArgs args, cudaStream_t stream)
{
    auto kernel = mhaOnlineF16Kernel<BNSD>;
    cudaError_t const e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "mha: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    int32_t const nqMax = (args.S + kTile - 1) / kTile;
    int64_t const items = static_cast<int64_t>(args.B) * args.N;
    args.tilesPerUnit = chooseTilesPerUnit(items, nqMax, smCount());
    args.chunks = (nqMax + args.tilesPerUnit - 1) / args.tilesPerUnit;
    int64_t const units = items * args.chunks;
    if (units > INT32_MAX)
        B200_FAIL(BERT_B200_NOT_SUPPORTED, "mha: too many work units (%lld)", static_cast<long long>(units));
    int const grid = static_cast<int>(units < smCount() ? units : smCount());
    args.stepChunk = grid % args.chunks;
    args.stepHead = (grid / args.chunks) % args.N;
    args.stepB = (grid / args.chunks) / args.N;
    cudaError_t const le = launchDependent(kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, maps[0], maps[1], maps[2], args);
    if (le != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "mhaOnlineF16Kernel: %s", cudaGetErrorString(le));
    return checkLaunch("mhaOnlineF16Kernel");
}

} // namespace

// FP16, head sizes 16 / 32 / 48 / 64, fused [N][3][d] tensor in the fixed or the packed layout.
int32_t mhaOnlineF16(bert_b200_mha_params const& p, cudaStream_t stream)
{
    bool const fixedLayout = p.cu_seqlens == nullptr;
    uint64_t const d = static_cast<uint64_t>(p.head_size);
    uint64_t const rowElems = 3ull * static_cast<uint64_t>(p.num_heads) * d;
    // dim0: the d channels of one of Q, K, V of a head (the box is 64 wide: channels beyond d arrive as zeros);
    // dim1: which of [N][3]; dim2: batch (fixed layout only); dim3: sequence position / packed row
    uint64_t const dims[4] = {d, 3ull * static_cast<uint64_t>(p.num_heads), fixedLayout ? static_cast<uint64_t>(p.B) : 1ull,
        fixedLayout ? static_cast<uint64_t>(p.S) : static_cast<uint64_t>(p.total)};
    uint64_t const strides[3] = {d * 2, rowElems * 2, (fixedLayout ? static_cast<uint64_t>(p.B) : 1ull) * rowElems * 2};
    uint32_t const box[4] = {kHeadSize, 1, 1, kTile};
    CUtensorMap maps[3];
    int32_t const st = makeTensorMap(&maps[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, p.qkv, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != BERT_B200_OK)
        return st;
    maps[1] = maps[0];
    maps[2] = maps[0];
    OnlineArgs const args{p.B, p.S, p.num_heads, p.total, p.head_size, fixedLayout ? 1 : 0, p.out, p.cu_seqlens, p.mask_idx,
        p.scale_bmm1, p.status_word, 1, 1, 0, 0, 0};
    return launchOnline<false>(maps, args, stream);
}

// Separate Q, K, V tensors of shape [B][N][S][d] (the operand layout of TensorRT's attention layer), output
// [B][N][S][d]: three tensor maps, the same kernel.
int32_t mhaOnlineF16Bnsd(bert_b200_attention_bnsd_params const& p, cudaStream_t stream)
{
    uint64_t const d = static_cast<uint64_t>(p.head_size), S = static_cast<uint64_t>(p.S), N = static_cast<uint64_t>(p.num_heads);
    CUtensorMap maps[3];
    void const* const base[3] = {p.q, p.k, p.v};
    for (int i = 0; i < 3; ++i)
    {
        uint64_t const dims[4] = {d, S, N, static_cast<uint64_t>(p.B)};
        uint64_t const strides[3] = {d * 2, S * d * 2, N * S * d * 2};
        uint32_t const box[4] = {kHeadSize, kTile, 1, 1};
        int32_t const st = makeTensorMap(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, base[i], dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != BERT_B200_OK)
            return st;
    }
    OnlineArgs const args{p.B, p.S, p.num_heads, 0, p.head_size, 1, p.out, nullptr, p.kv_lengths, p.scale_bmm1, p.status_word, 1, 1, 0, 0, 0};
    return launchOnline<true>(maps, args, stream);
}

} // namespace b200

// INT8 fused multi-head attention on the sm_100a tensor cores (head sizes 16, 32, 48, 64; sequence length <= 512),
// fixed [S,B,N,3,d], packed [total,N,3,d] and INT8 CHW32-interleaved layouts, and the C entry points of both
// attention kernels (FP16 runs the online-softmax kernel of mha_f16_online.cu).
//
// Replaces the precompiled fused INT8 attention kernels the reference launches through
// FusedMHARunnerInt8[v2]::run (plugin/bertQKVToContextPlugin/mhaRunner.cu:835-860, 1127-1265) and the head-size
// padding copies (zeroPadding2d.cu:190-204: here the TMA unit zero-fills the channels beyond the head size).
//
// The quantised probabilities P_q = rni(p / rowsum * scale_softmax) need the exact row maximum and the complete row
// sum before the first of them can be formed, so the whole score row lives in TMEM (<= 512 keys) and the softmax makes
// three sweeps over it; that is what keeps the result bit-identical with the reference's INT8 kernels.
//
// Persistent CTAs (one per SM) take (sequence, head) work items round-robin. Per item a CTA loops over the 128-query
// tiles of the sequence, so that K and V are loaded once and the tensor pipe works on the next tile (of this item or
// the next) while the softmax warps finish the current one. 19 warps:
//   warp 0    : TMA - the K / V blocks (128 keys each) of an item once, the Q tile of each iteration
//               (swizzled shared-memory tiles, one mbarrier each).
//   warp 1    : TMEM allocation (512 columns); one lane issues the context products
//                 O  += P_j V_j           (128 x 64, accumulator in TMEM columns 384..447; for S > 384 it re-uses
//                                          the columns of S_0, which serialises consecutive tiles)
//   warp 18   : one lane issues the scores of the following tile, per key block as soon as the softmax warps hold
//               the current S_j in registers:
//                 S_j = Q K_j^T           (128 x 128 per key block, accumulators in TMEM columns 128j..)
//               (with a single key block per sequence warp 1 issues both and this warp idles).
//   warps 2-17: softmax, four threads per query row (each owns 32 of every 128 key columns):
//                 pass A  row maximum over all key blocks straight from TMEM (integer maximum, no conversions),
//                 pass B  p = exp2((x - max) * scale * log2e), row sum; the exponentials go back to TMEM,
//                 pass C  P_q = rni(p / sum * scale_softmax) -> INT8 P_j into swizzled shared memory for the PV product,
//                 epilogue O * scale_bmm2, round, saturate -> 128-bit global stores, deferred until after pass A of
//                         the next tile.
//               The passes loop over the key blocks (not unrolled): unrolled, the kernel was bound by instruction
//               fetch (122 KB of text, 77 % instruction-cache hits).
// The kernel template also takes FP16 tensors (exact-maximum two-sweep form, P in shared memory); that instantiation
// is not built.
// Every wait is bounded (sm100.cuh); on expiry the CTA drains, frees TMEM, reports through the status word.
#include "sm100.cuh"

#include <cstdlib>
#include <type_traits>

namespace b200
{

int32_t mhaSimt(bert_b200_mha_params const& p, cudaStream_t stream);
int32_t mhaOnlineF16(bert_b200_mha_params const& p, cudaStream_t stream);
int32_t mhaOnlineF16Bnsd(bert_b200_attention_bnsd_params const& p, cudaStream_t stream);

namespace
{

constexpr int kQTile = 128;
constexpr int kKeyBlock = 128;
constexpr int kHeadSize = 64;
constexpr int kMaxBlocks = 4; // S <= 512
constexpr int kMhaThreads = 608;     // TMA warp, MMA warp, 16 softmax warps, second MMA warp (FP16)
constexpr int kSoftmaxThreads = 512;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kOColumn = 384;   // context accumulator when the scores need at most 384 columns

struct MhaArgs
{
    int32_t B, S, N, total;
    int32_t d; // head size: 16, 32, 48 or 64; the tiles are always 64 wide, TMA fills the missing channels with zeros
    int32_t fixedLayout;
    void* out;
    int32_t const* cu;
    int32_t const* maskIdx;
    float scaleBmm1, scaleSoftmax, scaleBmm2;
    uint32_t* statusWord;
};

template <typename T>
struct MhaSmem
{
    static constexpr int kElem = sizeof(T);
    static constexpr int kRowBytes = kHeadSize * kElem;           // 128 (FP16) or 64 (INT8)
    static constexpr int kTileBytes = kQTile * kRowBytes;         // Q tile, one K block, one V block
    static constexpr int kPBytes = kQTile * kKeyBlock * kElem;    // one P block: 32 KB (FP16) or 16 KB (INT8)
    // [ Q ][ K blocks ][ V blocks ][ P slots ][ barriers, reduction scratch ]
    static __host__ __device__ constexpr int kOffset()
    {
        return kTileBytes;
    }
    static __host__ __device__ constexpr int vOffset(int nb)
    {
        return (1 + nb) * kTileBytes;
    }
    static __host__ __device__ constexpr int pOffset(int nb)
    {
        return (1 + 2 * nb) * kTileBytes;
    }
    // one P slot per key block up to three blocks; four blocks share two slots (shared memory is full then)
    static __host__ __device__ constexpr int pSlots(int nb)
    {
        return nb <= 3 ? nb : 2;
    }
    static __host__ __device__ constexpr int barrierOffset(int nb)
    {
        return pOffset(nb) + pSlots(nb) * kPBytes;
    }
    // kFull[4] vFull[4] sFull[4] pReady[4] pFree[4] sFree[4] qFull qFree oFull oFree vFree, tmem slot + abort flag, max / sum scratch
    static constexpr int kBarrierBytes = (6 * kMaxBlocks + 5) * 8 + 16 + 8 * kQTile * 4;
    static __host__ __device__ constexpr int dynamicBytes(int nb)
    {
        return barrierOffset(nb) + kBarrierBytes + 1024;
    }
};

__device__ __forceinline__ float ex2Approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Four non-negative values -> round-to-nearest-even integers saturated at 127, packed into one word.
// Adding 1.5 * 2^23 leaves the rounded integer in the low mantissa bits (the FP32 adder rounds to nearest even,
// like cvt.rni); the clamp at 127 is the saturation of the reference's conversion for scale_softmax > 127.
// kClamp = false: the caller knows that no value exceeds 127.49 (scale_softmax <= 127 and p <= 1).
template <bool kClamp>
__device__ __forceinline__ uint32_t packProb4(float a, float b, float c, float d)
{
    constexpr float kMagic = 12582912.f;
    if (kClamp)
    {
        a = fminf(a, 127.f);
        b = fminf(b, 127.f);
        c = fminf(c, 127.f);
        d = fminf(d, 127.f);
    }
    uint32_t const ua = __float_as_uint(a + kMagic), ub = __float_as_uint(b + kMagic);
    uint32_t const uc = __float_as_uint(c + kMagic), ud = __float_as_uint(d + kMagic);
    return __byte_perm(__byte_perm(ua, ub, 0x0040), __byte_perm(uc, ud, 0x0040), 0x5410);
}

// The row reductions only join the four warps that own the columns of the same 32 query rows (one TMEM lane
// quadrant). FP16: one named barrier per quadrant, so that the quadrants drift apart instead of waiting for the
// slowest (+6 % at S = 384). INT8: all sixteen warps in step - its per-key-block hand-overs to the MMA threads need
// every warp's arrival anyway, and drifting quadrants delay them (per-quadrant barriers: -4 %).
template <bool kPerQuadrant>
__device__ __forceinline__ void softmaxBarrier(int quad)
{
    if (kPerQuadrant)
        asm volatile("bar.sync %0, 128;" ::"r"(1 + quad) : "memory");
    else
        asm volatile("bar.sync 1, 512;" ::: "memory");
}

__device__ __forceinline__ void tmemStore32(uint32_t taddr, uint32_t const (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmemStoreWait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// IL (INT8 only): CHW32-interleaved tensors. Q, K and V tiles then arrive as two 32-channel sub-tiles of
// [128 tokens][32 B] (32-byte swizzle); the head dimension is covered by one MMA per sub-tile.
// BNSD: Q, K and V are three separate [B][N][S][d] tensors (mapQkv, mapK, mapV) and the output is [B][N][S][d];
// otherwise mapQkv covers the fused tensor and the other two maps are not used.
template <typename T, bool IL, bool BNSD>
__global__ void __launch_bounds__(kMhaThreads, 1)
    mhaTcgen05Kernel(const __grid_constant__ CUtensorMap mapQkv, const __grid_constant__ CUtensorMap mapK,
        const __grid_constant__ CUtensorMap mapV, MhaArgs const args)
{
    static_assert(!BNSD || !IL, "separate Q / K / V tensors: linear layout");
    using L = MhaSmem<T>;
    constexpr bool kInt8 = sizeof(T) == 1;
    static_assert(!IL || kInt8, "the interleaved layout is INT8 only");
    // Q, K, V rows are 128 B (FP16), 64 B (INT8) or 32 B (interleaved INT8 sub-tiles)
    constexpr uint64_t kSwz = IL ? kSwizzle32B : (kInt8 ? kSwizzle64B : kSwizzle128B);
    constexpr uint32_t kAtomBytes = IL ? 256u : 8 * L::kRowBytes; // 8 rows of a swizzle atom: SBO
    constexpr uint32_t kSubTile = L::kTileBytes / 2;              // interleaved: bytes of one 32-channel sub-tile
    constexpr int kQkMmas = kInt8 ? 2 : 4;                        // head size 64 = 2 x 32 (INT8) or 4 x 16 (FP16)
    constexpr int kPvMmas = kInt8 ? 4 : 8;                        // 128 keys = 4 x 32 or 8 x 16
    constexpr uint32_t kIdescQk = makeInstrDesc(kInt8 ? 2u : 1u, kInt8 ? 1u : 0u, 0u, 0u, 128u, 128u);
    constexpr uint32_t kIdescPv = makeInstrDesc(kInt8 ? 2u : 1u, kInt8 ? 1u : 0u, 0u, 1u, 128u, 64u);

    int const warp = threadIdx.x >> 5;
    int const lane = threadIdx.x & 31;

    // ---- work items: one (sequence, head) each, item = b * N + head, dealt round-robin to the persistent CTAs ----
    struct Item
    {
        int32_t b, head, rowBase, rows, len, nb, nq;
    };
    int const numItems = args.B * args.N;
    // Geometry of item i (uniform over the CTA; every role derives the same values). Returns whether the item has
    // work for the tensor pipeline (at least one query row and one valid key).
    auto getItem = [&](int i, Item& it) -> bool {
        it.b = i / args.N;
        it.head = i - it.b * args.N;
        if (args.fixedLayout)
        {
            it.rowBase = 0;
            it.rows = args.S;
            it.len = args.maskIdx ? min(max(__ldg(args.maskIdx + it.b), 0), args.S) : args.S;
        }
        else
        {
            it.rowBase = __ldg(args.cu + it.b);
            it.len = min(max(__ldg(args.cu + it.b + 1) - it.rowBase, 0), args.S);
            it.rows = it.len;
        }
        it.nb = (it.len + kKeyBlock - 1) / kKeyBlock; // key blocks
        it.nq = (it.rows + kQTile - 1) / kQTile;      // query tiles
        return it.rows > 0 && it.len > 0;
    };
    // first item >= i of this CTA's sequence that has pipeline work; numItems or more if there is none
    auto nextWork = [&](int i, Item& it) -> int {
        while (i < numItems && !getItem(i, it))
            i += gridDim.x;
        return i;
    };

    // The layout of shared memory and TMEM follows the longest sequence the launch admits.
    int const nbMax = (args.S + kKeyBlock - 1) / kKeyBlock;
    // S > 384: the context accumulator has to share TMEM columns with the scores of key block 0
    bool const oAliasesScores = nbMax > 3;
    uint32_t const oCol = oAliasesScores ? 0u : kOColumn;
    auto slotOf = [&](int j) { return nbMax <= 3 ? j : (j & 1); };

    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sQ = smem;                          // kTileBytes
    uint8_t* sK = smem + L::kOffset();           // nbMax x kTileBytes
    uint8_t* sV = smem + L::vOffset(nbMax);      // nbMax x kTileBytes
    uint8_t* sP = smem + L::pOffset(nbMax);      // pSlots(nbMax) x kPBytes
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::barrierOffset(nbMax));
    uint64_t* kFull = bars;                      // [4] K_j landed                        (once per item using block j)
    uint64_t* vFull = bars + kMaxBlocks;         // [4] V_j landed                        (once per item using block j)
    uint64_t* sFull = bars + 2 * kMaxBlocks;     // [4] scores of block j complete        (once per tile using block j)
    uint64_t* pReady = bars + 3 * kMaxBlocks;    // [4] P_j written, 512 arrivals         (once per tile using block j)
    uint64_t* pFree = bars + 4 * kMaxBlocks;     // [4] PV product consumed P slot        (once per fill of the slot)
    uint64_t* sFree = bars + 5 * kMaxBlocks;     // [4] softmax holds S_j in registers, 512 arrivals (once per tile using block j)
    uint64_t* qFull = sFree + kMaxBlocks;        // Q tile landed                         (once per tile)
    uint64_t* qFree = qFull + 1;                 // all score MMAs of the tile done: Q slot (after an item's last tile: K) reusable
    uint64_t* oFull = qFree + 1;                 // context accumulator complete          (once per tile)
    uint64_t* oFree = oFull + 1;                 // epilogue has read it, 512 arrivals    (once per tile)
    uint64_t* vFree = oFree + 1;                 // all PV products of an item done: V reusable (once per item)
    uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(vFree + 1);
    volatile uint32_t* abortFlag = tmemSlot + 1;
    float* rowRed = reinterpret_cast<float*>(tmemSlot + 4); // [2][4][128]: max then sum, per 32-column owner

    if (threadIdx.x == 0)
    {
        for (int i = 0; i < kMaxBlocks; ++i)
        {
            mbarInit(&kFull[i], 1);
            mbarInit(&vFull[i], 1);
            mbarInit(&sFull[i], 1);
            mbarInit(&pReady[i], kSoftmaxThreads);
        }
        for (int i = 0; i < kMaxBlocks; ++i)
        {
            mbarInit(&pFree[i], 1);
            mbarInit(&sFree[i], kSoftmaxThreads);
        }
        mbarInit(qFull, 1);
        mbarInit(qFree, 1);
        mbarInit(oFull, 1);
        mbarInit(oFree, kSoftmaxThreads);
        mbarInit(vFree, 1);
        *abortFlag = 0;
        fenceBarrierInit();
        prefetchTensorMap(&mapQkv);
        if (BNSD)
        {
            prefetchTensorMap(&mapK);
            prefetchTensorMap(&mapV);
        }
    }
    if (warp == 1)
        tmemAlloc(tmemSlot, kTmemCols);
    tcFenceBefore();
    __syncthreads();
    tcFenceAfter();
    uint32_t const tmemBase = *tmemSlot;
    // set-up done: the next kernel of the stream may start its own; the inputs of this one must be complete
    gridDependencyLaunch();
    gridDependencyWait();

    // Barriers that complete once per tile (qFull, qFree, oFull, oFree) are waited on with the parity of the CTA's
    // running tile count; those that complete once per use of key block j keep one parity bit per block.
    if (warp == 0)
    {
        if (lane == 0)
        {
            Item it;
            uint32_t tiles = 0;       // Q tiles requested so far
            uint32_t itemsLoaded = 0; // items whose K / V have been requested
            bool ok = true;
            for (int item = nextWork(blockIdx.x, it); item < numItems && ok; item = nextWork(item + gridDim.x, it))
            {
                int32_t const rowK = args.fixedLayout ? 0 : it.rowBase;
                int32_t const rowKv = rowK; // first key of this item
                // linear: (channel, which of [N][3], batch, row). interleaved: (channel, row, 32-channel group, which of [3][N])
                auto load = [&](uint8_t* dst, uint64_t* bar, int which, int32_t row) {
                    if (BNSD) // (channel, position, head, sequence) of the tensor `which` selects
                        tmaLoad4d(dst, which == 0 ? &mapQkv : (which == 1 ? &mapK : &mapV), bar, 0, row, it.head, it.b);
                    else if (IL)
                        tmaLoad4d(dst, &mapQkv, bar, 0, row, 0, which * args.N + it.head);
                    else
                        tmaLoad4d(dst, &mapQkv, bar, 0, it.head * 3 + which, args.fixedLayout ? it.b : 0, row);
                };
                for (int t = 0; t < it.nq && ok; ++t)
                {
                    // the score MMAs of the previous tile have read Q (and, across items, K)
                    if (tiles > 0)
                        ok = mbarWait(qFree, (tiles - 1) & 1, abortFlag, kWaitStageFree);
                    if (!ok)
                        break;
                    mbarArriveExpectTx(qFull, L::kTileBytes);
                    load(sQ, qFull, 0, rowK + t * kQTile);
                    if (t == 0)
                    {
                        for (int j = 0; j < it.nb; ++j)
                        {
                            mbarArriveExpectTx(&kFull[j], L::kTileBytes);
                            load(sK + j * L::kTileBytes, &kFull[j], 1, rowKv + j * kKeyBlock);
                        }
                        // The PV products of the previous item have read V. (Not oFull: this thread may run ahead of
                        // or behind the per-tile barriers by more than one phase, and a parity wait is only meaningful
                        // for the very next phase; vFree completes once per item, in step with this loop.)
                        if (itemsLoaded > 0)
                            ok = mbarWait(vFree, (itemsLoaded - 1) & 1, abortFlag, kWaitStageFree);
                        if (!ok)
                            break;
                        for (int j = 0; j < it.nb; ++j)
                        {
                            mbarArriveExpectTx(&vFull[j], L::kTileBytes);
                            load(sV + j * L::kTileBytes, &vFull[j], 2, rowKv + j * kKeyBlock);
                        }
                    }
                    ++tiles;
                }
                ++itemsLoaded;
            }
        }
    }
    else if (warp == 1 || warp == kMhaThreads / 32 - 1)
    {
        // ---- MMA issue: scores S_j = Q K_j^T of the tile after the one the softmax warps work on, and
        //      context_t += P_j V_j as they hand over P_j ----
        // Every tcgen05.mma / tcgen05.commit keeps its issuing thread busy for some 50 cycles (measured), and one
        // thread issuing both products of a tile was the slowest link of the tile pipeline: the scores are issued by
        // a second thread in the last warp (+11 % at S = 384). Sequences of a single key block have too few MMAs per
        // tile for that to pay (INT8, S = 128: -7 %) and keep one issuer.
        bool const twoIssuers = !kInt8 || nbMax > 1;
        // Operand descriptors are formed arithmetically: one low word per operand tile (+ bytes >> 4 per key block
        // and MMA step, compile-time constants of the unrolled loops) and one high word per operand kind (mmaLoHi).
        auto issuer = [&](auto doScoresTag, auto doContextTag) {
            constexpr bool kDoScores = decltype(doScoresTag)::value;
            constexpr bool kDoContext = decltype(doContextTag)::value;
            bool ok = true;
            uint64_t const dQk = makeSmemDesc(0, 16, kAtomBytes, kSwz);
            // P: K-major, 128-byte rows, 128-byte swizzle. FP16 holds the block as two 64-key tiles.
            uint64_t const dP = makeSmemDesc(0, 16, 1024, kSwizzle128B);
            // V: MN-major (head dimension contiguous), one MMA consumes 16 (FP16) / 32 (INT8) key rows.
            // Interleaved: the two 32-channel sub-tiles are LBO apart, 32 key rows are 1024 bytes.
            uint64_t const dV = IL ? makeSmemDesc(0, kSubTile, kAtomBytes, kSwz) : makeSmemDesc(0, kAtomBytes, kAtomBytes, kSwz);
            uint32_t const hiQk = static_cast<uint32_t>(dQk >> 32), hiP = static_cast<uint32_t>(dP >> 32),
                           hiV = static_cast<uint32_t>(dV >> 32);
            uint32_t const qLo = static_cast<uint32_t>(dQk) + (smemAddr(sQ) >> 4);
            uint32_t const kLo = static_cast<uint32_t>(dQk) + (smemAddr(sK) >> 4);
            uint32_t const vLo = static_cast<uint32_t>(dV) + (smemAddr(sV) >> 4);
            uint32_t const pLo = static_cast<uint32_t>(dP) + (smemAddr(sP) >> 4);
            uint32_t const pPairStep = nbMax <= 3 ? 2u * (L::kPBytes >> 4) : 0u; // slotOf(j) = (j & 1) + (j >> 1) * (2 or 0)
            constexpr uint32_t kTile16 = L::kTileBytes >> 4;
            uint32_t qkTiles = 0;  // tiles whose scores have been issued
            uint32_t pvTiles = 0;  // tiles of this CTA that the loop below has passed (= whose context has been issued)
            uint32_t kBits = 0, vBits = 0, pBits = 0, fBits = 0; // parity per key block: K landed, V landed, P written, S read
            // scores of key block j for the query tile whose Q is in shared memory; nbOf = key blocks of that tile's item
            auto issueScores = [&](int j, int nbOf) {
#pragma unroll
                for (int k = 0; k < kQkMmas; ++k)
                {
                    uint32_t const off = (IL ? k * kSubTile : k * 32) >> 4; // next 32 bytes of the head dimension
                    mmaLoHi<kInt8>(tmemBase + j * kKeyBlock, qLo + off, hiQk, kLo + j * kTile16 + off, hiQk, kIdescQk, k != 0);
                }
                tcCommit(&sFull[j]);
                if (j == nbOf - 1)
                    tcCommit(qFree);
            };
            // first use of K_j by an item: wait for it to land
            auto waitK = [&](int j) -> bool {
                bool const got = mbarWait(&kFull[j], (kBits >> j) & 1u, abortFlag, kWaitTmaFull);
                kBits ^= 1u << j;
                return got;
            };
            Item cur, nxt;
            int item = nextWork(blockIdx.x, cur);
            if (kDoScores && item < numItems)
            {
                ok = mbarWait(qFull, 0, abortFlag, kWaitTmaFull);
#pragma unroll 1
                for (int j = 0; j < kMaxBlocks; ++j)
                {
                    if (j < cur.nb && ok)
                    {
                        ok = waitK(j);
                        if (ok)
                        {
                            tcFenceAfter();
                            issueScores(j, cur.nb);
                        }
                    }
                }
                qkTiles = 1;
            }
            while (item < numItems && ok)
            {
                // only the scores look one item ahead (its geometry comes from global memory: not in the way of a
                // thread that only issues context products)
                int const nextItem = kDoScores ? nextWork(item + gridDim.x, nxt) : numItems;
                for (int t = 0; t < cur.nq && ok; ++t)
                {
                    bool const lastT = t + 1 == cur.nq;
                    // the scores issued while this tile's context is formed: the item's next tile, or the first tile
                    // of the CTA's next item (whose K then has to have landed), or none
                    int const nbFollow = !lastT ? cur.nb : (nextItem < numItems ? nxt.nb : 0);
#pragma unroll 1
                    for (int j = 0; j < kMaxBlocks; ++j)
                    {
                        if (j < cur.nb && ok)
                        {
                            // Scores of the following tile for this key block first: they only need the softmax warps
                            // to hold this tile's S_j in registers (sFree), not the finished P_j, and the next pass A
                            // waits for them, while this tile's context is not read before the pass after.
                            if (kDoScores && j < nbFollow && !oAliasesScores)
                            {
                                if (j == 0)
                                    ok = mbarWait(qFull, qkTiles & 1, abortFlag, kWaitTmaFull);
                                if (ok && lastT)
                                    ok = waitK(j);
                                ok = ok && mbarWait(&sFree[j], (fBits >> j) & 1u, abortFlag, kWaitSoftmax);
                                if (ok)
                                {
                                    tcFenceAfter();
                                    issueScores(j, nbFollow);
                                }
                            }
                            fBits ^= 1u << j; // the softmax warps complete this phase in every tile that uses block j
                            if (kDoContext)
                            {
                                if (ok && t == 0)
                                {
                                    ok = mbarWait(&vFull[j], (vBits >> j) & 1u, abortFlag, kWaitTmaFull);
                                    vBits ^= 1u << j;
                                }
                                if (ok && j == 0 && pvTiles > 0) // the previous tile's context must have been read out
                                    ok = mbarWait(oFree, (pvTiles - 1) & 1, abortFlag, kWaitAccFree);
                                ok = ok && mbarWait(&pReady[j], (pBits >> j) & 1u, abortFlag, kWaitSoftmax);
                                pBits ^= 1u << j;
                                if (ok)
                                {
                                    tcFenceAfter();
                                    uint32_t const a = pLo + (j & 1) * (L::kPBytes >> 4) + (j >> 1) * pPairStep;
                                    uint32_t const b = vLo + j * kTile16;
#pragma unroll
                                    for (int k = 0; k < kPvMmas; ++k)
                                    {
                                        constexpr uint32_t kVStep = (IL ? 1024u : 2048u) >> 4;
                                        uint32_t const pOff = (kInt8 ? k * 32 : (k / 4) * (kQTile * 128) + (k % 4) * 32) >> 4;
                                        mmaLoHi<kInt8>(tmemBase + oCol, a + pOff, hiP, b + k * kVStep, hiV, kIdescPv, (j | k) != 0);
                                    }
                                    if (oAliasesScores) // otherwise every tile has its own P slots, released with oFull
                                        tcCommit(&pFree[slotOf(j)]);
                                    if (j == cur.nb - 1)
                                    {
                                        tcCommit(oFull);
                                        if (lastT)
                                            tcCommit(vFree);
                                    }
                                }
                            }
                        }
                    }
                    if (kDoScores && ok && !oAliasesScores)
                    {
                        // key blocks the next item has beyond this one's: their score columns are idle
#pragma unroll 1
                        for (int j = 1; j < kMaxBlocks; ++j)
                        {
                            if (j >= cur.nb && j < nbFollow && ok)
                            {
                                ok = waitK(j);
                                if (ok)
                                {
                                    tcFenceAfter();
                                    issueScores(j, nbFollow);
                                }
                            }
                        }
                    }
                    if (kDoScores && ok && nbFollow > 0 && oAliasesScores)
                    {
                        // the context accumulator occupies score columns: wait until the epilogue has read it
                        ok = mbarWait(oFree, pvTiles & 1, abortFlag, kWaitAccFree) && mbarWait(qFull, qkTiles & 1, abortFlag, kWaitTmaFull);
#pragma unroll 1
                        for (int j = 0; j < kMaxBlocks; ++j)
                        {
                            if (j < nbFollow && ok)
                            {
                                if (lastT)
                                    ok = waitK(j);
                                if (ok)
                                {
                                    tcFenceAfter();
                                    issueScores(j, nbFollow);
                                }
                            }
                        }
                    }
                    if (nbFollow > 0)
                        ++qkTiles;
                    ++pvTiles;
                }
                if (kDoScores)
                {
                    cur = nxt;
                    item = nextItem;
                }
                else
                    item = nextWork(item + gridDim.x, cur);
            }
        };
        if (lane == 0)
        {
            if (!twoIssuers)
            {
                if (warp == 1)
                    issuer(std::true_type{}, std::true_type{});
            }
            else if (warp == 1)
                issuer(std::false_type{}, std::true_type{});
            else
                issuer(std::true_type{}, std::false_type{});
        }
    }
    else if (warp < 2 + kSoftmaxThreads / 32)
    {
        int const quad = warp & 3;        // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may touch
        int const sub = (warp - 2) >> 2;  // which 32 of every 128 key columns this thread owns (4 warps per quadrant)
        int const r = quad * 32 + lane;   // query row inside the tile = TMEM lane
        uint32_t const tRow = tmemBase + (static_cast<uint32_t>(quad * 32) << 16);
        float const sl2 = args.scaleBmm1 * 1.4426950408889634f;
        constexpr float kMagic = 12582912.f;       // 1.5 * 2^23: as_float(0x4B400000 + v) == kMagic + v for |v| < 2^22
        constexpr uint32_t kMagicBits = 0x4B400000u;
        bool ok = true;
        auto colOf = [&](int j) { return j * kKeyBlock + sub * 32; };
        uint32_t tiles = 0;       // tiles this CTA has started
        uint32_t sBits = 0;       // parity per key block of sFull (and of this thread's arrivals on pReady)
        uint32_t slotFilled = 0;  // per P slot: has it been filled before ...
        uint32_t slotParity = 0;  // ... and the parity of the pFree phase that ends its latest fill
        // Before a P slot is refilled, the PV product that read its previous contents must have completed (pFree is only
        // signalled when four key blocks share two slots).
        auto acquireP = [&](int j) -> bool {
            // One slot per key block (up to three blocks): a slot is refilled one tile later, after this thread has
            // waited for the previous tile's complete context in its (deferred) epilogue - nothing to wait for.
            if (!oAliasesScores)
                return true;
            int const slot = slotOf(j);
            bool got = true;
            if ((slotFilled >> slot) & 1u)
            {
                got = mbarWait(&pFree[slot], (slotParity >> slot) & 1u, abortFlag, kWaitSoftmax);
                slotParity ^= 1u << slot;
            }
            slotFilled |= 1u << slot;
            return got;
        };
        // Reads 16 of the 64 context values of this row (tile number `tileNo` of the CTA), normalises / requantises
        // and stores them to `dst` (null: row beyond the sequence).
        auto epilogue = [&](uint32_t tileNo, T* dst, float inv) {
            if (ok)
                ok = mbarWait(oFull, tileNo & 1, abortFlag, kWaitAccFull);
            if (!ok)
                return;
            tcFenceAfter();
            uint32_t x[16];
            tmemLoad16(tRow + oCol + sub * 16, x);
            tmemLoadWait16(x);
            tcFenceBefore();
            mbarArrive(oFree);
            if (dst == nullptr)
                return;
            if (kInt8)
            {
                float const s2 = args.scaleBmm2;
                uint4 o;
                uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    w[i] = packChar4(static_cast<float>(static_cast<int32_t>(x[4 * i])) * s2,
                        static_cast<float>(static_cast<int32_t>(x[4 * i + 1])) * s2,
                        static_cast<float>(static_cast<int32_t>(x[4 * i + 2])) * s2,
                        static_cast<float>(static_cast<int32_t>(x[4 * i + 3])) * s2);
                *reinterpret_cast<uint4*>(dst) = o;
            }
            else
            {
#pragma unroll
                for (int g = 0; g < 2; ++g)
                {
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        f[i] = __uint_as_float(x[g * 8 + i]) * inv;
                    reinterpret_cast<uint4*>(dst)[g] = packHalf8(f);
                }
            }
        };

        // The epilogue of a tile runs after pass A of the CTA's next tile (of the same or the next item): the last PV
        // product then completes under useful work instead of a stall. Not possible when the context accumulator
        // shares columns with the scores.
        bool const deferEpilogue = !oAliasesScores;
        bool pending = false;
        T* pendDst = nullptr;
        float pendInv = 0.f;

        Item it;
        for (int item = blockIdx.x; item < numItems; item += gridDim.x)
        {
            bool const work = getItem(item, it);
            int64_t const outRowStride = static_cast<int64_t>(args.N) * args.d; // elements
            T* const outBase = static_cast<T*>(args.out) + static_cast<int64_t>(it.head) * args.d;
            // linear layouts: the d values of (token, head) are contiguous
            auto outRow = [&](int q) -> T* {
                if (BNSD)
                    return static_cast<T*>(args.out) + ((static_cast<int64_t>(it.b) * args.N + it.head) * args.S + q) * args.d;
                int64_t const rr = args.fixedLayout ? static_cast<int64_t>(q) * args.B + it.b : static_cast<int64_t>(it.rowBase) + q;
                return outBase + rr * outRowStride;
            };
            // interleaved output [N][d/32][total][32]: 32-channel group `grp` of (token, head)
            auto outPtrIl = [&](int q, int grp) -> T* {
                return static_cast<T*>(args.out)
                    + ((static_cast<int64_t>(it.head) * (args.d / 32) + grp) * args.total + it.rowBase + q) * 32;
            };
            if (!work)
            {
                // no valid key: every probability is zero and so is the context row
                int const kChunks = args.d * L::kElem / 16;
                for (int i = threadIdx.x - 64; i < it.rows * kChunks; i += kSoftmaxThreads)
                {
                    int const q = i / kChunks;
                    int const c = i % kChunks;
                    if (IL)
                        reinterpret_cast<uint4*>(outPtrIl(q, c / 2))[c % 2] = make_uint4(0, 0, 0, 0);
                    else
                        reinterpret_cast<uint4*>(outRow(q))[c] = make_uint4(0, 0, 0, 0);
                }
                continue;
            }
            int const nb = it.nb;
            int const len = it.len;
            for (int t = 0; t < it.nq; ++t)
            {
                uint32_t x[32];

                // ---- pass A: row maximum (INT8: integer maximum, no conversions) ----
                float mx = -INFINITY;
                int32_t mxi = INT32_MIN;
#pragma unroll 1
                for (int j = 0; j < nb; ++j)
                {
                    if (j < nb)
                    {
                        ok = ok && mbarWait(&sFull[j], (sBits >> j) & 1u, abortFlag, kWaitSoftmax);
                        tcFenceAfter();
                        tmemLoad32(tRow + colOf(j), x);
                        tmemLoadWait32(x);
                        int const limit = len - colOf(j);
                        if (limit >= 32)
                        {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                            {
                                if (kInt8)
                                    mxi = max(mxi, static_cast<int32_t>(x[i]));
                                else
                                    mx = fmaxf(mx, __uint_as_float(x[i]));
                            }
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                            {
                                if (i < limit)
                                {
                                    if (kInt8)
                                        mxi = max(mxi, static_cast<int32_t>(x[i]));
                                    else
                                        mx = fmaxf(mx, __uint_as_float(x[i]));
                                }
                            }
                        }
                    }
                }
                if (kInt8)
                    mx = mxi == INT32_MIN ? -INFINITY : static_cast<float>(mxi);
                if (pending)
                {
                    epilogue(tiles - 1, pendDst, pendInv);
                    pending = false;
                }
                rowRed[sub * kQTile + r] = mx;
                softmaxBarrier<!kInt8>(quad);
                mx = fmaxf(fmaxf(rowRed[r], rowRed[kQTile + r]), fmaxf(rowRed[2 * kQTile + r], rowRed[3 * kQTile + r]));
                float const mOff = mx * sl2;
                float const mxMagic = kMagic + mx; // exact: both are integers below 2^24

                // ---- pass B: exponentials, row sum; FP16 writes P here, INT8 parks exp values in TMEM ----
                float sum = 0.f;
#pragma unroll 1
                for (int j = 0; j < nb; ++j)
                {
                    if (j < nb)
                    {
                        tmemLoad32(tRow + colOf(j), x);
                        tmemLoadWait32(x);
                        if (!kInt8)
                        {
                            // the scores are in registers: their TMEM columns may take the next tile's scores
                            tcFenceBefore();
                            mbarArrive(&sFree[j]);
                        }
                        int const limit = len - colOf(j);
                        // INT8: (acc - max) is formed exactly (integers through the 2^23 trick, no conversion unit),
                        // so the exponent carries a single rounding; FP16: one fused multiply-add.
                        auto expOf = [&](uint32_t v) {
                            return kInt8 ? ex2Approx((__uint_as_float(v + kMagicBits) - mxMagic) * sl2)
                                         : ex2Approx(fmaf(__uint_as_float(v), sl2, -mOff));
                        };
                        if (limit >= 32) // all 32 keys valid: no per-element select
                        {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                            {
                                float const e = expOf(x[i]);
                                sum += e;
                                x[i] = __float_as_uint(e);
                            }
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                            {
                                float const e = i < limit ? expOf(x[i]) : 0.f;
                                sum += e;
                                x[i] = __float_as_uint(e);
                            }
                        }
                        if (kInt8)
                        {
                            tmemStore32(tRow + colOf(j), x);
                        }
                        else
                        {
                            ok = acquireP(j) && ok;
                            // FP16 P block = two [128 rows][64 keys] tiles of 128-byte rows; this thread owns 4 chunks of a row
                            uint8_t* pRow = sP + slotOf(j) * L::kPBytes + (sub >> 1) * (kQTile * 128) + r * 128;
#pragma unroll
                            for (int g = 0; g < 4; ++g)
                            {
                                float f[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    f[i] = __uint_as_float(x[g * 8 + i]);
                                int const chunk = (sub & 1) * 4 + g;
                                *reinterpret_cast<uint4*>(pRow + ((chunk ^ (r & 7)) << 4)) = packHalf8(f);
                            }
                            fenceProxyAsync();
                            tcFenceBefore();
                            mbarArrive(&pReady[j]);
                        }
                    }
                }
                if (kInt8)
                    tmemStoreWait();
                rowRed[4 * kQTile + sub * kQTile + r] = sum;
                softmaxBarrier<!kInt8>(quad);
                sum = (rowRed[4 * kQTile + r] + rowRed[5 * kQTile + r]) + (rowRed[6 * kQTile + r] + rowRed[7 * kQTile + r]);
                float const inv = 1.f / sum;

                if (kInt8)
                {
                    // ---- pass C (INT8): P_q = rni(p / sum * scale_softmax) ----
                    float const pq = inv * args.scaleSoftmax;
#pragma unroll 1
                    for (int j = 0; j < nb; ++j)
                    {
                        if (j < nb)
                        {
                            tmemLoad32(tRow + colOf(j), x);
                            tmemLoadWait32(x);
                            tcFenceBefore();
                            mbarArrive(&sFree[j]); // the parked exponentials are in registers: columns free for new scores
                            ok = acquireP(j) && ok;
                            uint8_t* pRow = sP + slotOf(j) * L::kPBytes + r * 128; // INT8 P block: [128 rows][128 keys]
#pragma unroll
                            for (int g = 0; g < 2; ++g)
                            {
                                uint4 o;
                                uint32_t* w = reinterpret_cast<uint32_t*>(&o);
                                // p / sum <= 1 (the sum contains p; a rounded-up reciprocal adds a few ulp at most), so
                                // with scale_softmax <= 127 nothing can round beyond 127 and the clamp is left out
                                if (args.scaleSoftmax <= 127.f)
                                {
#pragma unroll
                                    for (int i = 0; i < 4; ++i)
                                        w[i] = packProb4<false>(__uint_as_float(x[g * 16 + 4 * i]) * pq,
                                            __uint_as_float(x[g * 16 + 4 * i + 1]) * pq, __uint_as_float(x[g * 16 + 4 * i + 2]) * pq,
                                            __uint_as_float(x[g * 16 + 4 * i + 3]) * pq);
                                }
                                else
                                {
#pragma unroll
                                    for (int i = 0; i < 4; ++i)
                                        w[i] = packProb4<true>(__uint_as_float(x[g * 16 + 4 * i]) * pq,
                                            __uint_as_float(x[g * 16 + 4 * i + 1]) * pq, __uint_as_float(x[g * 16 + 4 * i + 2]) * pq,
                                            __uint_as_float(x[g * 16 + 4 * i + 3]) * pq);
                                }
                                int const chunk = sub * 2 + g; // 16 keys per 16-byte chunk
                                *reinterpret_cast<uint4*>(pRow + ((chunk ^ (r & 7)) << 4)) = o;
                            }
                            fenceProxyAsync();
                            tcFenceBefore();
                            mbarArrive(&pReady[j]);
                        }
                    }
                }
                sBits ^= (1u << nb) - 1u; // every block of this tile used its sFull / pReady phase
                int const q = t * kQTile + r;
                // this thread's 16 of the 64 context columns; columns >= d are the zero padding
                T* const dst = q >= it.rows || sub * 16 >= args.d
                    ? nullptr
                    : (IL ? outPtrIl(q, sub >> 1) + (sub & 1) * 16 : outRow(q) + sub * 16);
                ++tiles;
                if (deferEpilogue)
                {
                    pending = true;
                    pendDst = dst;
                    pendInv = inv;
                }
                else
                    epilogue(tiles - 1, dst, inv);
            }
        }
        if (pending)
            epilogue(tiles - 1, pendDst, pendInv);
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
    if (warp == 1)
    {
        __syncwarp();
        tcFenceAfter();
        tmemFree(tmemBase, kTmemCols);
    }
}

template <typename T, bool IL>
int32_t launchMha(bert_b200_mha_params const& p, cudaStream_t stream)
{
    using L = MhaSmem<T>;
    bool const fixedLayout = p.cu_seqlens == nullptr;
    uint64_t const d = static_cast<uint64_t>(p.head_size);
    uint64_t const rowElems = 3ull * static_cast<uint64_t>(p.num_heads) * d;
    // The boxes are always 64 channels wide (two 32-channel groups when interleaved); for a smaller head the channels
    // beyond d lie outside the tensor's channel dimension and arrive as zeros, which change neither Q.K nor P.V.
    CUtensorMap map;
    if (IL)
    {
        // [3][N][d/32][total][32]: dim0 the 32 channels of a group, dim1 the token, dim2 the group, dim3 which of [3][N]
        uint64_t const dims[4] = {32, static_cast<uint64_t>(p.total), d / 32, 3ull * static_cast<uint64_t>(p.num_heads)};
        uint64_t const strides[3] = {32, static_cast<uint64_t>(p.total) * 32, (d / 32) * static_cast<uint64_t>(p.total) * 32};
        uint32_t const box[4] = {32, kKeyBlock, 2, 1};
        int32_t const st = makeTensorMap(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, p.qkv, dims, strides, box,
            CU_TENSOR_MAP_SWIZZLE_32B);
        if (st != BERT_B200_OK)
            return st;
    }
    else
    {
        // dim0: the d channels of one of Q, K, V of a head; dim1: which of [N][3]; dim2: batch (fixed layout only);
        // dim3: sequence position / packed row
        uint64_t const dims[4] = {d, 3ull * static_cast<uint64_t>(p.num_heads), fixedLayout ? static_cast<uint64_t>(p.B) : 1ull,
            fixedLayout ? static_cast<uint64_t>(p.S) : static_cast<uint64_t>(p.total)};
        uint64_t const strides[3] = {d * sizeof(T), rowElems * sizeof(T),
            (fixedLayout ? static_cast<uint64_t>(p.B) : 1ull) * rowElems * sizeof(T)};
        uint32_t const box[4] = {kHeadSize, 1, 1, kKeyBlock};
        int32_t const st = makeTensorMap(&map, sizeof(T) == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
            4, p.qkv, dims, strides, box, sizeof(T) == 1 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != BERT_B200_OK)
            return st;
    }
    int const nbMax = (p.S + kKeyBlock - 1) / kKeyBlock;
    int const smem = L::dynamicBytes(nbMax);
    auto kernel = mhaTcgen05Kernel<T, IL, false>;
    cudaError_t const e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "mha: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    MhaArgs args{p.B, p.S, p.num_heads, p.total, p.head_size, fixedLayout ? 1 : 0, p.out, p.cu_seqlens, p.mask_idx, p.scale_bmm1,
        p.scale_softmax, p.scale_bmm2, p.status_word};
    // one persistent CTA per SM (512 TMEM columns and most of the shared memory each), items dealt round-robin
    int64_t const items = static_cast<int64_t>(p.num_heads) * p.B;
    int const grid = static_cast<int>(items < smCount() ? items : smCount());
    cudaError_t const le = launchDependent(kernel, dim3(grid), dim3(kMhaThreads), smem, stream, map, map, map, args);
    if (le != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "mhaTcgen05Kernel: %s", cudaGetErrorString(le));
    return checkLaunch("mhaTcgen05Kernel");
}

// Separate Q, K, V tensors of shape [B][N][S][d] (the operand layout of TensorRT's attention layer), output
// [B][N][S][d]: three tensor maps, the same kernel.
template <typename T>
int32_t launchMhaBnsd(bert_b200_attention_bnsd_params const& p, cudaStream_t stream)
{
    using L = MhaSmem<T>;
    uint64_t const d = static_cast<uint64_t>(p.head_size), S = static_cast<uint64_t>(p.S), N = static_cast<uint64_t>(p.num_heads);
    CUtensorMap maps[3];
    void const* const base[3] = {p.q, p.k, p.v};
    for (int i = 0; i < 3; ++i)
    {
        // dim0: channel (box 64 wide, zero-filled beyond d); dim1: position; dim2: head; dim3: sequence
        uint64_t const dims[4] = {d, S, N, static_cast<uint64_t>(p.B)};
        uint64_t const strides[3] = {d * sizeof(T), S * d * sizeof(T), N * S * d * sizeof(T)};
        uint32_t const box[4] = {kHeadSize, kKeyBlock, 1, 1};
        int32_t const st = makeTensorMap(&maps[i], sizeof(T) == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
            base[i], dims, strides, box, sizeof(T) == 1 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != BERT_B200_OK)
            return st;
    }
    int const nbMax = (p.S + kKeyBlock - 1) / kKeyBlock;
    int const smem = L::dynamicBytes(nbMax);
    auto kernel = mhaTcgen05Kernel<T, false, true>;
    cudaError_t const e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "attention_bnsd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    MhaArgs args{p.B, p.S, p.num_heads, 0, p.head_size, 1, p.out, nullptr, p.kv_lengths, p.scale_bmm1, p.scale_softmax,
        p.scale_bmm2, p.status_word};
    int64_t const items = static_cast<int64_t>(p.num_heads) * p.B;
    int const grid = static_cast<int>(items < smCount() ? items : smCount());
    cudaError_t const le = launchDependent(kernel, dim3(grid), dim3(kMhaThreads), smem, stream, maps[0], maps[1], maps[2], args);
    if (le != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "mhaTcgen05Kernel: %s", cudaGetErrorString(le));
    return checkLaunch("mhaTcgen05Kernel");
}

} // namespace

} // namespace b200

using namespace b200;

extern "C" int32_t bert_b200_attention_bnsd(bert_b200_attention_bnsd_params const* params, void* stream)
{
    B200_REQUIRE(params != nullptr, "attention_bnsd: null params");
    bert_b200_attention_bnsd_params const& p = *params;
    B200_REQUIRE(p.B >= 0 && p.S > 0 && p.num_heads > 0 && p.head_size > 0, "attention_bnsd: bad sizes B=%d S=%d N=%d d=%d", p.B,
        p.S, p.num_heads, p.head_size);
    B200_REQUIRE(p.q && p.k && p.v && p.out, "attention_bnsd: null pointer");
    if (p.B == 0)
        return BERT_B200_OK;
    B200_REQUIRE(p.B <= 65535 && p.num_heads <= 65535, "attention_bnsd: B and num_heads are limited to 65535");
    B200_REQUIRE(p.type_id == BERT_B200_FP16 || p.type_id == BERT_B200_INT8, "attention_bnsd: type_id %d", p.type_id);
    if (p.head_size > kHeadSize || p.head_size % 16 != 0)
        B200_FAIL(BERT_B200_NOT_SUPPORTED, "attention_bnsd: head sizes 16, 32, 48 and 64, got %d", p.head_size);
    if (p.S > kMaxBlocks * kKeyBlock && p.type_id == BERT_B200_INT8)
        B200_FAIL(BERT_B200_NOT_SUPPORTED, "attention_bnsd: INT8 takes S <= %d, got %d", kMaxBlocks * kKeyBlock, p.S);
    B200_REQUIRE(aligned16(p.q) && aligned16(p.k) && aligned16(p.v) && aligned16(p.out),
        "attention_bnsd: q, k, v and out must be 16-byte aligned");
    auto s = static_cast<cudaStream_t>(stream);
    if (p.type_id == BERT_B200_FP16)
    {
        B200_REQUIRE(p.scale_bmm1 > 0.f, "attention_bnsd: scale_bmm1 must be positive");
        return mhaOnlineF16Bnsd(p, s);
    }
    return launchMhaBnsd<int8_t>(p, s);
}

extern "C" int32_t bert_b200_mha(bert_b200_mha_params const* params, void* stream)
{
    B200_REQUIRE(params != nullptr, "mha: null params");
    bert_b200_mha_params const& p = *params;
    B200_REQUIRE(p.B >= 0 && p.S > 0 && p.num_heads > 0 && p.head_size > 0, "mha: bad sizes B=%d S=%d N=%d d=%d", p.B, p.S,
        p.num_heads, p.head_size);
    B200_REQUIRE(p.qkv && p.out, "mha: null pointer");
    B200_REQUIRE(p.cu_seqlens == nullptr || p.total >= 0, "mha: packed layout needs total >= 0");
    if (p.B == 0 || (p.cu_seqlens && p.total == 0))
        return BERT_B200_OK;
    B200_REQUIRE(p.B <= 65535 && p.num_heads <= 65535, "mha: B and num_heads are limited to 65535");
    auto s = static_cast<cudaStream_t>(stream);
    if (p.type_id == BERT_B200_FP32)
        return mhaSimt(p, s);
    B200_REQUIRE(p.type_id == BERT_B200_FP16 || p.type_id == BERT_B200_INT8, "mha: type_id %d", p.type_id);
    B200_REQUIRE(!p.interleaved || (p.type_id == BERT_B200_INT8 && p.cu_seqlens != nullptr),
        "mha: the interleaved (CHW32) layout needs INT8 and the packed (cu_seqlens) form");
    bool const headOk = p.head_size <= kHeadSize && p.head_size % 16 == 0 && (!p.interleaved || p.head_size % 32 == 0);
    bool const lengthOk = p.S <= kMaxBlocks * kKeyBlock;
    if (headOk && p.type_id == BERT_B200_FP16 && !p.interleaved && p.scale_bmm1 > 0.f)
    {
        B200_REQUIRE(aligned16(p.qkv) && aligned16(p.out), "mha: qkv and out must be 16-byte aligned");
        return mhaOnlineF16(p, s);
    }
    // Outside the tensor-core kernel's shapes FP16 takes the SIMT kernel, like the reference's unfused runner
    // (qkvToContextPlugin.cpp:335-341, 522-531); INT8 has no such path there either (qkvToContextPlugin.cpp:530).
    if (p.type_id == BERT_B200_FP16) // heads wider than 64 or not a multiple of 16 (or a non-positive scale)
        return mhaSimt(p, s);
    if (!headOk)
        B200_FAIL(BERT_B200_NOT_SUPPORTED,
            "mha: INT8 takes head sizes 16, 32, 48 and 64 (32 and 64 when interleaved), got %d", p.head_size);
    if (!lengthOk)
        B200_FAIL(BERT_B200_NOT_SUPPORTED, "mha: INT8 takes S <= %d, got %d", kMaxBlocks * kKeyBlock, p.S);
    B200_REQUIRE(aligned16(p.qkv) && aligned16(p.out), "mha: qkv and out must be 16-byte aligned");
    if (p.interleaved)
        return launchMha<int8_t, true>(p, s);
    return launchMha<int8_t, false>(p, s);
}

extern "C" int64_t bert_b200_mha_workspace_size(bert_b200_mha_params const* params)
{
    (void) params; // no attention kernel of this library needs scratch memory
    return 0;
}

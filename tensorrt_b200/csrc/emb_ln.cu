// Embedding gather (word + position + segment) + LayerNorm for sm_100a, plus the mask helpers the
// attention kernels consume (mask index, packed fragment mask, cu_seqlens).
//
// Replaces embLayerNormKernel / maskIdxKernel* / fillSBSMaskKernel
// (plugin/embLayerNormPlugin/embLayerNormKernel.cu:41-235) and embLayerNormKernelHFace/MTron
// (plugin/embLayerNormPlugin/embLayerNormVarSeqlenKernel{HFace,MTron}.cu:38-104).
//
// The reference launches one 256-thread CTA per (s, b) with 2-byte scalar loads and writes the
// un-normalised row to global memory before re-reading it. Here one token is owned by WPR warps,
// every lane keeps its CPL 16-byte chunks of the row in registers, the word row is streamed with
// 128-bit loads, and the row is written exactly once. The packed variant is token-parallel, so no
// CTA idles on the padding of a short sequence.
#include "common.cuh"

namespace b200
{
namespace
{

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;

template <typename T>
struct Chunk;
template <>
struct Chunk<__half>
{
    static constexpr int kElems = 8;
    static __device__ __forceinline__ void unpack(uint4 const& v, float (&f)[8])
    {
        unpackHalf8(v, f);
    }
    static __device__ __forceinline__ uint4 pack(float const (&f)[8])
    {
        return packHalf8(f);
    }
};
template <>
struct Chunk<float>
{
    static constexpr int kElems = 4;
    static __device__ __forceinline__ void unpack(uint4 const& v, float (&f)[4])
    {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ uint4 pack(float const (&f)[4])
    {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};

template <int WPR>
__device__ __forceinline__ float tokSum(float v, float* slot, int wInRow, int lane)
{
    v = warpSum(v);
    if (WPR == 1)
        return v;
    if (lane == 0)
        slot[wInRow] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w)
        t += slot[w];
    __syncthreads();
    return t;
}

// First s with mask[s][b] == 0 in column b of the [S, B] mask, S if there is none; one warp per sequence.
__device__ __forceinline__ void maskIdxOfSequence(int32_t const S, int32_t const B, int32_t const b, int const lane,
    int32_t const* __restrict__ mask, int32_t* __restrict__ maskIdx)
{
    int first = S;
    for (int base = 0; base < S && first == S; base += 32)
    {
        int const s = base + lane;
        bool const zero = s < S && mask[static_cast<int64_t>(s) * B + b] == 0;
        uint32_t const ballot = __ballot_sync(0xffffffffu, zero);
        if (ballot)
            first = base + __ffs(ballot) - 1;
    }
    if (lane == 0)
        maskIdx[b] = first;
}

// PACKED = false: token t = s*B + b, position s = t / B.
// PACKED = true : token t belongs to the sequence b with cu[b] <= t < cu[b+1]; position t - cu[b].
// PACKED = false with maskIdx != nullptr: `cuSeqlens` is the [S, B] input mask and the same launch also writes the mask
// index of every sequence (the second output of the fixed-length embedding plugin), one warp per sequence after the
// warp's share of the rows.
template <typename T, int CPL, int WPR, bool PACKED>
__global__ void __launch_bounds__(kThreads, 4) embLnKernel(int32_t const ld, int32_t const B, int32_t const tokens,
    int32_t const* __restrict__ inputIds, int32_t const* __restrict__ tokenIds, int32_t const* __restrict__ cuSeqlens,
    float const* __restrict__ beta, float const* __restrict__ gamma, T const* __restrict__ wordEmb,
    T const* __restrict__ posEmb, T const* __restrict__ tokEmb, int32_t const wordSize, int32_t const tokSize, int32_t const posSize,
    T* __restrict__ out, T* __restrict__ skipOut, int8_t* __restrict__ outI8, float const qScale,
    int32_t* __restrict__ maskIdx)
{
    constexpr int E = Chunk<T>::kElems;
    constexpr int kTokPerCta = kWarpsPerCta / WPR;
    __shared__ float red[kTokPerCta][WPR > 1 ? WPR : 1];

    int const lane = threadIdx.x & 31;
    int const warp = threadIdx.x >> 5;
    int const tokInCta = warp / WPR;
    int const wInRow = warp % WPR;
    int const chunksPerRow = ld / E;
    float const rld = 1.f / static_cast<float>(ld);

    int const tokensRounded = (tokens + kTokPerCta - 1) / kTokPerCta * kTokPerCta;
    // ids and position of token t (zeros beyond the last token)
    auto fetchIds = [&](int t, int& wordId, int& segId, int& pos) {
        wordId = 0, segId = 0, pos = 0;
        if (t < tokens)
        {
            wordId = __ldg(inputIds + t);
            segId = __ldg(tokenIds + t);
            if (PACKED)
            {
                // largest b with cu[b] <= t
                int lo = 0, hi = B;
                while (hi - lo > 1)
                {
                    int const mid = (lo + hi) >> 1;
                    if (__ldg(cuSeqlens + mid) <= t)
                        lo = mid;
                    else
                        hi = mid;
                }
                pos = t - __ldg(cuSeqlens + lo);
            }
            else
            {
                pos = t / B;
            }
        }
    };
    // The gather is a chain of two dependent reads per token (id, then the row): the ids of the warp's NEXT token are
    // fetched while the rows of the current one are in flight, so only the row read stays on the chain.
    int const tStride = gridDim.x * kTokPerCta;
    int nextWord, nextSeg, nextPos;
    fetchIds(blockIdx.x * kTokPerCta + tokInCta, nextWord, nextSeg, nextPos);
    for (int t = blockIdx.x * kTokPerCta + tokInCta; t < tokensRounded; t += tStride)
    {
        bool const tokOk = t < tokens;
        int const wordId = nextWord, segId = nextSeg, pos = nextPos;
        // ids or a position outside their tables (a sequence longer than the position table, a cu_seqlens that does not
        // start at 0 or runs backwards) read nothing: such a token produces the row `beta`
        bool const idOk = tokOk && wordId >= 0 && wordId < wordSize && segId >= 0 && segId < tokSize && pos >= 0 && pos < posSize;

        float x[CPL][E];
        float s = 0.f;
        uint4 w[CPL];
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            bool const ok = idOk && c < chunksPerRow;
            w[i] = ok ? ldgStream(wordEmb + static_cast<int64_t>(wordId) * ld + c * E) : make_uint4(0, 0, 0, 0);
        }
        if (t + tStride < tokensRounded)
            fetchIds(t + tStride, nextWord, nextSeg, nextPos);
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            bool const ok = idOk && c < chunksPerRow;
            Chunk<T>::unpack(w[i], x[i]);
            if (ok)
            {
                float p[E], g[E];
                Chunk<T>::unpack(ldgKeep(posEmb + static_cast<int64_t>(pos) * ld + c * E), p);
                Chunk<T>::unpack(ldgKeep(tokEmb + static_cast<int64_t>(segId) * ld + c * E), g);
                // the reference sums word + segment + position in the table type T
                // (plugin/embLayerNormPlugin/embLayerNormKernel.cu:222-225); FP32 here is at least as accurate
#pragma unroll
                for (int j = 0; j < E; ++j)
                    x[i][j] = x[i][j] + g[j] + p[j];
            }
#pragma unroll
            for (int j = 0; j < E; ++j)
                s += x[i][j];
        }
        float const mu = tokSum<WPR>(s, red[tokInCta], wInRow, lane) * rld;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            if (c < chunksPerRow)
            {
#pragma unroll
                for (int j = 0; j < E; ++j)
                {
                    float const d = x[i][j] - mu;
                    q += d * d;
                }
            }
        }
        float const var = tokSum<WPR>(q, red[tokInCta], wInRow, lane) * rld;
        // no epsilon (plugin/common/common.cuh:269); an all-zero row (ids outside the tables) yields beta
        float const rsigma = idOk ? rsqrtf(var) : 0.f;

#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            if (tokOk && c < chunksPerRow)
            {
                int64_t const off = static_cast<int64_t>(t) * ld + c * E;
                if (skipOut)
                    stgStream(skipOut + off, Chunk<T>::pack(x[i]));
                float y[E];
#pragma unroll
                for (int j4 = 0; j4 < E; j4 += 4)
                {
                    float4 const g = __ldg(reinterpret_cast<float4 const*>(gamma + c * E + j4));
                    float4 const bt = __ldg(reinterpret_cast<float4 const*>(beta + c * E + j4));
                    y[j4 + 0] = g.x * (x[i][j4 + 0] - mu) * rsigma + bt.x;
                    y[j4 + 1] = g.y * (x[i][j4 + 1] - mu) * rsigma + bt.y;
                    y[j4 + 2] = g.z * (x[i][j4 + 2] - mu) * rsigma + bt.z;
                    y[j4 + 3] = g.w * (x[i][j4 + 3] - mu) * rsigma + bt.w;
                }
                stgStream(out + off, Chunk<T>::pack(y));
                if (outI8)
                {
                    uint32_t words[E / 4];
#pragma unroll
                    for (int j4 = 0; j4 < E; j4 += 4)
                        words[j4 / 4] = packChar4(y[j4] * qScale, y[j4 + 1] * qScale, y[j4 + 2] * qScale, y[j4 + 3] * qScale);
                    uint32_t* dst = reinterpret_cast<uint32_t*>(outI8 + off);
#pragma unroll
                    for (int j = 0; j < E / 4; ++j)
                        dst[j] = words[j];
                }
            }
        }
    }
    if (!PACKED && maskIdx != nullptr)
    {
        for (int b = blockIdx.x * kWarpsPerCta + warp; b < B; b += gridDim.x * kWarpsPerCta)
            maskIdxOfSequence(tokens / B, B, b, lane, cuSeqlens, maskIdx);
    }
}

// Scalar version for row lengths that are not a multiple of the 16-byte chunk; one warp per token.
template <typename T, bool PACKED>
__global__ void __launch_bounds__(kThreads) embLnScalarKernel(int32_t const ld, int32_t const B, int32_t const tokens,
    int32_t const* __restrict__ inputIds, int32_t const* __restrict__ tokenIds, int32_t const* __restrict__ cuSeqlens,
    float const* __restrict__ beta, float const* __restrict__ gamma, T const* __restrict__ wordEmb,
    T const* __restrict__ posEmb, T const* __restrict__ tokEmb, int32_t const wordSize, int32_t const tokSize, int32_t const posSize,
    T* __restrict__ out, T* __restrict__ skipOut, int8_t* __restrict__ outI8, float const qScale,
    int32_t* __restrict__ maskIdx)
{
    int const lane = threadIdx.x & 31;
    int const warp = threadIdx.x >> 5;
    float const rld = 1.f / static_cast<float>(ld);
    for (int t = blockIdx.x * kWarpsPerCta + warp; t < tokens; t += gridDim.x * kWarpsPerCta)
    {
        int const wordId = inputIds[t];
        int const segId = tokenIds[t];
        int pos = t / B;
        if (PACKED)
        {
            int lo = 0, hi = B;
            while (hi - lo > 1)
            {
                int const mid = (lo + hi) >> 1;
                if (cuSeqlens[mid] <= t)
                    lo = mid;
                else
                    hi = mid;
            }
            pos = t - cuSeqlens[lo];
        }
        bool const idOk = wordId >= 0 && wordId < wordSize && segId >= 0 && segId < tokSize && pos >= 0 && pos < posSize;
        T const* wr = wordEmb + static_cast<int64_t>(wordId) * ld;
        T const* pr = posEmb + static_cast<int64_t>(pos) * ld;
        T const* tr = tokEmb + static_cast<int64_t>(segId) * ld;
        float s = 0.f;
        if (idOk)
            for (int i = lane; i < ld; i += 32)
                s += static_cast<float>(wr[i]) + static_cast<float>(tr[i]) + static_cast<float>(pr[i]);
        float const mu = warpSum(s) * rld;
        float q = 0.f;
        for (int i = lane; i < ld; i += 32)
        {
            float const v
                = idOk ? static_cast<float>(wr[i]) + static_cast<float>(tr[i]) + static_cast<float>(pr[i]) : 0.f;
            q += (v - mu) * (v - mu);
        }
        float const rsigma = idOk ? rsqrtf(warpSum(q) * rld) : 0.f;
        for (int i = lane; i < ld; i += 32)
        {
            float const v
                = idOk ? static_cast<float>(wr[i]) + static_cast<float>(tr[i]) + static_cast<float>(pr[i]) : 0.f;
            int64_t const off = static_cast<int64_t>(t) * ld + i;
            float const y = gamma[i] * (v - mu) * rsigma + beta[i];
            if (skipOut)
                skipOut[off] = static_cast<T>(v);
            out[off] = static_cast<T>(y);
            if (outI8)
                outI8[off] = quantChar(y * qScale);
        }
    }
    if (!PACKED && maskIdx != nullptr)
    {
        for (int b = blockIdx.x * kWarpsPerCta + warp; b < B; b += gridDim.x * kWarpsPerCta)
            maskIdxOfSequence(tokens / B, B, b, lane, cuSeqlens, maskIdx);
    }
}

// One warp per sequence: first s with mask[s][b] == 0, S if none.
__global__ void __launch_bounds__(kThreads) maskIdxKernel(int32_t const S, int32_t const B, int32_t const* __restrict__ mask,
    int32_t* __restrict__ maskIdx)
{
    int const b = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (b < B)
        maskIdxOfSequence(S, B, b, threadIdx.x & 31, mask, maskIdx);
}

// Bit layout of the reference fused-attention mask: see bert_b200_convert_mask in the header.
__global__ void packMaskKernel(uint32_t const warpsM, uint32_t const warpsN, uint32_t const S,
    int32_t const* __restrict__ maskSB, uint32_t* __restrict__ maskX)
{
    extern __shared__ int32_t shMask[];
    uint32_t const xmmasN = (S + 16 * warpsN - 1) / (16 * warpsN);
    uint32_t const threadsPerCta = blockDim.x;
    uint32_t const xmmasM = gridDim.x;
    uint32_t const B = gridDim.y;
    uint32_t const mi = blockIdx.x;
    uint32_t const bi = blockIdx.y;
    uint32_t const tidx = threadIdx.x;
    uint32_t const warpN = (tidx / 32) / warpsM;
    uint32_t const col = warpN * 16 + (tidx % 4) * 2;
    // positions beyond S read as masked (the reference leaves them uninitialised)
    uint32_t const padded = xmmasN * 16 * warpsN + 16;
    for (uint32_t si = tidx; si < padded; si += threadsPerCta)
        shMask[si] = si < S ? maskSB[static_cast<size_t>(si) * B + bi] : 0;
    __syncthreads();
    uint32_t bits = 0u;
    for (uint32_t ni = 0; ni < xmmasN; ++ni)
    {
        uint32_t const off = ni * 16 * warpsN + col;
        uint32_t const m0 = shMask[off + 0] == 1 ? 1u : 0u;
        uint32_t const m1 = shMask[off + 1] == 1 ? 1u : 0u;
        uint32_t const m8 = shMask[off + 8] == 1 ? 1u : 0u;
        uint32_t const m9 = shMask[off + 9] == 1 ? 1u : 0u;
        bits |= (m0 | (m1 << 1) | (m0 << 2) | (m1 << 3) | (m8 << 4) | (m9 << 5) | (m8 << 6) | (m9 << 7)) << (8 * ni);
    }
    maskX[(static_cast<size_t>(bi) * xmmasM + mi) * threadsPerCta + tidx] = bits;
}

// Inverse of packMaskKernel for prefix masks: lengths[b] = first key position whose bit is clear (S if none).
// Key s lives in row mi = 0, thread ((s % (16*warpsN)) / 16 * warpsM) * 32 + ((s % 8) / 2),
// bit 8 * (s / (16*warpsN)) + ((s % 16) >= 8 ? 4 : 0) + (s % 2).
__global__ void __launch_bounds__(kThreads) packedMaskToLengthsKernel(uint32_t const warpsM, uint32_t const warpsN,
    uint32_t const rowWords, int32_t const S, int32_t const B, uint32_t const* __restrict__ maskX, int32_t* __restrict__ lengths)
{
    int const lane = threadIdx.x & 31;
    int const b = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (b >= B)
        return;
    int first = S;
    for (int base = 0; base < S && first == S; base += 32)
    {
        int const s = base + lane;
        bool zero = false;
        if (s < S)
        {
            uint32_t const span = 16 * warpsN;
            uint32_t const ni = s / span;
            uint32_t const rem = s % span;
            uint32_t const t = (rem / 16) * warpsM * 32 + ((rem % 8) / 2);
            uint32_t const bit = 8 * ni + ((rem % 16) >= 8 ? 4u : 0u) + (rem % 2);
            zero = ((maskX[static_cast<size_t>(b) * rowWords + t] >> bit) & 1u) == 0u;
        }
        uint32_t const ballot = __ballot_sync(0xffffffffu, zero);
        if (ballot)
            first = base + __ffs(ballot) - 1;
    }
    if (lane == 0)
        lengths[b] = first;
}

// Single-CTA exclusive scan of up to 65536 lengths.
__global__ void __launch_bounds__(1024) cuSeqlensKernel(int32_t const B, int32_t const* __restrict__ lengths,
    int32_t* __restrict__ cu)
{
    __shared__ int32_t warpTotals[32];
    __shared__ int32_t carry;
    int const lane = threadIdx.x & 31;
    int const warp = threadIdx.x >> 5;
    if (threadIdx.x == 0)
    {
        carry = 0;
        cu[0] = 0;
    }
    __syncthreads();
    for (int base = 0; base < B; base += 1024)
    {
        int const i = base + threadIdx.x;
        int32_t v = i < B ? lengths[i] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            int32_t const n = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o)
                v += n;
        }
        if (lane == 31)
            warpTotals[warp] = v;
        __syncthreads();
        if (warp == 0)
        {
            int32_t w = warpTotals[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1)
            {
                int32_t const n = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o)
                    w += n;
            }
            warpTotals[lane] = w;
        }
        __syncthreads();
        int32_t const incl = v + (warp > 0 ? warpTotals[warp - 1] : 0) + carry;
        if (i < B)
            cu[i + 1] = incl;
        __syncthreads();
        if (threadIdx.x == 1023)
            carry = incl;
        __syncthreads();
    }
}

// Grid for a grid-stride loop over `groups` units of work with at most ctasPerSm CTAs per SM: every CTA takes the same
// number of passes (the last pass may be short for a few), instead of a grid of exactly the cap in which some CTAs
// make one pass more than the others and the rest idle meanwhile (24576 rows: 7 passes against 6 for a third of them).
inline int gridFor(int64_t groups, int ctasPerSm)
{
    int64_t const cap = static_cast<int64_t>(smCount()) * ctasPerSm;
    if (groups <= cap)
        return static_cast<int>(groups > 0 ? groups : 1);
    int64_t const passes = (groups + cap - 1) / cap;
    return static_cast<int>((groups + passes - 1) / passes);
}

template <typename T, bool PACKED>
int32_t dispatchEmb(cudaStream_t stream, int32_t ld, int32_t B, int32_t tokens, int32_t const* ids, int32_t const* seg,
    int32_t const* cu, float const* beta, float const* gamma, T const* word, T const* pos, T const* tok, int32_t wordSize,
    int32_t tokSize, int32_t posSize, T* out, T* skipOut, int8_t* outI8, float qScale, int32_t* maskIdx = nullptr)
{
    constexpr int E = 16 / sizeof(T);
    bool const vec = ld % E == 0 && ld / E <= 32 * 4 * 8 && aligned16(word) && aligned16(pos) && aligned16(tok)
        && aligned16(out) && (!skipOut || aligned16(skipOut)) && aligned16(beta) && aligned16(gamma)
        && (!outI8 || (reinterpret_cast<uintptr_t>(outI8) & 3u) == 0);
    if (!vec)
    {
        int const grid = gridFor((tokens + kWarpsPerCta - 1) / kWarpsPerCta, 8);
        embLnScalarKernel<T, PACKED><<<grid, kThreads, 0, stream>>>(ld, B, tokens, ids, seg, cu, beta, gamma, word, pos,
            tok, wordSize, tokSize, posSize, out, skipOut, outI8, qScale, maskIdx);
        return checkLaunch("embLnScalarKernel");
    }
    int const chunks = ld / E;
    int wpr = 1;
    while (chunks > 32 * 4 * wpr)
        wpr *= 2;
    int const cpl = (chunks + 32 * wpr - 1) / (32 * wpr);
#define B200_EMB_CASE(C, W)                                                                                            \
    if (cpl == C && wpr == W)                                                                                          \
    {                                                                                                                  \
        int const tokPerCta = kWarpsPerCta / W;                                                                        \
        int const grid = gridFor((tokens + tokPerCta - 1) / tokPerCta, 8);                                             \
        embLnKernel<T, C, W, PACKED><<<grid, kThreads, 0, stream>>>(ld, B, tokens, ids, seg, cu, beta, gamma, word,    \
            pos, tok, wordSize, tokSize, posSize, out, skipOut, outI8, qScale, maskIdx);                               \
        return checkLaunch("embLnKernel");                                                                             \
    }
    B200_EMB_CASE(1, 1)
    B200_EMB_CASE(2, 1)
    B200_EMB_CASE(3, 1)
    B200_EMB_CASE(4, 1)
    B200_EMB_CASE(3, 2)
    B200_EMB_CASE(4, 2)
    B200_EMB_CASE(3, 4)
    B200_EMB_CASE(4, 4)
    B200_EMB_CASE(3, 8)
    B200_EMB_CASE(4, 8)
#undef B200_EMB_CASE
    B200_FAIL(BERT_B200_NOT_SUPPORTED, "emb_layer_norm: no kernel for ld=%d", ld);
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int32_t bert_b200_emb_layer_norm_mask_idx(void* stream, int32_t type_id, int32_t ld, int32_t B, int32_t S,
    int32_t const* input_ids, int32_t const* token_ids, float const* beta, float const* gamma, void const* word_emb,
    void const* pos_emb, void const* tok_emb, int32_t word_size, int32_t tok_size, int32_t pos_size, void* output,
    int8_t* out_i8, float q_scale, int32_t const* mask, int32_t* mask_idx)
{
    B200_REQUIRE(ld > 0 && B >= 0 && S >= 0, "emb_layer_norm: bad sizes ld=%d B=%d S=%d", ld, B, S);
    B200_REQUIRE(static_cast<int64_t>(B) * S < (1ll << 31), "emb_layer_norm: B*S overflows int32");
    B200_REQUIRE(input_ids && token_ids && beta && gamma && word_emb && pos_emb && tok_emb && output,
        "emb_layer_norm: null pointer");
    B200_REQUIRE(word_size > 0 && tok_size > 0 && pos_size > 0, "emb_layer_norm: empty table");
    B200_REQUIRE(S <= pos_size, "emb_layer_norm: S=%d exceeds the position table (%d rows)", S, pos_size);
    B200_REQUIRE(mask_idx == nullptr || mask != nullptr || S == 0, "emb_layer_norm: mask_idx without a mask");
    if (B * S == 0)
        return mask_idx && B > 0 ? bert_b200_compute_mask_idx(stream, S, B, mask, mask_idx) : BERT_B200_OK;
    auto s = static_cast<cudaStream_t>(stream);
    if (type_id == BERT_B200_FP16)
        return dispatchEmb<__half, false>(s, ld, B, B * S, input_ids, token_ids, mask, beta, gamma,
            static_cast<__half const*>(word_emb), static_cast<__half const*>(pos_emb), static_cast<__half const*>(tok_emb),
            word_size, tok_size, pos_size, static_cast<__half*>(output), nullptr, out_i8, q_scale, mask_idx);
    if (type_id == BERT_B200_FP32)
        return dispatchEmb<float, false>(s, ld, B, B * S, input_ids, token_ids, mask, beta, gamma,
            static_cast<float const*>(word_emb), static_cast<float const*>(pos_emb), static_cast<float const*>(tok_emb),
            word_size, tok_size, pos_size, static_cast<float*>(output), nullptr, out_i8, q_scale, mask_idx);
    B200_FAIL(BERT_B200_NOT_SUPPORTED, "emb_layer_norm: type_id %d", type_id);
}

extern "C" int32_t bert_b200_emb_layer_norm(void* stream, int32_t type_id, int32_t ld, int32_t B, int32_t S,
    int32_t const* input_ids, int32_t const* token_ids, float const* beta, float const* gamma, void const* word_emb,
    void const* pos_emb, void const* tok_emb, int32_t word_size, int32_t tok_size, int32_t pos_size, void* output,
    int8_t* out_i8, float q_scale)
{
    return bert_b200_emb_layer_norm_mask_idx(stream, type_id, ld, B, S, input_ids, token_ids, beta, gamma, word_emb, pos_emb,
        tok_emb, word_size, tok_size, pos_size, output, out_i8, q_scale, nullptr, nullptr);
}

extern "C" int32_t bert_b200_emb_layer_norm_var_seqlen(void* stream, int32_t type_id, int32_t ld, int32_t B, int32_t S,
    int32_t total, int32_t const* input_ids, int32_t const* token_ids, int32_t const* cu_seqlens, float const* beta,
    float const* gamma, void const* word_emb, void const* pos_emb, void const* tok_emb, int32_t word_size,
    int32_t tok_size, int32_t pos_size, void* output, void* skip_out, int8_t* out_i8, float q_scale)
{
    (void) S;
    B200_REQUIRE(ld > 0 && B >= 0 && total >= 0, "emb_layer_norm_var_seqlen: bad sizes ld=%d B=%d total=%d", ld, B, total);
    B200_REQUIRE(input_ids && token_ids && cu_seqlens && beta && gamma && word_emb && pos_emb && tok_emb && output,
        "emb_layer_norm_var_seqlen: null pointer");
    B200_REQUIRE(word_size > 0 && tok_size > 0 && pos_size > 0, "emb_layer_norm_var_seqlen: empty table");
    if (total == 0 || B == 0)
        return BERT_B200_OK;
    auto s = static_cast<cudaStream_t>(stream);
    if (type_id == BERT_B200_FP16)
        return dispatchEmb<__half, true>(s, ld, B, total, input_ids, token_ids, cu_seqlens, beta, gamma,
            static_cast<__half const*>(word_emb), static_cast<__half const*>(pos_emb), static_cast<__half const*>(tok_emb),
            word_size, tok_size, pos_size, static_cast<__half*>(output), static_cast<__half*>(skip_out), out_i8, q_scale);
    if (type_id == BERT_B200_FP32)
        return dispatchEmb<float, true>(s, ld, B, total, input_ids, token_ids, cu_seqlens, beta, gamma,
            static_cast<float const*>(word_emb), static_cast<float const*>(pos_emb), static_cast<float const*>(tok_emb),
            word_size, tok_size, pos_size, static_cast<float*>(output), static_cast<float*>(skip_out), out_i8, q_scale);
    B200_FAIL(BERT_B200_NOT_SUPPORTED, "emb_layer_norm_var_seqlen: type_id %d", type_id);
}

extern "C" int32_t bert_b200_compute_mask_idx(void* stream, int32_t S, int32_t B, int32_t const* mask, int32_t* mask_idx)
{
    B200_REQUIRE(S >= 0 && B >= 0, "compute_mask_idx: bad sizes S=%d B=%d", S, B);
    B200_REQUIRE(mask_idx && (mask || S == 0), "compute_mask_idx: null pointer");
    if (B == 0)
        return BERT_B200_OK;
    maskIdxKernel<<<(B + kWarpsPerCta - 1) / kWarpsPerCta, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        S, B, mask, mask_idx);
    return checkLaunch("maskIdxKernel");
}

extern "C" int32_t bert_b200_convert_mask(uint32_t S, uint32_t B, uint32_t warps_m, uint32_t warps_n, uint32_t warps_k,
    int32_t const* input_mask_sb, uint32_t* input_mask_x, void* stream)
{
    B200_REQUIRE(S > 0 && warps_m > 0 && warps_n > 0 && warps_k > 0, "convert_mask: bad sizes");
    B200_REQUIRE(warps_m * warps_n * warps_k * 32 <= 1024, "convert_mask: more than 1024 threads per CTA");
    B200_REQUIRE((S + 16 * warps_n - 1) / (16 * warps_n) <= 4, "convert_mask: S=%u needs more than 32 mask bits per thread", S);
    B200_REQUIRE(input_mask_sb && input_mask_x, "convert_mask: null pointer");
    if (B == 0)
        return BERT_B200_OK;
    uint32_t const xmmasM = (S + 16 * warps_m - 1) / (16 * warps_m);
    uint32_t const xmmasN = (S + 16 * warps_n - 1) / (16 * warps_n);
    uint32_t const threads = warps_m * warps_n * warps_k * 32;
    size_t const smem = (static_cast<size_t>(xmmasN) * 16 * warps_n + 16) * sizeof(int32_t);
    packMaskKernel<<<dim3(xmmasM, B), threads, smem, static_cast<cudaStream_t>(stream)>>>(
        warps_m, warps_n, S, input_mask_sb, input_mask_x);
    return checkLaunch("packMaskKernel");
}

extern "C" int32_t bert_b200_packed_mask_to_lengths(void* stream, int32_t S, int32_t B, uint32_t warps_m, uint32_t warps_n,
    uint32_t row_words, uint32_t const* packed_mask, int32_t* lengths)
{
    B200_REQUIRE(S > 0 && B >= 0 && warps_m > 0 && warps_n > 0, "packed_mask_to_lengths: bad sizes");
    B200_REQUIRE((S + 16 * warps_n - 1) / (16 * warps_n) <= 4, "packed_mask_to_lengths: S=%d needs more than 32 mask bits", S);
    B200_REQUIRE(row_words >= warps_m * warps_n * 32, "packed_mask_to_lengths: row_words smaller than one CTA row");
    B200_REQUIRE(packed_mask && lengths, "packed_mask_to_lengths: null pointer");
    if (B == 0)
        return BERT_B200_OK;
    packedMaskToLengthsKernel<<<(B + kWarpsPerCta - 1) / kWarpsPerCta, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        warps_m, warps_n, row_words, S, B, packed_mask, lengths);
    return checkLaunch("packedMaskToLengthsKernel");
}

extern "C" int32_t bert_b200_lengths_to_cu_seqlens(void* stream, int32_t B, int32_t const* lengths, int32_t* cu_seqlens)
{
    B200_REQUIRE(B >= 0 && B <= 65536, "lengths_to_cu_seqlens: B=%d out of range", B);
    B200_REQUIRE(cu_seqlens && (lengths || B == 0), "lengths_to_cu_seqlens: null pointer");
    cuSeqlensKernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(B, lengths, cu_seqlens);
    return checkLaunch("cuSeqlensKernel");
}

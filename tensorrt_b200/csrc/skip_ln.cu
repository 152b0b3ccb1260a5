// Residual + bias + LayerNorm for sm_100a: FP32/FP16 rows, INT8 linear rows and INT8 CHW32-interleaved
// tokens. All kernels are single pass (every input byte is read once, every output byte written
// once), use 128-bit global accesses, keep the row in registers and accumulate statistics in FP32.
//
// Replaces the reference kernels skipln_vec / skipLayerNormKernel[Small] / skiplnDQQ
// (plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:43-217) and skiplnDQQ_vec3/4,
// skipln_vec32_hface/mtron (plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedKernel{HFace,MTron}.cu).
#include "common.cuh"

#include <limits>

namespace b200
{
namespace
{

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;

// Sums `v` over the WPR warps that share one row. `slots` is this row's scratch in shared memory, two lines used
// alternately (`turn` flips per call): a warp can only reach its next-but-one reduction after every warp of the row
// has passed the barrier in between, so one barrier per reduction is enough. The barrier is a named one over just
// the row's WPR warps (id 1 + row in CTA), not the whole CTA.
template <int WPR>
__device__ __forceinline__ float rowSum(float v, float (*slots)[WPR > 1 ? WPR : 1], int rowInCta, int wInRow, int lane, int& turn)
{
    v = warpSum(v);
    if (WPR == 1)
        return v;
    float* const slot = slots[turn];
    turn ^= 1;
    if (lane == 0)
        slot[wInRow] = v;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + rowInCta), "n"(WPR * 32) : "memory");
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; ++w)
        t += slot[w];
    return t;
}

// Two sums at once (sum and sum of squares): one barrier for both.
template <int WPR>
__device__ __forceinline__ float2 rowSum2(float a, float b, float2 (*slots)[WPR > 1 ? WPR : 1], int rowInCta, int wInRow, int lane,
    int& turn)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    if (WPR == 1)
        return make_float2(a, b);
    float2* const slot = slots[turn];
    turn ^= 1;
    if (lane == 0)
        slot[wInRow] = make_float2(a, b);
    asm volatile("bar.sync %0, %1;" ::"r"(1 + rowInCta), "n"(WPR * 32) : "memory");
    float2 t = make_float2(0.f, 0.f);
#pragma unroll
    for (int w = 0; w < WPR; ++w)
    {
        t.x += slot[w].x;
        t.y += slot[w].y;
    }
    return t;
}

template <typename T>
struct Vec;
template <>
struct Vec<__half>
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
struct Vec<float>
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

// One row is shared by WPR warps; each lane owns CPL 16-byte chunks: chunk (i*WPR + wInRow)*32 + lane.
// The grid strides over rows, so gamma/beta/bias chunks (always the same columns for a lane) stay
// in L1 after the first row.
template <typename T, int CPL, int WPR, bool HAS_BIAS>
__global__ void __launch_bounds__(kThreads, (WPR == 2 && CPL == 2) ? 4 : 1) skipLnKernel(int32_t const ld, int64_t const rows, T const* __restrict__ in,
    T const* __restrict__ skip, T const* __restrict__ beta, T const* __restrict__ gamma, T const* __restrict__ bias,
    T* __restrict__ out, float const eps)
{
    constexpr int E = Vec<T>::kElems;
    constexpr int kRowsPerCta = kWarpsPerCta / WPR;
    __shared__ float red[kRowsPerCta][2][WPR > 1 ? WPR : 1];
    int turn = 0;

    int const lane = threadIdx.x & 31;
    int const warp = threadIdx.x >> 5;
    int const rowInCta = warp / WPR;
    int const wInRow = warp % WPR;
    int const chunksPerRow = ld / E;
    float const rld = 1.f / static_cast<float>(ld);
    gridDependencyLaunch();
    gridDependencyWait(); // the rows come from the previous kernel of the stream

    int64_t const rowsRounded = (rows + kRowsPerCta - 1) / kRowsPerCta * kRowsPerCta;
    int64_t const rowStride = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
    uint4 a[CPL], b[CPL];
    // the two input rows of `r` into a / b (zeros beyond the last row or the row's end)
    auto loadRow = [&](int64_t r) {
        bool const rOk = r < rows;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            bool const ok = rOk && c < chunksPerRow;
            a[i] = ok ? ldgStream(in + r * ld + c * E) : make_uint4(0, 0, 0, 0);
            b[i] = ok ? ldgStream(skip + r * ld + c * E) : make_uint4(0, 0, 0, 0);
        }
    };
    // Rows shared by four or more warps (4096 values and up) load their next row while the statistics and the store of
    // the current one run: measured +34 % at 4096 halves. Narrower rows lose 2 % to the registers it costs (four CTAs per
    // SM become three) and load at the top of the loop - except two warps x two chunks (1024 halves), which fits the 64
    // registers of four CTAs per SM without spilling and gains 3-5 %.
    constexpr bool kPipelined = WPR >= 4 || (WPR == 2 && CPL == 2);
    if (kPipelined)
        loadRow(static_cast<int64_t>(blockIdx.x) * kRowsPerCta + rowInCta);
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + rowInCta; row < rowsRounded; row += rowStride)
    {
        bool const rowOk = row < rows;
        if (!kPipelined)
            loadRow(row);
        float x[CPL][E];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            float fb[E];
            Vec<T>::unpack(a[i], x[i]);
            Vec<T>::unpack(b[i], fb);
#pragma unroll
            for (int j = 0; j < E; ++j)
                x[i][j] += fb[j];
            if (HAS_BIAS && c < chunksPerRow)
            {
                uint4 const bv = ldgKeep(bias + c * E);
                Vec<T>::unpack(bv, fb);
#pragma unroll
                for (int j = 0; j < E; ++j)
                    x[i][j] += fb[j];
            }
#pragma unroll
            for (int j = 0; j < E; ++j)
                s += x[i][j];
        }
        // a / b are unpacked: the next row's loads go out now and land during the statistics and the store of this row
        if (kPipelined && row + rowStride < rowsRounded)
            loadRow(row + rowStride);
        float const mu = rowSum<WPR>(s, red[rowInCta], rowInCta, wInRow, lane, turn) * rld;
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
        float const var = rowSum<WPR>(q, red[rowInCta], rowInCta, wInRow, lane, turn) * rld;
        float const rsigma = rsqrtf(var + eps);

#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            if (rowOk && c < chunksPerRow)
            {
                float g[E], bt[E];
                Vec<T>::unpack(ldgKeep(gamma + c * E), g);
                Vec<T>::unpack(ldgKeep(beta + c * E), bt);
#pragma unroll
                for (int j = 0; j < E; ++j)
                    x[i][j] = g[j] * (x[i][j] - mu) * rsigma + bt[j];
                stgStream(out + row * ld + c * E, Vec<T>::pack(x[i]));
            }
        }
    }
}

// Any ld, scalar accesses, one warp per row; the row is revisited from L1/L2 instead of registers.
template <typename T, bool HAS_BIAS>
__global__ void __launch_bounds__(kThreads) skipLnScalarKernel(int32_t const ld, int64_t const rows,
    T const* __restrict__ in, T const* __restrict__ skip, T const* __restrict__ beta, T const* __restrict__ gamma,
    T const* __restrict__ bias, T* __restrict__ out, float const eps)
{
    int const lane = threadIdx.x & 31;
    int const warp = threadIdx.x >> 5;
    float const rld = 1.f / static_cast<float>(ld);
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + warp; row < rows;
         row += static_cast<int64_t>(gridDim.x) * kWarpsPerCta)
    {
        T const* a = in + row * ld;
        T const* b = skip + row * ld;
        float s = 0.f;
        for (int i = lane; i < ld; i += 32)
            s += static_cast<float>(a[i]) + static_cast<float>(b[i]) + (HAS_BIAS ? static_cast<float>(bias[i]) : 0.f);
        float const mu = warpSum(s) * rld;
        float q = 0.f;
        for (int i = lane; i < ld; i += 32)
        {
            float const d
                = static_cast<float>(a[i]) + static_cast<float>(b[i]) + (HAS_BIAS ? static_cast<float>(bias[i]) : 0.f) - mu;
            q += d * d;
        }
        float const rsigma = rsqrtf(warpSum(q) * rld + eps);
        for (int i = lane; i < ld; i += 32)
        {
            float const v
                = static_cast<float>(a[i]) + static_cast<float>(b[i]) + (HAS_BIAS ? static_cast<float>(bias[i]) : 0.f);
            out[row * ld + i] = static_cast<T>(static_cast<float>(gamma[i]) * (v - mu) * rsigma + static_cast<float>(beta[i]));
        }
    }
}

// INT8 linear rows: 16 values per 128-bit load, FP16 parameters (two 128-bit loads per chunk).
template <int CPL, int WPR, bool HAS_BIAS>
__global__ void __launch_bounds__(kThreads) skipLnDqqKernel(int32_t const ld, int64_t const rows,
    int8_t const* __restrict__ in, int8_t const* __restrict__ skip, __half const* __restrict__ beta,
    __half const* __restrict__ gamma, __half const* __restrict__ bias, int8_t* __restrict__ out, float const dqIn,
    float const dqSkip, float const qScale, float const eps)
{
    constexpr int E = 16;
    constexpr int kRowsPerCta = kWarpsPerCta / WPR;
    __shared__ float2 red[kRowsPerCta][2][WPR > 1 ? WPR : 1];
    int turn = 0;

    int const lane = threadIdx.x & 31;
    int const warp = threadIdx.x >> 5;
    int const rowInCta = warp / WPR;
    int const wInRow = warp % WPR;
    int const chunksPerRow = ld / E;
    float const rld = 1.f / static_cast<float>(ld);
    gridDependencyLaunch();
    gridDependencyWait(); // the rows come from the previous kernel of the stream

    int64_t const rowsRounded = (rows + kRowsPerCta - 1) / kRowsPerCta * kRowsPerCta;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + rowInCta; row < rowsRounded;
         row += static_cast<int64_t>(gridDim.x) * kRowsPerCta)
    {
        bool const rowOk = row < rows;
        uint4 a[CPL], b[CPL];
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            bool const ok = rowOk && c < chunksPerRow;
            a[i] = ok ? ldgStream(in + row * ld + c * E) : make_uint4(0, 0, 0, 0);
            b[i] = ok ? ldgStream(skip + row * ld + c * E) : make_uint4(0, 0, 0, 0);
        }
        // Statistics in one sweep: FP32 sum and sum of squares (the reference's kernel forms the same two sums, in
        // FP16: plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:58-74), one block reduction for both.
        float x[CPL][E];
        float s = 0.f, q = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            uint32_t const* aw = reinterpret_cast<uint32_t const*>(&a[i]);
            uint32_t const* bw = reinterpret_cast<uint32_t const*>(&b[i]);
            // the bias rides in the second FMA of the dequantising sum
            float fbias[E];
            if (HAS_BIAS && c < chunksPerRow)
            {
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    float f8[8];
                    unpackHalf8(ldgKeep(bias + c * E + 8 * h), f8);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        fbias[8 * h + j] = f8[j];
                }
            }
            else
            {
#pragma unroll
                for (int j = 0; j < E; ++j)
                    fbias[j] = 0.f;
            }
#pragma unroll
            for (int w = 0; w < 4; ++w)
            {
                float fa[4], fb[4];
                unpackChar4(aw[w], fa);
                unpackChar4(bw[w], fb);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    x[i][4 * w + j] = fmaf(dqIn, fa[j], fmaf(dqSkip, fb[j], fbias[4 * w + j]));
            }
            // chunks beyond the row hold zeros (zero inputs, zero bias) and add nothing to either sum
#pragma unroll
            for (int j = 0; j < E; ++j)
            {
                s += x[i][j];
                q = fmaf(x[i][j], x[i][j], q);
            }
        }
        float2 const sums = rowSum2<WPR>(s, q, red[rowInCta], rowInCta, wInRow, lane, turn);
        float const mu = sums.x * rld;
        float const rsigma = rsqrtf(fmaxf(fmaf(sums.y, rld, -mu * mu), 0.f) + eps);
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            if (rowOk && c < chunksPerRow)
            {
                uint4 o;
                uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    float g[8], bt[8], y[8];
                    unpackHalf8(ldgKeep(gamma + c * E + 8 * h), g);
                    unpackHalf8(ldgKeep(beta + c * E + 8 * h), bt);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        y[j] = fmaf(g[j] * rsigma, x[i][8 * h + j] - mu, bt[j]);
                    // multiply + saturating convert: the conversion unit has nothing else to do in this kernel and
                    // the kernel is bound by issue slots (one slot less per value than clamp + rounding FMA)
                    ow[2 * h] = packChar4Cvt(y[0], y[1], y[2], y[3], qScale);
                    ow[2 * h + 1] = packChar4Cvt(y[4], y[5], y[6], y[7], qScale);
                }
                stgStream(out + row * ld + c * E, o);
            }
        }
    }
}

// INT8 linear rows, packed arithmetic. The kernel above spends 21 instructions per element and is bound by issue slots at
// 42 % of the memory bandwidth; this one needs about 10:
//   * statistics on the raw bytes with dp4a: sum a, sum b, sum a^2, sum b^2, sum a*b are exact integers (five
//     instructions per four elements) and give sum x and sum x^2 of x = dq_in a + dq_skip b in FP32; a bias adds
//     2 sum t*bias, accumulated alongside in half2 (a term three orders of magnitude below sum x^2), and two constants;
//   * the element-wise part in half2, two elements per instruction, like the reference's kernel
//     (plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:58-103): bytes -> FP16 through the exponent of 1024 (PRMT),
//     dequantise, (+ bias,) one fused multiply-add for gamma (x - mean) rsigma + beta, already scaled to the INT8 grid
//     and shifted to [0, 1] so that the instruction's own saturation is the clamp, one more to round (adding 1408 leaves
//     the integer in the low byte);
//   * gamma, beta (pre-scaled) and bias sit as half2 tables in shared memory, built once per CTA (no per-row parameter
//     conversions); the lanes of a row add their integer sums with redux.sync.
// Every value is within 1 LSB of the exact result (the FP16 steps add up to a few tenths of an LSB at most).
// CB = bytes per chunk: 16, or 8 for rows that fill 16-byte chunks unevenly (768 = 48 chunks of 16 for 32 lanes, but
// exactly three chunks of 8 per lane).
template <int CPL, int WPR, bool HAS_BIAS, int CB = 16>
__global__ void __launch_bounds__(kThreads, 3) skipLnDqqPackedKernel(int32_t const ld, int64_t const rows,
    int8_t const* __restrict__ in, int8_t const* __restrict__ skip, __half const* __restrict__ beta,
    __half const* __restrict__ gamma, __half const* __restrict__ bias, int8_t* __restrict__ out, float const dqIn,
    float const dqSkip, float const qScale, float const eps)
{
    constexpr int E = CB;
    constexpr int kWords = CB / 4;     // 32-bit words (four INT8 values each) per chunk
    constexpr int kPairs = CB / 2;     // half2 values per chunk
    constexpr int kRowsPerCta = kWarpsPerCta / WPR;
    __shared__ float2 red[kRowsPerCta][2][WPR > 1 ? WPR : 1];
    int turn = 0;

    int const lane = threadIdx.x & 31;
    int const warp = threadIdx.x >> 5;
    int const rowInCta = warp / WPR;
    int const wInRow = warp % WPR;
    int const chunksPerRow = ld / E;
    float const rld = 1.f / static_cast<float>(ld);

    // sums the per-warp values of the WPR warps that share a row (the values are warp totals already)
    auto rowCombine = [&](float a, float b) -> float2 {
        if (WPR == 1)
            return make_float2(a, b);
        float2* const slot = red[rowInCta][turn];
        turn ^= 1;
        if (lane == 0)
            slot[wInRow] = make_float2(a, b);
        asm volatile("bar.sync %0, %1;" ::"r"(1 + rowInCta), "n"(WPR * 32) : "memory");
        float2 t = make_float2(0.f, 0.f);
#pragma unroll
        for (int w = 0; w < WPR; ++w)
        {
            t.x += slot[w].x;
            t.y += slot[w].y;
        }
        return t;
    };

    // ---- gamma, (beta * q_scale + 128) / 255 and bias as half2 tables in shared memory, built once per CTA: a lane
    //      reads the eight half2 of a chunk with two 128-bit loads per table and row (no conversions in the row loop,
    //      and no registers held across it: three CTAs fit an SM). Each table is two planes - half2 0..3 of every
    //      chunk, then half2 4..7 - so that consecutive lanes read consecutive 16 bytes (no bank conflicts) ----
    int const plane = ld / 4; // half2 per plane (16-byte chunks; an 8-byte chunk is one 128-bit table read already)
    extern __shared__ uint4 paramSmem[];
    __half2* const gTab = reinterpret_cast<__half2*>(paramSmem);
    __half2* const bqTab = gTab + ld / 2;
    __half2* const biTab = bqTab + ld / 2;
    float sBias = 0.f, sBias2 = 0.f;
    for (int p = threadIdx.x; p < ld / 2; p += kThreads)
    {
        float2 const g = __half22float2(reinterpret_cast<__half2 const*>(gamma)[p]);
        float2 const bt = __half22float2(reinterpret_cast<__half2 const*>(beta)[p]);
        int const d = CB == 16 ? ((p >> 2) & 1) * plane + (p >> 3) * 4 + (p & 3) : p;
        gTab[d] = __floats2half2_rn(g.x, g.y);
        bqTab[d] = __floats2half2_rn(fmaf(bt.x, qScale, 128.f) * (1.f / 255.f), fmaf(bt.y, qScale, 128.f) * (1.f / 255.f));
        if (HAS_BIAS)
            biTab[d] = reinterpret_cast<__half2 const*>(bias)[p];
    }
    __syncthreads();
    if (HAS_BIAS)
    {
        // sum and sum of squares of the bias over the whole row, by every warp (the statistics use the bias as the
        // element-wise part sees it: FP16)
        for (int p = lane; p < ld / 2; p += 32)
        {
            float2 const bs = __half22float2(biTab[p]);
            sBias += bs.x + bs.y;
            sBias2 = fmaf(bs.x, bs.x, fmaf(bs.y, bs.y, sBias2));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
        {
            sBias += __shfl_xor_sync(0xffffffffu, sBias, o);
            sBias2 += __shfl_xor_sync(0xffffffffu, sBias2, o);
        }
    }
    __half2 const dqIn2 = __float2half2_rn(dqIn), dqSkip2 = __float2half2_rn(dqSkip);
    // the integer sums are weighted with the scales the element-wise part actually multiplies by
    float const dqInH = __low2float(dqIn2), dqSkipH = __low2float(dqSkip2);
    __half2 const kMagic = __float2half2_rn(1152.f); // 1024 + 128: exponent byte 0x64 over (byte ^ 0x80)
    gridDependencyLaunch();
    gridDependencyWait(); // the rows come from the previous kernel of the stream

    int64_t const rowsRounded = (rows + kRowsPerCta - 1) / kRowsPerCta * kRowsPerCta;
    int64_t const rowStride = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
    uint32_t a[CPL][kWords], b[CPL][kWords];
    // the two input rows of `r` into a / b (zeros beyond the last row or the row's end)
    auto loadRow = [&](int64_t r) {
        bool const rOk = r < rows;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            bool const ok = rOk && c < chunksPerRow;
            if (CB == 16)
            {
                uint4 const va = ok ? ldgStream(in + r * ld + c * E) : make_uint4(0, 0, 0, 0);
                uint4 const vb = ok ? ldgStream(skip + r * ld + c * E) : make_uint4(0, 0, 0, 0);
                a[i][0] = va.x, a[i][1] = va.y, a[i][kWords - 2] = va.z, a[i][kWords - 1] = va.w;
                b[i][0] = vb.x, b[i][1] = vb.y, b[i][kWords - 2] = vb.z, b[i][kWords - 1] = vb.w;
            }
            else
            {
                uint2 const va = ok ? ldgStream8(in + r * ld + c * E) : make_uint2(0, 0);
                uint2 const vb = ok ? ldgStream8(skip + r * ld + c * E) : make_uint2(0, 0);
                a[i][0] = va.x, a[i][1] = va.y;
                b[i][0] = vb.x, b[i][1] = vb.y;
            }
        }
    };
    loadRow(static_cast<int64_t>(blockIdx.x) * kRowsPerCta + rowInCta);
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + rowInCta; row < rowsRounded; row += rowStride)
    {
        bool const rowOk = row < rows;
        int32_t sa = 0, sb = 0, saa = 0, sbb = 0, sab = 0;
        __half2 cross0 = __float2half2_rn(0.f), cross1 = cross0;
        __half2 x2[CPL][kPairs];
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            uint32_t const* aw = a[i];
            uint32_t const* bw = b[i];
            __half2 bi2[kPairs];
            if (HAS_BIAS)
            {
                int const c = min((i * WPR + wInRow) * 32 + lane, chunksPerRow - 1); // chunks beyond the row carry zeros
                *reinterpret_cast<uint4*>(&bi2[0]) = *reinterpret_cast<uint4 const*>(biTab + c * 4);
                if (CB == 16)
                    *reinterpret_cast<uint4*>(&bi2[kPairs - 4]) = *reinterpret_cast<uint4 const*>(biTab + plane + c * 4);
            }
#pragma unroll
            for (int w = 0; w < kWords; ++w)
            {
                int32_t const ia = static_cast<int32_t>(aw[w]), ib = static_cast<int32_t>(bw[w]);
                sa = __dp4a(ia, 0x01010101, sa);
                sb = __dp4a(ib, 0x01010101, sb);
                saa = __dp4a(ia, ia, saa);
                sbb = __dp4a(ib, ib, sbb);
                sab = __dp4a(ia, ib, sab);
                uint32_t const ua = aw[w] ^ 0x80808080u, ub = bw[w] ^ 0x80808080u;
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    uint32_t const am = __byte_perm(ua, 0x64646464u, h == 0 ? 0x5140 : 0x7362);
                    uint32_t const bm = __byte_perm(ub, 0x64646464u, h == 0 ? 0x5140 : 0x7362);
                    __half2 const fa = __hsub2(*reinterpret_cast<__half2 const*>(&am), kMagic);
                    __half2 const fb = __hsub2(*reinterpret_cast<__half2 const*>(&bm), kMagic);
                    __half2 t = __hfma2(dqIn2, fa, __hmul2(dqSkip2, fb));
                    if (HAS_BIAS)
                    {
                        __half2 const bs = bi2[2 * w + h];
                        if (h == 0)
                            cross0 = __hfma2(t, bs, cross0);
                        else
                            cross1 = __hfma2(t, bs, cross1);
                        t = __hadd2(t, bs);
                    }
                    x2[i][2 * w + h] = t;
                }
            }
        }
        // a / b are consumed: the next row's loads go out now and land during the reductions, the element-wise part
        // and the store of this row
        if (row + rowStride < rowsRounded)
            loadRow(row + rowStride);
        // row sums: exact integers over the warp, the small cross term in FP32
        sa = __reduce_add_sync(0xffffffffu, sa);
        sb = __reduce_add_sync(0xffffffffu, sb);
        saa = __reduce_add_sync(0xffffffffu, saa);
        sbb = __reduce_add_sync(0xffffffffu, sbb);
        sab = __reduce_add_sync(0xffffffffu, sab);
        float s1 = fmaf(dqInH, static_cast<float>(sa), dqSkipH * static_cast<float>(sb));
        float s2 = fmaf(dqInH * dqInH, static_cast<float>(saa),
            fmaf(dqSkipH * dqSkipH, static_cast<float>(sbb), 2.f * dqInH * dqSkipH * static_cast<float>(sab)));
        if (HAS_BIAS)
        {
            float2 const c0 = __half22float2(cross0), c1 = __half22float2(cross1);
            float cr = (c0.x + c0.y) + (c1.x + c1.y);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                cr += __shfl_xor_sync(0xffffffffu, cr, o);
            s2 = fmaf(2.f, cr, s2);
        }
        float2 const sums = rowCombine(s1, s2);
        float const mu = (sums.x + sBias) * rld;
        float const rsigma = rsqrtf(fmaxf(fmaf(sums.y + sBias2, rld, -mu * mu), 0.f) + eps);
        // (gamma (x - mu) rsigma + beta) q_scale, shifted and scaled to [0, 1] <-> [-128, 127]
        __half2 const k1 = __float2half2_rn(rsigma * qScale * (1.f / 255.f));
        __half2 const negMu = __float2half2_rn(-mu);
        __half2 const k255 = __float2half2_rn(255.f), k1408 = __float2half2_rn(1408.f);
#pragma unroll
        for (int i = 0; i < CPL; ++i)
        {
            int const c = (i * WPR + wInRow) * 32 + lane;
            if (rowOk && c < chunksPerRow)
            {
                uint32_t ow[kWords];
                __half2 g2[kPairs], bq2[kPairs];
                *reinterpret_cast<uint4*>(&g2[0]) = *reinterpret_cast<uint4 const*>(gTab + c * 4);
                *reinterpret_cast<uint4*>(&bq2[0]) = *reinterpret_cast<uint4 const*>(bqTab + c * 4);
                if (CB == 16)
                {
                    *reinterpret_cast<uint4*>(&g2[kPairs - 4]) = *reinterpret_cast<uint4 const*>(gTab + plane + c * 4);
                    *reinterpret_cast<uint4*>(&bq2[kPairs - 4]) = *reinterpret_cast<uint4 const*>(bqTab + plane + c * 4);
                }
#pragma unroll
                for (int w = 0; w < kWords; ++w)
                {
                    uint32_t r[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                    {
                        __half2 const c1 = __hmul2(g2[2 * w + h], k1);
                        __half2 const c0 = __hfma2(c1, negMu, bq2[2 * w + h]);
                        __half2 const v = __hfma2_sat(c1, x2[i][2 * w + h], c0);
                        __half2 const q = __hfma2(v, k255, k1408); // round to nearest even; the integer sits in the low byte
                        r[h] = *reinterpret_cast<uint32_t const*>(&q);
                    }
                    ow[w] = __byte_perm(r[0], r[1], 0x6420);
                }
                if (CB == 16)
                    stgStream(out + row * ld + c * E, make_uint4(ow[0], ow[1], ow[kWords - 2], ow[kWords - 1]));
                else
                    stgStream8(out + row * ld + c * E, make_uint2(ow[0], ow[1]));
            }
        }
    }
}

// INT8 CHW32-interleaved tokens: element (token t, channel c) lives at ((c/32)*total + t)*32 + c%32.
// A CTA owns 8 consecutive tokens, i.e. 256 contiguous bytes in each of the ld/32 channel groups.
// Thread -> 16-byte unit u = tid%16 (token u/2, half u%2) of channel group (tid/16 + 16*i), so a
// quarter warp reads 256 contiguous bytes. Per-token statistics are reduced over lane bits 0 and 4
// by shuffles and over the 8 warps through shared memory.
constexpr int kIlTokens = 8;

template <int NI, bool PRELN>
__global__ void __launch_bounds__(kThreads) skipLnInterleavedKernel(int32_t const ld, int32_t const total,
    int8_t const* __restrict__ in, int8_t const* __restrict__ skip, __half const* __restrict__ beta,
    __half const* __restrict__ gamma, int8_t* __restrict__ out, int8_t* __restrict__ preln, float const dqIn,
    float const dqSkip, float const qScale, float const qSkipScale, float const eps)
{
    __shared__ float red[2][kWarpsPerCta][kIlTokens];
    int const tid = threadIdx.x;
    int const lane = tid & 31;
    int const warp = tid >> 5;
    int const unit = tid & 15;
    int const tokInCta = unit >> 1;
    int const half = unit & 1;
    int const groups = ld / 32;
    float const rld = 1.f / static_cast<float>(ld);
    int const numTiles = (total + kIlTokens - 1) / kIlTokens;

    for (int tile = blockIdx.x; tile < numTiles; tile += gridDim.x)
    {
        int const tok = tile * kIlTokens + tokInCta;
        bool const tokOk = tok < total;
        uint4 a[NI], b[NI];
#pragma unroll
        for (int i = 0; i < NI; ++i)
        {
            int const g = (tid >> 4) + 16 * i;
            bool const ok = tokOk && g < groups;
            int64_t const off = (static_cast<int64_t>(g) * total + tok) * 32 + half * 16;
            a[i] = ok ? ldgStream(in + off) : make_uint4(0, 0, 0, 0);
            b[i] = ok ? ldgStream(skip + off) : make_uint4(0, 0, 0, 0);
        }
        float x[NI][16];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i)
        {
            uint32_t const* aw = reinterpret_cast<uint32_t const*>(&a[i]);
            uint32_t const* bw = reinterpret_cast<uint32_t const*>(&b[i]);
#pragma unroll
            for (int w = 0; w < 4; ++w)
            {
                float fa[4], fb[4];
                unpackChar4(aw[w], fa);
                unpackChar4(bw[w], fb);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    x[i][4 * w + j] = dqIn * fa[j] + dqSkip * fb[j];
                    s += x[i][4 * w + j];
                }
            }
        }
        // lanes with equal token: differ in lane bit 0 (half) and bit 4 (group parity)
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 16);
        if ((lane & 17) == 0)
            red[0][warp][tokInCta] = s;
        __syncthreads();
        float mu = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsPerCta; ++w)
            mu += red[0][w][tokInCta];
        mu *= rld;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i)
        {
            int const g = (tid >> 4) + 16 * i;
            if (g < groups)
            {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                {
                    float const d = x[i][j] - mu;
                    q += d * d;
                }
            }
        }
        q += __shfl_xor_sync(0xffffffffu, q, 1);
        q += __shfl_xor_sync(0xffffffffu, q, 16);
        if ((lane & 17) == 0)
            red[1][warp][tokInCta] = q;
        __syncthreads();
        float var = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsPerCta; ++w)
            var += red[1][w][tokInCta];
        float const rsigma = rsqrtf(var * rld + eps);

#pragma unroll
        for (int i = 0; i < NI; ++i)
        {
            int const g = (tid >> 4) + 16 * i;
            if (tokOk && g < groups)
            {
                int64_t const off = (static_cast<int64_t>(g) * total + tok) * 32 + half * 16;
                int const ch = g * 32 + half * 16;
                uint4 o, p;
                uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
                uint32_t* pw = reinterpret_cast<uint32_t*>(&p);
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    float gm[8], bt[8], y[8];
                    unpackHalf8(ldgKeep(gamma + ch + 8 * h), gm);
                    unpackHalf8(ldgKeep(beta + ch + 8 * h), bt);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        y[j] = (gm[j] * (x[i][8 * h + j] - mu) * rsigma + bt[j]) * qScale;
                    ow[2 * h] = packChar4(y[0], y[1], y[2], y[3]);
                    ow[2 * h + 1] = packChar4(y[4], y[5], y[6], y[7]);
                    if (PRELN)
                    {
                        pw[2 * h] = packChar4(x[i][8 * h] * qSkipScale, x[i][8 * h + 1] * qSkipScale,
                            x[i][8 * h + 2] * qSkipScale, x[i][8 * h + 3] * qSkipScale);
                        pw[2 * h + 1] = packChar4(x[i][8 * h + 4] * qSkipScale, x[i][8 * h + 5] * qSkipScale,
                            x[i][8 * h + 6] * qSkipScale, x[i][8 * h + 7] * qSkipScale);
                    }
                }
                stgStream(out + off, o);
                if (PRELN)
                    stgStream(preln + off, p);
            }
        }
        // red[] is rewritten in the next iteration only after both barriers of that iteration's
        // first phase, and all reads of this iteration precede the next write of the same array
        // by at least one barrier (red[0] read before barrier 2; red[1] read before next barrier 1).
    }
}

// The same operator with the arithmetic of skipLnDqqPackedKernel: exact integer statistics by dp4a (one reduction and
// one barrier per tile instead of two), the element-wise part in half2 with the clamp as the saturation of the FMA,
// gamma and beta as half2 tables in shared memory (two planes, conflict-free 128-bit reads), and the next tile's loads
// issued as soon as this tile's bytes are unpacked. Thread (group g = tid / 16 + 16 i, token tid % 16 / 2, half tid % 2)
// owns 16 channels of one token, as above; NI <= 4 (ld <= 2048).
template <int NI, bool PRELN>
__global__ void __launch_bounds__(kThreads, NI <= 2 ? 3 : 2) skipLnInterleavedPackedKernel(int32_t const ld,
    int32_t const total, int8_t const* __restrict__ in, int8_t const* __restrict__ skip, __half const* __restrict__ beta,
    __half const* __restrict__ gamma, int8_t* __restrict__ out, int8_t* __restrict__ preln, float const dqIn,
    float const dqSkip, float const qScale, float const qSkipScale, float const eps)
{
    __shared__ float2 red[2][kWarpsPerCta][kIlTokens];
    extern __shared__ uint4 paramSmem[];
    __half2* const gTab = reinterpret_cast<__half2*>(paramSmem);
    __half2* const bqTab = gTab + ld / 2;
    int const tid = threadIdx.x;
    int const lane = tid & 31;
    int const warp = tid >> 5;
    int const unit = tid & 15;
    int const tokInCta = unit >> 1;
    int const half = unit & 1;
    int const groups = ld / 32;
    float const rld = 1.f / static_cast<float>(ld);
    int const numTiles = (total + kIlTokens - 1) / kIlTokens;
    int const plane = ld / 4; // half2 per plane: half2 0..3 of every 16-channel chunk, then half2 4..7

    for (int p = tid; p < ld / 2; p += kThreads)
    {
        float2 const g = __half22float2(reinterpret_cast<__half2 const*>(gamma)[p]);
        float2 const bt = __half22float2(reinterpret_cast<__half2 const*>(beta)[p]);
        int const d = ((p >> 2) & 1) * plane + (p >> 3) * 4 + (p & 3);
        gTab[d] = __floats2half2_rn(g.x, g.y);
        bqTab[d] = __floats2half2_rn(fmaf(bt.x, qScale, 128.f) * (1.f / 255.f), fmaf(bt.y, qScale, 128.f) * (1.f / 255.f));
    }
    __syncthreads();
    __half2 const dqIn2 = __float2half2_rn(dqIn), dqSkip2 = __float2half2_rn(dqSkip);
    // the integer sums are weighted with the scales the element-wise part actually multiplies by
    float const dqInH = __low2float(dqIn2), dqSkipH = __low2float(dqSkip2);
    __half2 const kMagic = __float2half2_rn(1152.f); // 1024 + 128: exponent byte 0x64 over (byte ^ 0x80)
    __half2 const k255 = __float2half2_rn(255.f), k1408 = __float2half2_rn(1408.f);
    __half2 const kPre1 = __float2half2_rn(qSkipScale * (1.f / 255.f)), kPre0 = __float2half2_rn(128.f / 255.f);
    int turn = 0;

    uint4 a[NI], b[NI];
    auto loadTile = [&](int tile) {
        int const tok = tile * kIlTokens + tokInCta;
#pragma unroll
        for (int i = 0; i < NI; ++i)
        {
            int const g = (tid >> 4) + 16 * i;
            bool const ok = tok < total && g < groups;
            int64_t const off = (static_cast<int64_t>(g) * total + tok) * 32 + half * 16;
            a[i] = ok ? ldgStream(in + off) : make_uint4(0, 0, 0, 0);
            b[i] = ok ? ldgStream(skip + off) : make_uint4(0, 0, 0, 0);
        }
    };
    if (static_cast<int>(blockIdx.x) < numTiles)
        loadTile(blockIdx.x);
    for (int tile = blockIdx.x; tile < numTiles; tile += gridDim.x)
    {
        int const tok = tile * kIlTokens + tokInCta;
        bool const tokOk = tok < total;
        int32_t sa = 0, sb = 0, saa = 0, sbb = 0, sab = 0;
        __half2 x2[NI][8];
#pragma unroll
        for (int i = 0; i < NI; ++i)
        {
            uint32_t const* aw = reinterpret_cast<uint32_t const*>(&a[i]);
            uint32_t const* bw = reinterpret_cast<uint32_t const*>(&b[i]);
#pragma unroll
            for (int w = 0; w < 4; ++w)
            {
                int32_t const ia = static_cast<int32_t>(aw[w]), ib = static_cast<int32_t>(bw[w]);
                sa = __dp4a(ia, 0x01010101, sa);
                sb = __dp4a(ib, 0x01010101, sb);
                saa = __dp4a(ia, ia, saa);
                sbb = __dp4a(ib, ib, sbb);
                sab = __dp4a(ia, ib, sab);
                uint32_t const ua = aw[w] ^ 0x80808080u, ub = bw[w] ^ 0x80808080u;
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    uint32_t const am = __byte_perm(ua, 0x64646464u, h == 0 ? 0x5140 : 0x7362);
                    uint32_t const bm = __byte_perm(ub, 0x64646464u, h == 0 ? 0x5140 : 0x7362);
                    __half2 const fa = __hsub2(*reinterpret_cast<__half2 const*>(&am), kMagic);
                    __half2 const fb = __hsub2(*reinterpret_cast<__half2 const*>(&bm), kMagic);
                    x2[i][2 * w + h] = __hfma2(dqIn2, fa, __hmul2(dqSkip2, fb));
                }
            }
        }
        if (tile + static_cast<int>(gridDim.x) < numTiles)
            loadTile(tile + gridDim.x);
        // sums of this thread's 16 * NI channels; lanes with equal token differ in lane bit 0 (half) and bit 4 (group parity)
        float s1 = fmaf(dqInH, static_cast<float>(sa), dqSkipH * static_cast<float>(sb));
        float s2 = fmaf(dqInH * dqInH, static_cast<float>(saa),
            fmaf(dqSkipH * dqSkipH, static_cast<float>(sbb), 2.f * dqInH * dqSkipH * static_cast<float>(sab)));
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
        s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 16);
        s2 += __shfl_xor_sync(0xffffffffu, s2, 16);
        if ((lane & 17) == 0)
            red[turn][warp][tokInCta] = make_float2(s1, s2);
        __syncthreads();
        float t1 = 0.f, t2 = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsPerCta; ++w)
        {
            float2 const r = red[turn][w][tokInCta];
            t1 += r.x;
            t2 += r.y;
        }
        // the other buffer next time: its readers of two tiles ago have all passed the barrier of the last tile
        turn ^= 1;
        float const mu = t1 * rld;
        float const rsigma = rsqrtf(fmaxf(fmaf(t2, rld, -mu * mu), 0.f) + eps);
        // (gamma (x - mu) rsigma + beta) q_scale, shifted and scaled to [0, 1] <-> [-128, 127]
        __half2 const k1 = __float2half2_rn(rsigma * qScale * (1.f / 255.f));
        __half2 const negMu = __float2half2_rn(-mu);
#pragma unroll
        for (int i = 0; i < NI; ++i)
        {
            int const g = (tid >> 4) + 16 * i;
            if (tokOk && g < groups)
            {
                int64_t const off = (static_cast<int64_t>(g) * total + tok) * 32 + half * 16;
                int const c = g * 2 + half; // 16-channel chunk of the row
                uint4 o, pre;
                uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
                uint32_t* pw = reinterpret_cast<uint32_t*>(&pre);
                __half2 g2[8], bq2[8];
                *reinterpret_cast<uint4*>(&g2[0]) = *reinterpret_cast<uint4 const*>(gTab + c * 4);
                *reinterpret_cast<uint4*>(&g2[4]) = *reinterpret_cast<uint4 const*>(gTab + plane + c * 4);
                *reinterpret_cast<uint4*>(&bq2[0]) = *reinterpret_cast<uint4 const*>(bqTab + c * 4);
                *reinterpret_cast<uint4*>(&bq2[4]) = *reinterpret_cast<uint4 const*>(bqTab + plane + c * 4);
#pragma unroll
                for (int w = 0; w < 4; ++w)
                {
                    uint32_t r[2], rp[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                    {
                        __half2 const c1 = __hmul2(g2[2 * w + h], k1);
                        __half2 const c0 = __hfma2(c1, negMu, bq2[2 * w + h]);
                        __half2 const v = __hfma2_sat(c1, x2[i][2 * w + h], c0);
                        __half2 const q = __hfma2(v, k255, k1408); // round to nearest even; the integer sits in the low byte
                        r[h] = *reinterpret_cast<uint32_t const*>(&q);
                        if (PRELN)
                        {
                            __half2 const vp = __hfma2_sat(kPre1, x2[i][2 * w + h], kPre0);
                            __half2 const qp = __hfma2(vp, k255, k1408);
                            rp[h] = *reinterpret_cast<uint32_t const*>(&qp);
                        }
                    }
                    ow[w] = __byte_perm(r[0], r[1], 0x6420);
                    if (PRELN)
                        pw[w] = __byte_perm(rp[0], rp[1], 0x6420);
                }
                stgStream(out + off, o);
                if (PRELN)
                    stgStream(preln + off, pre);
            }
        }
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

template <typename T, int CPL, int WPR>
int32_t launchSkipLn(cudaStream_t stream, int32_t ld, int64_t rows, T const* in, T const* skip, T const* beta,
    T const* gamma, T const* bias, T* out, float eps)
{
    int const rowsPerCta = kWarpsPerCta / WPR;
    int const grid = gridFor((rows + rowsPerCta - 1) / rowsPerCta, 8);
    if (bias)
        launchDependent(skipLnKernel<T, CPL, WPR, true>, dim3(grid), dim3(kThreads), 0, stream, ld, rows, in, skip, beta, gamma, bias,
            out, eps);
    else
        launchDependent(skipLnKernel<T, CPL, WPR, false>, dim3(grid), dim3(kThreads), 0, stream, ld, rows, in, skip, beta, gamma, bias,
            out, eps);
    return checkLaunch("skipLnKernel");
}

template <typename T>
int32_t dispatchSkipLn(cudaStream_t stream, int32_t ld, int64_t rows, T const* in, T const* skip, T const* beta,
    T const* gamma, T const* bias, T* out)
{
    // FP16: the reference adds numeric_limits<half>::epsilon(), which is value-initialised (0) because no
    // specialisation for __half exists; FP32 adds 1.19e-7 (plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:149).
    float const eps = sizeof(T) == 4 ? std::numeric_limits<float>::epsilon() : 0.f;
    constexpr int E = 16 / sizeof(T);
    bool const vec = (ld % E == 0) && ld / E <= 32 * 4 * 8 && aligned16(in) && aligned16(skip) && aligned16(out)
        && aligned16(beta) && aligned16(gamma) && (!bias || aligned16(bias));
    if (!vec)
    {
        int const grid = gridFor((rows + kWarpsPerCta - 1) / kWarpsPerCta, 8);
        if (bias)
            skipLnScalarKernel<T, true><<<grid, kThreads, 0, stream>>>(ld, rows, in, skip, beta, gamma, bias, out, eps);
        else
            skipLnScalarKernel<T, false><<<grid, kThreads, 0, stream>>>(ld, rows, in, skip, beta, gamma, bias, out, eps);
        return checkLaunch("skipLnScalarKernel");
    }
    int const chunks = ld / E;
    // Smallest number of warps per row that leaves at most 4 chunks per lane.
    int wpr = 1;
    while (chunks > 32 * 4 * wpr)
        wpr *= 2;
    // Four chunks per lane and a single warp per row (128 chunks: 1024 halves) keeps too few rows in flight; two
    // warps with two chunks each measured 20-28 % faster.
    if (wpr == 1 && chunks > 32 * 3)
        wpr = 2;
    int const cpl = (chunks + 32 * wpr - 1) / (32 * wpr);
#define B200_SKIPLN_CASE(C, W)                                                                                         \
    if (cpl == C && wpr == W)                                                                                          \
        return launchSkipLn<T, C, W>(stream, ld, rows, in, skip, beta, gamma, bias, out, eps);
    B200_SKIPLN_CASE(1, 1)
    B200_SKIPLN_CASE(2, 1)
    B200_SKIPLN_CASE(3, 1)
    B200_SKIPLN_CASE(4, 1)
    B200_SKIPLN_CASE(2, 2)
    B200_SKIPLN_CASE(3, 2)
    B200_SKIPLN_CASE(4, 2)
    B200_SKIPLN_CASE(3, 4)
    B200_SKIPLN_CASE(4, 4)
    B200_SKIPLN_CASE(3, 8)
    B200_SKIPLN_CASE(4, 8)
#undef B200_SKIPLN_CASE
    B200_FAIL(BERT_B200_NOT_SUPPORTED, "skip_layer_norm: no kernel for ld=%d", ld);
}

template <int CPL, int WPR>
int32_t launchDqq(cudaStream_t stream, int32_t ld, int64_t rows, int8_t const* in, int8_t const* skip,
    __half const* beta, __half const* gamma, __half const* bias, int8_t* out, float dqIn, float dqSkip, float qScale)
{
    int const rowsPerCta = kWarpsPerCta / WPR;
    if (CPL <= 2)
    {
        // tables built once per CTA: few CTAs with many rows each
        int const grid = gridFor((rows + rowsPerCta - 1) / rowsPerCta, 3);
        size_t const smem = static_cast<size_t>(ld) * 2 * 3; // three half2 tables of ld / 2 entries
        // rows of 8192 values: the tables plus the kernel's static scratch pass the 48 KB a launch gets without asking
        if (smem > 40 * 1024)
        {
            cudaFuncSetAttribute(skipLnDqqPackedKernel<CPL <= 2 ? CPL : 1, WPR, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                static_cast<int>(smem));
            cudaFuncSetAttribute(skipLnDqqPackedKernel<CPL <= 2 ? CPL : 1, WPR, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                static_cast<int>(smem));
        }
        if (bias)
            launchDependent(skipLnDqqPackedKernel<CPL <= 2 ? CPL : 1, WPR, true>, dim3(grid), dim3(kThreads), smem, stream, ld, rows, in,
                skip, beta, gamma, bias, out, dqIn, dqSkip, qScale, 0.f);
        else
            launchDependent(skipLnDqqPackedKernel<CPL <= 2 ? CPL : 1, WPR, false>, dim3(grid), dim3(kThreads), smem, stream, ld, rows, in,
                skip, beta, gamma, bias, out, dqIn, dqSkip, qScale, 0.f);
        return checkLaunch("skipLnDqqPackedKernel");
    }
    int const grid = gridFor((rows + rowsPerCta - 1) / rowsPerCta, 8);
    if (bias)
        launchDependent(skipLnDqqKernel<CPL, WPR, true>, dim3(grid), dim3(kThreads), 0, stream, ld, rows, in, skip, beta, gamma, bias,
            out, dqIn, dqSkip, qScale, 0.f);
    else
        launchDependent(skipLnDqqKernel<CPL, WPR, false>, dim3(grid), dim3(kThreads), 0, stream, ld, rows, in, skip, beta, gamma,
            bias, out, dqIn, dqSkip, qScale, 0.f);
    return checkLaunch("skipLnDqqKernel");
}

// One row per warp in 8-byte chunks, CPL of them per lane (see the kernel): rows such as 768 or 256 INT8 values.
template <int CPL>
int32_t launchDqq8(cudaStream_t stream, int32_t ld, int64_t rows, int8_t const* in, int8_t const* skip, __half const* beta,
    __half const* gamma, __half const* bias, int8_t* out, float dqIn, float dqSkip, float qScale)
{
    int const grid = gridFor((rows + kWarpsPerCta - 1) / kWarpsPerCta, 3);
    size_t const smem = static_cast<size_t>(ld) * 2 * 3;
    if (bias)
        launchDependent(skipLnDqqPackedKernel<CPL, 1, true, 8>, dim3(grid), dim3(kThreads), smem, stream, ld, rows, in, skip, beta,
            gamma, bias, out, dqIn, dqSkip, qScale, 0.f);
    else
        launchDependent(skipLnDqqPackedKernel<CPL, 1, false, 8>, dim3(grid), dim3(kThreads), smem, stream, ld, rows, in, skip, beta,
            gamma, bias, out, dqIn, dqSkip, qScale, 0.f);
    return checkLaunch("skipLnDqqPackedKernel");
}

template <bool PRELN>
int32_t launchInterleaved(cudaStream_t stream, int32_t ld, int32_t total, int8_t const* in, int8_t const* skip,
    __half const* beta, __half const* gamma, int8_t* out, int8_t* preln, float dqIn, float dqSkip, float qScale,
    float qSkipScale)
{
    int const groups = ld / 32;
    int const ni = (groups + 15) / 16;
    int const tiles = (total + kIlTokens - 1) / kIlTokens;
    int const grid = gridFor(tiles, 8);
    // The large interleaved reference kernels add FP32 epsilon
    // (plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedKernelHFace.cu:178).
    float const eps = std::numeric_limits<float>::epsilon();
    // rows of up to 2048 channels: the packed-arithmetic kernel (tables built once per CTA: few CTAs, many tiles each)
#define B200_IL_PACKED_CASE(N)                                                                                         \
    if (ni == N)                                                                                                       \
    {                                                                                                                  \
        int const gridP = gridFor(tiles, N <= 2 ? 3 : 2);                                                              \
        skipLnInterleavedPackedKernel<N, PRELN><<<gridP, kThreads, static_cast<size_t>(ld) * 4, stream>>>(              \
            ld, total, in, skip, beta, gamma, out, preln, dqIn, dqSkip, qScale, qSkipScale, eps);                      \
        return checkLaunch("skipLnInterleavedPackedKernel");                                                           \
    }
    B200_IL_PACKED_CASE(1)
    B200_IL_PACKED_CASE(2)
    B200_IL_PACKED_CASE(3)
    B200_IL_PACKED_CASE(4)
#undef B200_IL_PACKED_CASE
#define B200_IL_CASE(N)                                                                                                \
    if (ni == N)                                                                                                       \
    {                                                                                                                  \
        skipLnInterleavedKernel<N, PRELN><<<grid, kThreads, 0, stream>>>(                                              \
            ld, total, in, skip, beta, gamma, out, preln, dqIn, dqSkip, qScale, qSkipScale, eps);                      \
        return checkLaunch("skipLnInterleavedKernel");                                                                 \
    }
    B200_IL_CASE(1)
    B200_IL_CASE(2)
    B200_IL_CASE(3)
    B200_IL_CASE(4)
    B200_IL_CASE(6)
    B200_IL_CASE(8)
#undef B200_IL_CASE
    B200_FAIL(BERT_B200_NOT_SUPPORTED, "interleaved skip_layer_norm: unsupported ld=%d", ld);
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int32_t bert_b200_skip_layer_norm(void* stream, int32_t type_id, int32_t ld, int64_t n, void const* input,
    void const* skip, void const* beta, void const* gamma, void* output, void const* bias)
{
    B200_REQUIRE(ld > 0 && n >= 0 && n % ld == 0, "skip_layer_norm: n=%lld is not a multiple of ld=%d",
        static_cast<long long>(n), ld);
    if (n == 0)
        return BERT_B200_OK;
    B200_REQUIRE(input && skip && beta && gamma && output, "skip_layer_norm: null pointer");
    auto s = static_cast<cudaStream_t>(stream);
    if (type_id == BERT_B200_FP16)
        return dispatchSkipLn<__half>(s, ld, n / ld, static_cast<__half const*>(input), static_cast<__half const*>(skip),
            static_cast<__half const*>(beta), static_cast<__half const*>(gamma), static_cast<__half const*>(bias),
            static_cast<__half*>(output));
    if (type_id == BERT_B200_FP32)
        return dispatchSkipLn<float>(s, ld, n / ld, static_cast<float const*>(input), static_cast<float const*>(skip),
            static_cast<float const*>(beta), static_cast<float const*>(gamma), static_cast<float const*>(bias),
            static_cast<float*>(output));
    B200_FAIL(BERT_B200_NOT_SUPPORTED, "skip_layer_norm: type_id %d (INT8 uses bert_b200_skip_layer_norm_dqq)", type_id);
}

extern "C" int32_t bert_b200_skip_layer_norm_dqq(void* stream, int32_t ld, int64_t n, int8_t const* input,
    int8_t const* skip, void const* beta, void const* gamma, int8_t* output, void const* bias, float dq_scale_in,
    float dq_scale_skip, float q_scale)
{
    B200_REQUIRE(ld > 0 && n >= 0 && n % ld == 0, "skip_layer_norm_dqq: n=%lld is not a multiple of ld=%d",
        static_cast<long long>(n), ld);
    if (n == 0)
        return BERT_B200_OK;
    B200_REQUIRE(input && skip && beta && gamma && output, "skip_layer_norm_dqq: null pointer");
    B200_REQUIRE(ld % 16 == 0 && ld <= 16 * 32 * 4 * 8, "skip_layer_norm_dqq: ld=%d must be a multiple of 16, <= 16384", ld);
    B200_REQUIRE(q_scale > 0.f, "skip_layer_norm_dqq: q_scale must be positive");
    B200_REQUIRE(aligned16(input) && aligned16(skip) && aligned16(output) && aligned16(beta) && aligned16(gamma)
            && (!bias || aligned16(bias)),
        "skip_layer_norm_dqq: pointers must be 16-byte aligned");
    if (n == 0)
        return BERT_B200_OK;
    auto s = static_cast<cudaStream_t>(stream);
    int const chunks = ld / 16;
    int wpr = 1;
    while (chunks > 32 * 4 * wpr)
        wpr *= 2;
    // Prefer <= 2 chunks per lane: 16 INT8 values expand to 16 FP32 registers per chunk.
    while (wpr < 8 && chunks > 32 * 2 * wpr)
        wpr *= 2;
    int const cpl = (chunks + 32 * wpr - 1) / (32 * wpr);
    auto const* b = static_cast<__half const*>(beta);
    auto const* g = static_cast<__half const*>(gamma);
    auto const* bi = static_cast<__half const*>(bias);
    // A row that leaves lanes idle in 16-byte chunks but is a whole number of 8-byte chunks per lane (768 = 3 x 32 x 8,
    // 256 = 32 x 8) takes the 8-byte form of the packed kernel: every lane has the same amount of work.
    if (chunks % 32 != 0 && (ld / 8) % 32 == 0 && ld / 8 <= 32 * 3)
    {
        int const cpl8 = ld / 8 / 32;
        if (cpl8 == 1)
            return launchDqq8<1>(s, ld, n / ld, input, skip, b, g, bi, output, dq_scale_in, dq_scale_skip, q_scale);
        if (cpl8 == 3)
            return launchDqq8<3>(s, ld, n / ld, input, skip, b, g, bi, output, dq_scale_in, dq_scale_skip, q_scale);
    }
#define B200_DQQ_CASE(C, W)                                                                                            \
    if (cpl == C && wpr == W)                                                                                          \
        return launchDqq<C, W>(s, ld, n / ld, input, skip, b, g, bi, output, dq_scale_in, dq_scale_skip, q_scale);
    B200_DQQ_CASE(1, 1)
    B200_DQQ_CASE(2, 1)
    B200_DQQ_CASE(2, 2)
    B200_DQQ_CASE(2, 4)
    B200_DQQ_CASE(2, 8)
    B200_DQQ_CASE(3, 8)
    B200_DQQ_CASE(4, 8)
#undef B200_DQQ_CASE
    B200_FAIL(BERT_B200_NOT_SUPPORTED, "skip_layer_norm_dqq: no kernel for ld=%d", ld);
}

static int32_t checkInterleaved(char const* name, int32_t ld, int32_t total, void const* a, void const* b,
    void const* c, void const* d, void const* e)
{
    B200_REQUIRE(ld > 0 && ld % 32 == 0 && ld <= 4096, "%s: ld=%d must be a multiple of 32, <= 4096", name, ld);
    B200_REQUIRE(total >= 0, "%s: total=%d", name, total);
    B200_REQUIRE(a && b && c && d && e, "%s: null pointer", name);
    B200_REQUIRE(aligned16(a) && aligned16(b) && aligned16(c) && aligned16(d) && aligned16(e),
        "%s: pointers must be 16-byte aligned", name);
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_skip_layer_norm_interleaved_hface(void* stream, int32_t ld, int32_t total,
    int8_t const* input, int8_t const* skip, void const* beta, void const* gamma, int8_t* output, float dq_scale_in,
    float dq_scale_skip, float q_scale)
{
    int32_t const st = checkInterleaved("skip_layer_norm_interleaved_hface", ld, total, input, skip, beta, gamma, output);
    if (st != BERT_B200_OK || total == 0)
        return st;
    return launchInterleaved<false>(static_cast<cudaStream_t>(stream), ld, total, input, skip,
        static_cast<__half const*>(beta), static_cast<__half const*>(gamma), output, nullptr, dq_scale_in, dq_scale_skip,
        q_scale, 0.f);
}

extern "C" int32_t bert_b200_skip_layer_norm_interleaved_mtron(void* stream, int32_t ld, int32_t total,
    int8_t const* input, int8_t const* skip, void const* beta, void const* gamma, int8_t* output, int8_t* preln,
    float dq_scale_in, float dq_scale_skip, float q_scale, float q_skip_scale)
{
    int32_t const st = checkInterleaved("skip_layer_norm_interleaved_mtron", ld, total, input, skip, beta, gamma, output);
    if (st != BERT_B200_OK)
        return st;
    B200_REQUIRE(preln && aligned16(preln), "skip_layer_norm_interleaved_mtron: preln must be a 16-byte aligned pointer");
    if (total == 0)
        return st;
    return launchInterleaved<true>(static_cast<cudaStream_t>(stream), ld, total, input, skip,
        static_cast<__half const*>(beta), static_cast<__half const*>(gamma), output, preln, dq_scale_in, dq_scale_skip,
        q_scale, q_skip_scale);
}

// FP32 (type_id 0) fully-connected and attention kernels. FP32 has no tensor-core path that keeps
// full precision (TF32 would break the 1e-5 tolerance the reference configuration states for FP32,
// plugin/bertQKVToContextPlugin/CustomQKVToContextPluginDynamic_PluginConfig.yaml:72-76), so these
// are plain SIMT kernels; the FP16 / INT8 paths live in fc_tcgen05.cu and mha_tcgen05.cu.
// The attention kernel also serves FP16 tensors (FP32 arithmetic) for the shapes the tensor-core kernel does not
// take - heads wider than 64 or not a multiple of 16, sequences longer than 512 - the shapes the reference sends
// to its unfused runner as well.
//
// Replaces cublas{S,H}gemmStridedBatched + softmax kernels of UnfusedMHARunner::run
// (plugin/bertQKVToContextPlugin/mhaRunner.cu:533-601) and the FP32 cublasLtMatmul of the FC plugin
// (plugin/fcPlugin/fcPlugin.cpp:551-610).
#include "common.cuh"

namespace b200
{

namespace
{

__device__ __forceinline__ float geluErf(float x)
{
    return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f));
}

constexpr int kTile = 64;
constexpr int kTileK = 16;

// C[m,n] = act(alpha * sum_k A[m,k] * Wt[n,k] + bias[n]); 64x64 tile, 256 threads, 4x4 per thread.
__global__ void __launch_bounds__(256) fcF32Kernel(int64_t const M, int64_t const N, int64_t const K,
    float const* __restrict__ A, int64_t const lda, float const* __restrict__ Wt, float* __restrict__ C,
    int64_t const ldc, float const* __restrict__ bias, int32_t const act, float const alpha)
{
    __shared__ float sA[kTileK][kTile + 1];
    __shared__ float sB[kTileK][kTile + 1];
    int const tx = threadIdx.x % 16;
    int const ty = threadIdx.x / 16;
    int64_t const m0 = static_cast<int64_t>(blockIdx.y) * kTile;
    int64_t const n0 = static_cast<int64_t>(blockIdx.x) * kTile;
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < K; k0 += kTileK)
    {
        for (int i = threadIdx.x; i < kTile * kTileK; i += 256)
        {
            int const r = i / kTileK;
            int const c = i % kTileK;
            sA[c][r] = (m0 + r < M && k0 + c < K) ? A[(m0 + r) * lda + k0 + c] : 0.f;
            sB[c][r] = (n0 + r < N && k0 + c < K) ? Wt[(n0 + r) * K + k0 + c] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTileK; ++k)
        {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
                a[i] = sA[k][ty * 4 + i];
                b[i] = sB[k][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        int64_t const m = m0 + ty * 4 + i;
        if (m >= M)
            continue;
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            int64_t const n = n0 + tx * 4 + j;
            if (n >= N)
                continue;
            float v = acc[i][j] * alpha + (bias ? bias[n] : 0.f);
            if (act == BERT_B200_ACT_GELU_ERF)
                v = geluErf(v);
            C[m * ldc + n] = v;
        }
    }
}

__device__ __forceinline__ float toFloat(float v)
{
    return v;
}
__device__ __forceinline__ float toFloat(__half v)
{
    return __half2float(v);
}
__device__ __forceinline__ void fromFloat(float& dst, float v)
{
    dst = v;
}
__device__ __forceinline__ void fromFloat(__half& dst, float v)
{
    dst = __float2half_rn(v);
}

// One warp per query row. Scores of the row live in shared memory ([warps][S]); all arithmetic in FP32.
template <typename T>
__global__ void __launch_bounds__(128) mhaSimtKernel(int32_t const B, int32_t const S, int32_t const N, int32_t const d,
    T const* __restrict__ qkv, T* __restrict__ out, int32_t const* __restrict__ cu,
    int32_t const* __restrict__ maskIdx, float const scale)
{
    extern __shared__ float sm[];
    int const lane = threadIdx.x & 31;
    int const warp = threadIdx.x >> 5;
    int const b = blockIdx.y;
    int const n = blockIdx.x;
    float* scores = sm + warp * (S + d);
    float* qs = scores + S;

    int rows, len;
    int64_t row0, rowStride;
    if (cu)
    {
        row0 = cu[b];
        len = cu[b + 1] - cu[b];
        rows = len;
        rowStride = 1;
    }
    else
    {
        row0 = b;
        rowStride = B;
        rows = S;
        len = maskIdx ? min(max(maskIdx[b], 0), S) : S;
    }
    int64_t const tokStride = static_cast<int64_t>(3) * N * d;
    int64_t const headOff = static_cast<int64_t>(n) * 3 * d;
    for (int s = blockIdx.z * 4 + warp; s < rows; s += gridDim.z * 4)
    {
        T const* q = qkv + (row0 + s * rowStride) * tokStride + headOff;
        for (int i = lane; i < d; i += 32)
            qs[i] = toFloat(q[i]);
        __syncwarp();
        float mx = -INFINITY;
        for (int j = lane; j < len; j += 32)
        {
            T const* k = qkv + (row0 + j * rowStride) * tokStride + headOff + d;
            float acc = 0.f;
            for (int i = 0; i < d; ++i)
                acc = fmaf(qs[i], toFloat(k[i]), acc);
            acc *= scale;
            scores[j] = acc;
            mx = fmaxf(mx, acc);
        }
        mx = warpMax(mx);
        float sum = 0.f;
        for (int j = lane; j < len; j += 32)
        {
            float const p = expf(scores[j] - mx);
            scores[j] = p;
            sum += p;
        }
        sum = warpSum(sum);
        float const inv = len > 0 ? 1.f / sum : 0.f;
        __syncwarp();
        T* o = out + (row0 + s * rowStride) * (static_cast<int64_t>(N) * d) + static_cast<int64_t>(n) * d;
        for (int i = lane; i < d; i += 32)
        {
            float acc = 0.f;
            for (int j = 0; j < len; ++j)
                acc = fmaf(scores[j], toFloat(qkv[(row0 + j * rowStride) * tokStride + headOff + 2 * d + i]), acc);
            fromFloat(o[i], acc * inv);
        }
        __syncwarp();
    }
}

} // namespace

int32_t fcF32(bert_b200_fc_params const& p, cudaStream_t stream)
{
    dim3 const grid(static_cast<unsigned>((p.n + kTile - 1) / kTile), static_cast<unsigned>((p.m + kTile - 1) / kTile));
    B200_REQUIRE(grid.y <= 65535, "fc (FP32): m=%lld too large", static_cast<long long>(p.m));
    fcF32Kernel<<<grid, 256, 0, stream>>>(p.m, p.n, p.k, static_cast<float const*>(p.a), p.lda,
        static_cast<float const*>(p.wt), static_cast<float*>(p.c), p.ldc, p.bias, p.activation, p.alpha);
    return checkLaunch("fcF32Kernel");
}

namespace
{

template <typename T>
int32_t launchMhaSimt(bert_b200_mha_params const& p, cudaStream_t stream)
{
    size_t const smem = 4 * static_cast<size_t>(p.S + p.head_size) * sizeof(float);
    B200_REQUIRE(smem <= 200 * 1024, "mha (SIMT): S=%d with head size %d does not fit shared memory", p.S, p.head_size);
    auto kernel = mhaSimtKernel<T>;
    if (smem > 48 * 1024)
    {
        cudaError_t const e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess)
            B200_FAIL(BERT_B200_CUDA_ERROR, "mha (SIMT): cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    int const z = (p.S + 3) / 4 < 32 ? (p.S + 3) / 4 : 32;
    dim3 const grid(p.num_heads, p.B, z > 0 ? z : 1);
    kernel<<<grid, 128, smem, stream>>>(p.B, p.S, p.num_heads, p.head_size, static_cast<T const*>(p.qkv),
        static_cast<T*>(p.out), p.cu_seqlens, p.mask_idx, p.scale_bmm1);
    return checkLaunch("mhaSimtKernel");
}

} // namespace

// FP32 always; FP16 for the shapes outside the tensor-core kernel.
int32_t mhaSimt(bert_b200_mha_params const& p, cudaStream_t stream)
{
    B200_REQUIRE(!p.interleaved, "mha (SIMT): the interleaved layout is INT8 only");
    return p.type_id == BERT_B200_FP16 ? launchMhaSimt<__half>(p, stream) : launchMhaSimt<float>(p, stream);
}

} // namespace b200

// C entry points around the REFERENCE's own kernels (TEST INFRASTRUCTURE, not product).
//
// oracle/build_ref.py compiles the TensorRT-OSS sources named there straight from the reference tree, plus this
// file, into oracle/_ref/libref_bert.so. The tests use it on a GPU to pin the CPU oracle (oracle/bert_oracle.py)
// and the product kernels against what the reference itself computes, and tests/golden/make_golden.py uses it to
// produce the committed golden vectors. Nothing under tensorrt_b200/ links or loads it.
//
// Only declarations of the reference's free functions appear here (signatures as in
// plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:219-286, skipLayerNormInt8InterleavedKernel{HFace,MTron}.cu,
// plugin/embLayerNormPlugin/embLayerNormKernel.cu:87-96, 159-183, 237-252, embLayerNormVarSeqlenKernel{HFace,MTron}.cu);
// the attention kernels are the precompiled sm100 binaries the reference ships, launched through its own
// FusedMultiHeadAttentionXMMAKernelV2::run (plugin/bertQKVToContextPlugin/fused_multihead_attention_v2/
// fused_multihead_attention_v2.h:1083-1239) with parameters filled like mhaRunner.cu:985-1035 and :1160-1200; the
// fixed-length kernels of plugin versions 1-3 through FusedMultiHeadAttentionXMMAKernel::run
// (fused_multihead_attention/fused_multihead_attention.h) with parameters filled like mhaRunner.cu:653-713 and :797-850.
#include "bertQKVToContextPlugin/fused_multihead_attention_v2/fused_multihead_attention_v2.h"
#include <NvInferRuntime.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>

namespace nvinfer1
{
namespace plugin
{
namespace bert
{
template <typename T, bool hasBias>
int32_t computeSkipLayerNorm(cudaStream_t stream, int32_t const ld, int32_t const n, T const* input, T const* skip,
    T const* beta, T const* gamma, T* output, T const* bias);
template <bool hasBias>
int32_t computeSkipLayerNormDQQ(cudaStream_t stream, int32_t const ld, int32_t const n, int8_t const* input,
    int8_t const* skip, __half const* beta, __half const* gamma, int8_t* output, __half const* bias, float const dqScaleIn,
    float const dqScaleSkip, float const qScale);
int32_t launch_small_hface(cudaStream_t stream, int32_t const ld, int32_t const total, int8_t const* input, int8_t const* skip,
    half const* beta, half const* gamma, int8_t* output, float const dqScaleIn, float const dqScaleSkip, float const qScale);
int32_t launch_large_hface(cudaStream_t stream, int32_t const ld, int32_t const total, int8_t const* input, int8_t const* skip,
    half const* beta, half const* gamma, int8_t* output, float const dqScaleIn, float const dqScaleSkip, float const qScale);
int32_t launch_small_mtron(cudaStream_t stream, int32_t const ld, int32_t const total, int8_t const* input, int8_t const* skip,
    half const* beta, half const* gamma, int8_t* output, int8_t* preln, float const dqScaleIn, float const dqScaleSkip,
    float const qScale, float const qSkipScale);
int32_t launch_large_mtron(cudaStream_t stream, int32_t const ld, int32_t const total, int8_t const* input, int8_t const* skip,
    half const* beta, half const* gamma, int8_t* output, int8_t* preln, float const dqScaleIn, float const dqScaleSkip,
    float const qScale, float const qSkipScale);
template <typename T>
int embSkipLayerNorm(cudaStream_t stream, int ld, int B, int S, int32_t const* inputIds, int32_t const* tokenIds,
    float const* beta, float const* gamma, T const* wordEmb, T const* posEmb, T const* tokEmb, int32_t const wordSize,
    int32_t const tokSize, T* output);
template <typename T>
int32_t embSkipLayerNormHFace(cudaStream_t stream, int32_t ld, int32_t B, int32_t S, int32_t const* inputIds,
    int32_t const* tokenIds, int32_t const* cuSeqlens, float const* beta, float const* gamma, T const* wordEmb,
    T const* posEmb, T const* tokEmb, int32_t const wordSize, int32_t const tokSize, T* output);
template <typename T>
int32_t embSkipLayerNormMTron(cudaStream_t stream, int32_t ld, int32_t B, int32_t S, int32_t const* inputIds,
    int32_t const* tokenIds, int32_t const* cuSeqlens, float const* beta, float const* gamma, T const* wordEmb,
    T const* posEmb, T const* tokEmb, int32_t const wordSize, int32_t const tokSize, T* output, T* skip);
int computeMaskIdx(cudaStream_t stream, int32_t const S, int32_t const B, int32_t const* mask, int* maskIdx);
cudaError_t convertMask(uint32_t const S, uint32_t const B, uint32_t const warps_m, uint32_t const warps_n,
    uint32_t const warps_k, int32_t const* inputMaskSB, uint32_t* inputMaskX, cudaStream_t stream);
} // namespace bert
} // namespace plugin
} // namespace nvinfer1

// The plugin sources log through ::getLogger(), which normally comes from libnvinfer (not installed): stderr stand-in.
namespace
{
class StderrLogger : public nvinfer1::ILogger
{
    void log(Severity severity, char const* msg) noexcept override
    {
        if (severity <= Severity::kWARNING)
            fprintf(stderr, "[reference] %s\n", msg);
    }
} gStderrLogger;
} // namespace

extern "C" nvinfer1::ILogger* getLogger() noexcept
{
    return &gStderrLogger;
}

using namespace nvinfer1::plugin::bert;
#define REF_API extern "C" __attribute__((visibility("default")))

REF_API int32_t ref_skip_layer_norm(void* stream, int32_t type_id, int32_t ld, int32_t n, void const* in, void const* skip,
    void const* beta, void const* gamma, void* out, void const* bias)
{
    auto s = static_cast<cudaStream_t>(stream);
    try
    {
        if (type_id == 1)
        {
            auto h = [](void const* p) { return static_cast<__half const*>(p); };
            return bias ? computeSkipLayerNorm<__half, true>(s, ld, n, h(in), h(skip), h(beta), h(gamma), static_cast<__half*>(out), h(bias))
                        : computeSkipLayerNorm<__half, false>(s, ld, n, h(in), h(skip), h(beta), h(gamma), static_cast<__half*>(out), h(bias));
        }
        auto f = [](void const* p) { return static_cast<float const*>(p); };
        return bias ? computeSkipLayerNorm<float, true>(s, ld, n, f(in), f(skip), f(beta), f(gamma), static_cast<float*>(out), f(bias))
                    : computeSkipLayerNorm<float, false>(s, ld, n, f(in), f(skip), f(beta), f(gamma), static_cast<float*>(out), f(bias));
    }
    catch (...)
    {
        return -1;
    }
}

REF_API int32_t ref_skip_layer_norm_dqq(void* stream, int32_t ld, int32_t n, int8_t const* in, int8_t const* skip, void const* beta,
    void const* gamma, int8_t* out, void const* bias, float dqIn, float dqSkip, float qScale)
{
    auto s = static_cast<cudaStream_t>(stream);
    auto h = [](void const* p) { return static_cast<__half const*>(p); };
    try
    {
        return bias ? computeSkipLayerNormDQQ<true>(s, ld, n, in, skip, h(beta), h(gamma), out, h(bias), dqIn, dqSkip, qScale)
                    : computeSkipLayerNormDQQ<false>(s, ld, n, in, skip, h(beta), h(gamma), out, h(bias), dqIn, dqSkip, qScale);
    }
    catch (...)
    {
        return -1;
    }
}

// variant: 0 small hface, 1 large hface, 2 small mtron, 3 large mtron
REF_API int32_t ref_skip_layer_norm_interleaved(void* stream, int32_t variant, int32_t ld, int32_t total, int8_t const* in,
    int8_t const* skip, void const* beta, void const* gamma, int8_t* out, int8_t* preln, float dqIn, float dqSkip, float qScale,
    float qSkipScale)
{
    auto s = static_cast<cudaStream_t>(stream);
    auto const* b = static_cast<half const*>(beta);
    auto const* g = static_cast<half const*>(gamma);
    try
    {
        switch (variant)
        {
        case 0: return launch_small_hface(s, ld, total, in, skip, b, g, out, dqIn, dqSkip, qScale);
        case 1: return launch_large_hface(s, ld, total, in, skip, b, g, out, dqIn, dqSkip, qScale);
        case 2: return launch_small_mtron(s, ld, total, in, skip, b, g, out, preln, dqIn, dqSkip, qScale, qSkipScale);
        case 3: return launch_large_mtron(s, ld, total, in, skip, b, g, out, preln, dqIn, dqSkip, qScale, qSkipScale);
        }
    }
    catch (...)
    {
    }
    return -1;
}

REF_API int32_t ref_emb_layer_norm(void* stream, int32_t type_id, int32_t ld, int32_t B, int32_t S, int32_t const* ids,
    int32_t const* seg, float const* beta, float const* gamma, void const* word, void const* pos, void const* tok,
    int32_t wordSize, int32_t tokSize, void* out)
{
    auto s = static_cast<cudaStream_t>(stream);
    try
    {
        if (type_id == 1)
            return embSkipLayerNorm<half>(s, ld, B, S, ids, seg, beta, gamma, static_cast<half const*>(word),
                static_cast<half const*>(pos), static_cast<half const*>(tok), wordSize, tokSize, static_cast<half*>(out));
        return embSkipLayerNorm<float>(s, ld, B, S, ids, seg, beta, gamma, static_cast<float const*>(word),
            static_cast<float const*>(pos), static_cast<float const*>(tok), wordSize, tokSize, static_cast<float*>(out));
    }
    catch (...)
    {
        return -1;
    }
}

// skip_out != NULL selects the MTron kernel (second output), else HFace. FP16 only.
REF_API int32_t ref_emb_layer_norm_var_seqlen(void* stream, int32_t ld, int32_t B, int32_t S, int32_t const* ids, int32_t const* seg,
    int32_t const* cu, float const* beta, float const* gamma, void const* word, void const* pos, void const* tok,
    int32_t wordSize, int32_t tokSize, void* out, void* skip_out)
{
    auto s = static_cast<cudaStream_t>(stream);
    auto h = [](void const* p) { return static_cast<half const*>(p); };
    try
    {
        if (skip_out)
            return embSkipLayerNormMTron<half>(s, ld, B, S, ids, seg, cu, beta, gamma, h(word), h(pos), h(tok), wordSize, tokSize,
                static_cast<half*>(out), static_cast<half*>(skip_out));
        return embSkipLayerNormHFace<half>(s, ld, B, S, ids, seg, cu, beta, gamma, h(word), h(pos), h(tok), wordSize, tokSize,
            static_cast<half*>(out));
    }
    catch (...)
    {
        return -1;
    }
}

REF_API int32_t ref_compute_mask_idx(void* stream, int32_t S, int32_t B, int32_t const* mask, int32_t* maskIdx)
{
    return computeMaskIdx(static_cast<cudaStream_t>(stream), S, B, mask, maskIdx);
}

REF_API int32_t ref_convert_mask(uint32_t S, uint32_t B, uint32_t wm, uint32_t wn, uint32_t wk, int32_t const* mask, uint32_t* maskX,
    void* stream)
{
    return static_cast<int32_t>(convertMask(S, B, wm, wn, wk, mask, maskX, static_cast<cudaStream_t>(stream)));
}

// The reference's precompiled sm100 var-seqlen attention kernels. type_id 1: FP16 [total][N][3][d];
// type_id 2: INT8, linear or (interleaved != 0) CHW32 [3][N][d/32][total][32]. S is the kernel's sequence-length
// bucket (64, 96, 128, (192 INT8), 256, 384, 512 - what the plugin picks from the maximum length).
REF_API int32_t ref_fmha_v2(void* stream, int32_t type_id, int32_t B, int32_t S, int32_t N, int32_t d, int32_t total, void* qkv,
    void* out, int32_t* cu_seqlens, int32_t interleaved, float scale_bmm1, float scale_softmax, float scale_bmm2)
{
    try
    {
        Data_type const dt = type_id == 2 ? DATA_TYPE_INT8 : DATA_TYPE_FP16;
        FusedMultiHeadAttentionXMMAKernelV2 const* k = getXMMAKernelsV2(dt, kSM_100);
        if (!k || !k->isValid(d, S))
            return -2;
        Fused_multihead_attention_params_v2 p{};
        p.b = B;
        p.h = N;
        p.s = S;
        p.d = d;
        p.qkv_ptr = qkv;
        p.o_ptr = out;
        p.cu_seqlens = cu_seqlens;
        p.packed_mask_ptr = nullptr;
        if (type_id == 2)
        {
            p.scale_bmm1 = reinterpret_cast<uint32_t const&>(scale_bmm1);
            p.scale_bmm2 = reinterpret_cast<uint32_t const&>(scale_bmm2);
            p.scale_softmax = reinterpret_cast<uint32_t const&>(scale_softmax);
            p.enable_i2f_trick = -double(1 << 22) * double(scale_bmm2) <= -128.f && double(1 << 22) * double(scale_bmm2) >= 127.f;
            p.use_int8_scale_max = true;
            p.interleaved = interleaved != 0;
            p.qkv_stride_in_bytes = interleaved ? total : 3 * N * d;
            p.o_stride_in_bytes = interleaved ? total : N * d;
        }
        else
        {
            half2 h1 = __float2half2_rn(scale_bmm1), h2 = __float2half2_rn(1.f);
            p.scale_bmm1 = reinterpret_cast<uint32_t const&>(h1);
            p.scale_softmax = reinterpret_cast<uint32_t const&>(h2);
            p.scale_bmm2 = reinterpret_cast<uint32_t const&>(h2);
            p.qkv_stride_in_bytes = 3 * N * d * 2;
            p.o_stride_in_bytes = N * d * 2;
        }
        k->run(p, static_cast<cudaStream_t>(stream));
        return static_cast<int32_t>(cudaPeekAtLastError());
    }
    catch (std::exception const& e)
    {
        fprintf(stderr, "[reference] %s\n", e.what());
        return -1;
    }
}

// The reference's precompiled sm100 FIXED-LENGTH attention kernels (plugin versions 1-3). qkv is [S][B][N][3][d]
// (FP16 or INT8), out [S][B][N][d], packed_mask the output of convertMask for the same S and B (warps 2 x 2 for
// S <= 128, 1 x 8 for S = 384). The runner accepts S in {64, 96, 128, 384} for FP16 and {128, 384} for INT8.
REF_API int32_t ref_fmha_v1(void* stream, int32_t type_id, int32_t B, int32_t S, int32_t N, int32_t d, void* qkv, void* out,
    void* packed_mask, float scale_bmm1, float scale_softmax, float scale_bmm2)
{
    try
    {
        bool const int8 = type_id == 2;
        if (!(S == 128 || S == 384 || (!int8 && (S == 64 || S == 96))))
            return -2;
        FusedMultiHeadAttentionXMMAKernel const* k = getXMMAKernels(int8 ? DATA_TYPE_INT8 : DATA_TYPE_FP16, kSM_100);
        if (!k || !k->isValid(d, S))
            return -2;
        uint32_t const warpsM = S == 384 ? 1 : 2, warpsN = S == 384 ? 8 : 2;
        uint32_t const threadsPerCta = warpsM * warpsN * 32;
        uint32_t const xmmasM = (S + 16 * warpsM - 1) / (16 * warpsM);
        Fused_multihead_attention_params p{};
        p.b = B;
        p.h = N;
        p.s = S;
        p.d = d;
        p.qkv_ptr = qkv;
        p.packed_mask_ptr = packed_mask;
        p.o_ptr = out;
        int64_t const elem = int8 ? 1 : 2;
        p.qkv_stride_in_bytes = static_cast<int64_t>(3) * B * N * d * elem;
        p.o_stride_in_bytes = static_cast<int64_t>(B) * N * d * elem;
        p.packed_mask_stride_in_bytes = static_cast<int64_t>(xmmasM) * threadsPerCta * sizeof(uint32_t);
        if (int8)
        {
            p.scale_bmm1 = reinterpret_cast<uint32_t const&>(scale_bmm1);
            p.scale_bmm2 = reinterpret_cast<uint32_t const&>(scale_bmm2);
            p.scale_softmax = reinterpret_cast<uint32_t const&>(scale_softmax);
            p.enable_i2f_trick = -double(1 << 22) * double(scale_bmm2) <= -128.f && double(1 << 22) * double(scale_bmm2) >= 127.f;
        }
        else
        {
            half2 h1 = __float2half2_rn(scale_bmm1), h2 = __float2half2_rn(1.f);
            p.scale_bmm1 = reinterpret_cast<uint32_t const&>(h1);
            p.scale_softmax = reinterpret_cast<uint32_t const&>(h2);
            p.scale_bmm2 = reinterpret_cast<uint32_t const&>(h2);
        }
        k->run(p, static_cast<cudaStream_t>(stream));
        return static_cast<int32_t>(cudaPeekAtLastError());
    }
    catch (std::exception const& e)
    {
        fprintf(stderr, "[reference] %s\n", e.what());
        return -1;
    }
}

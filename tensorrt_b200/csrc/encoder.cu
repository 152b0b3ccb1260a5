// Host-side BERT encoder driver: the layer loop that strings the plugin kernels together, in the
// order the reference BERT network used them (EmbLayerNorm -> per layer: FC(QKV) -> QKVToContext ->
// FC -> SkipLayerNorm -> FC+GELU -> FC -> SkipLayerNorm). The reference tree dropped that network
// builder (demo/BERT, CHANGELOG.md:24); its plugin-level pieces are
// plugin/embLayerNormPlugin/embLayerNormVarSeqlenPlugin.cpp:370-514, plugin/fcPlugin/fcPlugin.cpp:551-610,
// plugin/bertQKVToContextPlugin/qkvToContextPlugin.cpp:1210-1324 and
// plugin/skipLayerNormPlugin/skipLayerNormPlugin.cpp:698-785.
//
// All device memory (weights, workspace, I/O) belongs to the caller; nothing is allocated here.
#include "common.cuh"

#include <cmath>
#include <mutex>
#include <new>
#include <vector>

struct bert_b200_encoder
{
    bert_b200_encoder_config cfg;
    std::vector<bert_b200_layer_weights> layers;
    int32_t lastLaunches = 0;
    // optional per-launch timing: events[2*i], events[2*i+1] bracket launch i of kind kinds[i]
    bool timing = false;
    std::vector<cudaEvent_t> events;
    std::vector<int32_t> kinds;
    int32_t timedLaunches = 0;
    // optional calibration: device array [num_layers][8] receiving |x| maxima
    float* amaxDev = nullptr;
    // pipelined host interface: per slot "encoder output complete" and "output copied to the host" (created on first use)
    cudaEvent_t computeDone[2] = {nullptr, nullptr};
    cudaEvent_t copyDone[2] = {nullptr, nullptr};
    bool slotUsed[2] = {false, false};

    ~bert_b200_encoder()
    {
        for (cudaEvent_t e : events)
            cudaEventDestroy(e);
        for (int i = 0; i < 2; ++i)
        {
            if (computeDone[i])
                cudaEventDestroy(computeDone[i]);
            if (copyDone[i])
                cudaEventDestroy(copyDone[i]);
        }
    }
};

namespace b200
{
namespace
{

inline int64_t alignUp(int64_t v, int64_t a)
{
    return (v + a - 1) / a * a;
}

struct Workspace
{
    int32_t* ids;
    int32_t* seg;
    int32_t* cu;
    uint32_t* status;
    uint8_t* x;    // [T][E]   layer input / output
    uint8_t* qkv;  // [T][3E]
    uint8_t* ctx;  // [T][E]
    uint8_t* ao;   // [T][E]   attention output projection, later FFN output projection
    uint8_t* h1;   // [T][E]
    uint8_t* f1;   // [T][F]
    uint8_t* xf16; // [T][E]   FP16 copy of the embedding output (INT8 mode)
    int64_t bytes;
};

Workspace carve(bert_b200_encoder_config const& c, int32_t maxTokens, int32_t maxBatch, void* base)
{
    int64_t const elem = c.type_id == BERT_B200_INT8 ? 1 : 2;
    int64_t const T = maxTokens;
    int64_t const E = c.hidden_size;
    int64_t const F = c.ffn_size;
    int64_t off = 0;
    auto take = [&](int64_t n) {
        int64_t const o = off;
        off = alignUp(off + n, 1024);
        return o;
    };
    int64_t const oIds = take(T * 4);
    int64_t const oSeg = take(T * 4);
    int64_t const oCu = take((static_cast<int64_t>(maxBatch) + 1) * 4);
    int64_t const oStatus = take(16);
    int64_t const oX = take(T * E * elem);
    int64_t const oQkv = take(T * 3 * E * elem);
    int64_t const oCtx = take(T * E * elem);
    int64_t const oAo = take(T * E * elem);
    int64_t const oH1 = take(T * E * elem);
    int64_t const oF1 = take(T * F * elem);
    int64_t const oXf = c.type_id == BERT_B200_INT8 ? take(T * E * 2) : oX;
    Workspace w{};
    auto* b = static_cast<uint8_t*>(base);
    w.ids = reinterpret_cast<int32_t*>(b + oIds);
    w.seg = reinterpret_cast<int32_t*>(b + oSeg);
    w.cu = reinterpret_cast<int32_t*>(b + oCu);
    w.status = reinterpret_cast<uint32_t*>(b + oStatus);
    w.x = b + oX;
    w.qkv = b + oQkv;
    w.ctx = b + oCtx;
    w.ao = b + oAo;
    w.h1 = b + oH1;
    w.f1 = b + oF1;
    w.xf16 = b + oXf;
    w.bytes = off;
    return w;
}

__global__ void dequantKernel(int64_t const n16, int8_t const* __restrict__ in, __half* __restrict__ out, float const scale)
{
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n16;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        uint4 const v = ldgStream(in + i * 16);
        uint32_t const* w = reinterpret_cast<uint32_t const*>(&v);
        float f[16];
#pragma unroll
        for (int k = 0; k < 4; ++k)
        {
            float t[4];
            unpackChar4(w[k], t);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                f[4 * k + j] = t[j] * scale;
        }
        float lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            lo[j] = f[j];
            hi[j] = f[8 + j];
        }
        stgStream(out + i * 16, packHalf8(lo));
        stgStream(out + i * 16 + 8, packHalf8(hi));
    }
}

// |x| maximum of `n8` groups of eight FP16 values, folded into *dst with an integer max
// (non-negative floats order like their bit patterns).
__global__ void amaxKernel(int64_t const n8, __half const* __restrict__ in, float* __restrict__ dst)
{
    float m = 0.f;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n8;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        float f[8];
        unpackHalf8(ldgStream(in + i * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            m = fmaxf(m, fabsf(f[j]));
    }
    m = warpMax(m);
    if ((threadIdx.x & 31) == 0)
        atomicMax(reinterpret_cast<unsigned int*>(dst), __float_as_uint(m));
}

int32_t checkConfig(bert_b200_encoder_config const* c)
{
    B200_REQUIRE(c != nullptr, "encoder: null config");
    B200_REQUIRE(c->type_id == BERT_B200_FP16 || c->type_id == BERT_B200_INT8, "encoder: type_id %d", c->type_id);
    B200_REQUIRE(c->num_layers > 0 && c->hidden_size > 0 && c->num_heads > 0 && c->ffn_size > 0, "encoder: bad sizes");
    B200_REQUIRE(c->hidden_size % c->num_heads == 0 && c->hidden_size / c->num_heads <= 64
            && (c->hidden_size / c->num_heads) % 16 == 0,
        "encoder: head size must be 16, 32, 48 or 64 (hidden %d, heads %d)", c->hidden_size, c->num_heads);
    B200_REQUIRE(c->ffn_size % 16 == 0, "encoder: ffn_size must be a multiple of 16");
    B200_REQUIRE(c->word_emb && c->pos_emb && c->tok_emb && c->emb_gamma && c->emb_beta && c->layers_host,
        "encoder: null weight pointer");
    return BERT_B200_OK;
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int64_t bert_b200_encoder_workspace_size(bert_b200_encoder_config const* cfg, int32_t max_tokens, int32_t max_batch)
{
    if (checkConfig(cfg) != BERT_B200_OK || max_tokens < 0 || max_batch < 0)
        return -1;
    return carve(*cfg, max_tokens, max_batch, nullptr).bytes;
}

extern "C" int32_t bert_b200_encoder_create(bert_b200_encoder_config const* cfg, bert_b200_encoder** out)
{
    int32_t const st = checkConfig(cfg);
    if (st != BERT_B200_OK)
        return st;
    B200_REQUIRE(out != nullptr, "encoder_create: null output");
    auto* e = new (std::nothrow) bert_b200_encoder();
    if (!e)
        B200_FAIL(BERT_B200_FAILURE, "encoder_create: out of host memory");
    e->cfg = *cfg;
    e->layers.assign(cfg->layers_host, cfg->layers_host + cfg->num_layers);
    e->cfg.layers_host = e->layers.data();
    for (auto const& l : e->layers)
    {
        if (!(l.wt_qkv && l.b_qkv && l.wt_out && l.b_out && l.ln1_gamma && l.ln1_beta && l.wt_ffn1 && l.b_ffn1 && l.wt_ffn2
                && l.b_ffn2 && l.ln2_gamma && l.ln2_beta))
        {
            delete e;
            B200_FAIL(BERT_B200_BAD_PARAM, "encoder_create: null layer weight pointer");
        }
    }
    if (cfg->type_id == BERT_B200_INT8)
    {
        // a zero or non-finite scale turns 1 / s into inf / NaN inside the quantising epilogues, and a layer that
        // dequantises its input with another step than the one the previous layer quantised with is silently wrong
        auto good = [](float v) { return std::isfinite(v) && v > 0.f; };
        for (size_t i = 0; i < e->layers.size(); ++i)
        {
            auto const& l = e->layers[i];
            bool const ok = good(l.s_in) && good(l.s_wqkv) && good(l.s_qkv) && good(l.s_ctx) && good(l.s_wout) && good(l.s_attn_out)
                && good(l.s_ln1) && good(l.s_wffn1) && good(l.s_ffn1) && good(l.s_wffn2) && good(l.s_ffn2) && good(l.s_out)
                && good(cfg->dq_probs);
            bool const chained = i == 0 || e->layers[i - 1].s_out == l.s_in;
            if (!ok || !chained)
            {
                int const layer = static_cast<int>(i);
                delete e;
                if (!ok)
                    B200_FAIL(BERT_B200_BAD_PARAM, "encoder_create: layer %d has a scale (or dq_probs) that is not finite and positive", layer);
                B200_FAIL(BERT_B200_BAD_PARAM, "encoder_create: layer %d dequantises its input with s_in != s_out of layer %d", layer, layer - 1);
            }
        }
    }
    *out = e;
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_encoder_destroy(bert_b200_encoder* enc)
{
    delete enc;
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_encoder_last_launch_count(bert_b200_encoder const* enc)
{
    return enc ? enc->lastLaunches : 0;
}

static int32_t forwardImpl(bert_b200_encoder* enc, cudaStream_t stream, int32_t B, int32_t total, int32_t maxSeqlen,
    int32_t const* ids, int32_t const* seg, int32_t const* cu, Workspace const& w, void* output)
{
    bert_b200_encoder_config const& c = enc->cfg;
    bool const i8 = c.type_id == BERT_B200_INT8;
    int32_t const E = c.hidden_size;
    int32_t const F = c.ffn_size;
    int64_t const T = total;
    int32_t launches = 0;
    int32_t st;
    enc->timedLaunches = 0;
    auto mark = [&](int32_t kind, bool begin) -> int32_t {
        if (!enc->timing)
            return BERT_B200_OK;
        size_t const idx = static_cast<size_t>(enc->timedLaunches) * 2 + (begin ? 0 : 1);
        while (enc->events.size() <= idx)
        {
            cudaEvent_t e;
            if (cudaEventCreate(&e) != cudaSuccess)
                B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward: cudaEventCreate failed");
            enc->events.push_back(e);
        }
        if (begin)
        {
            if (enc->kinds.size() <= static_cast<size_t>(enc->timedLaunches))
                enc->kinds.resize(enc->timedLaunches + 1);
            enc->kinds[enc->timedLaunches] = kind;
        }
        if (cudaEventRecord(enc->events[idx], stream) != cudaSuccess)
            B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward: cudaEventRecord failed");
        if (!begin)
            ++enc->timedLaunches;
        return BERT_B200_OK;
    };
    // calibration: fold max|t| of an FP16 tensor of n elements into amaxDev[layer][slot]
    auto amax = [&](void const* t, int64_t n, int32_t layer, int32_t slot) {
        if (!enc->amaxDev)
            return;
        int64_t const n8 = n / 8;
        int const grid = static_cast<int>(n8 / 256 + 1 < smCount() * 8 ? n8 / 256 + 1 : smCount() * 8);
        amaxKernel<<<grid, 256, 0, stream>>>(n8, static_cast<__half const*>(t), enc->amaxDev + layer * 8 + slot);
    };
#define B200_STEP(kind, call)                                                                                          \
    do                                                                                                                 \
    {                                                                                                                  \
        st = mark(kind, true);                                                                                         \
        if (st == BERT_B200_OK)                                                                                        \
            st = (call);                                                                                               \
        if (st == BERT_B200_OK)                                                                                        \
            st = mark(kind, false);                                                                                    \
        if (st != BERT_B200_OK)                                                                                        \
            return st;                                                                                                 \
        ++launches;                                                                                                    \
    } while (0)

    if (cudaMemsetAsync(w.status, 0, sizeof(uint32_t), stream) != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward: clearing the status word failed");
    // FP16: embedding output is the first layer input. INT8: additionally quantised with the first layer's input scale.
    B200_STEP(BERT_B200_KIND_EMB, bert_b200_emb_layer_norm_var_seqlen(stream, BERT_B200_FP16, E, B, maxSeqlen, total, ids, seg, cu, c.emb_beta,
        c.emb_gamma, c.word_emb, c.pos_emb, c.tok_emb, c.vocab_size, c.type_vocab_size, c.max_positions, i8 ? static_cast<void*>(w.xf16) : w.x,
        nullptr, i8 ? reinterpret_cast<int8_t*>(w.x) : nullptr, i8 ? 1.f / enc->layers[0].s_in : 0.f));

    int32_t const headSize = c.hidden_size / c.num_heads;
    float const rsqrtD = 1.f / std::sqrt(static_cast<float>(headSize));
    for (int32_t li = 0; li < c.num_layers; ++li)
    {
        bert_b200_layer_weights const& l = enc->layers[li];
        bert_b200_fc_params fc{};
        fc.type_id = c.type_id;
        fc.out_type_id = c.type_id;
        fc.m = T;
        fc.status_word = w.status;

        // QKV projection (+ bias)
        fc.n = 3 * E;
        fc.k = E;
        fc.a = w.x;
        fc.lda = E;
        fc.wt = l.wt_qkv;
        fc.c = w.qkv;
        fc.ldc = 3 * E;
        fc.bias = l.b_qkv;
        fc.activation = BERT_B200_ACT_NONE;
        fc.alpha = i8 ? l.s_in * l.s_wqkv : 1.f;
        fc.out_scale = i8 ? 1.f / l.s_qkv : 1.f;
        amax(w.x, T * E, li, 0);
        B200_STEP(BERT_B200_KIND_FC, bert_b200_fc(&fc, stream));
        amax(w.qkv, T * 3 * E, li, 1);

        bert_b200_mha_params mha{};
        mha.type_id = c.type_id;
        mha.B = B;
        mha.S = maxSeqlen;
        mha.num_heads = c.num_heads;
        mha.head_size = headSize;
        mha.total = total;
        mha.qkv = w.qkv;
        mha.out = w.ctx;
        mha.cu_seqlens = cu;
        mha.scale_bmm1 = i8 ? l.s_qkv * l.s_qkv * rsqrtD : rsqrtD;
        mha.scale_softmax = i8 ? 1.f / c.dq_probs : 1.f;
        mha.scale_bmm2 = i8 ? c.dq_probs * l.s_qkv / l.s_ctx : 1.f;
        mha.status_word = w.status;
        B200_STEP(BERT_B200_KIND_MHA, bert_b200_mha(&mha, stream));
        amax(w.ctx, T * E, li, 2);

        // attention output projection (bias is applied by the SkipLayerNorm that follows)
        fc.n = E;
        fc.k = E;
        fc.a = w.ctx;
        fc.lda = E;
        fc.wt = l.wt_out;
        fc.c = w.ao;
        fc.ldc = E;
        fc.bias = nullptr;
        fc.alpha = i8 ? l.s_ctx * l.s_wout : 1.f;
        fc.out_scale = i8 ? 1.f / l.s_attn_out : 1.f;
        B200_STEP(BERT_B200_KIND_FC, bert_b200_fc(&fc, stream));
        amax(w.ao, T * E, li, 3);

        if (i8)
            B200_STEP(BERT_B200_KIND_SKIPLN, bert_b200_skip_layer_norm_dqq(stream, E, T * E, reinterpret_cast<int8_t*>(w.ao),
                reinterpret_cast<int8_t*>(w.x), l.ln1_beta, l.ln1_gamma, reinterpret_cast<int8_t*>(w.h1), l.b_out,
                l.s_attn_out, l.s_in, 1.f / l.s_ln1));
        else
            B200_STEP(BERT_B200_KIND_SKIPLN, bert_b200_skip_layer_norm(
                stream, BERT_B200_FP16, E, T * E, w.ao, w.x, l.ln1_beta, l.ln1_gamma, w.h1, l.b_out));

        amax(w.h1, T * E, li, 4);
        // FFN up projection + bias + erf-GELU
        fc.n = F;
        fc.k = E;
        fc.a = w.h1;
        fc.lda = E;
        fc.wt = l.wt_ffn1;
        fc.c = w.f1;
        fc.ldc = F;
        fc.bias = l.b_ffn1;
        fc.activation = BERT_B200_ACT_GELU_ERF;
        fc.alpha = i8 ? l.s_ln1 * l.s_wffn1 : 1.f;
        fc.out_scale = i8 ? 1.f / l.s_ffn1 : 1.f;
        B200_STEP(BERT_B200_KIND_FC, bert_b200_fc(&fc, stream));
        amax(w.f1, T * F, li, 5);

        // FFN down projection
        fc.n = E;
        fc.k = F;
        fc.a = w.f1;
        fc.lda = F;
        fc.wt = l.wt_ffn2;
        fc.c = w.ao;
        fc.ldc = E;
        fc.bias = nullptr;
        fc.activation = BERT_B200_ACT_NONE;
        fc.alpha = i8 ? l.s_ffn1 * l.s_wffn2 : 1.f;
        fc.out_scale = i8 ? 1.f / l.s_ffn2 : 1.f;
        B200_STEP(BERT_B200_KIND_FC, bert_b200_fc(&fc, stream));
        amax(w.ao, T * E, li, 6);

        bool const last = li + 1 == c.num_layers;
        if (i8)
            B200_STEP(BERT_B200_KIND_SKIPLN, bert_b200_skip_layer_norm_dqq(stream, E, T * E, reinterpret_cast<int8_t*>(w.ao),
                reinterpret_cast<int8_t*>(w.h1), l.ln2_beta, l.ln2_gamma, reinterpret_cast<int8_t*>(w.x), l.b_ffn2, l.s_ffn2,
                l.s_ln1, 1.f / l.s_out));
        else
            B200_STEP(BERT_B200_KIND_SKIPLN, bert_b200_skip_layer_norm(stream, BERT_B200_FP16, E, T * E, w.ao, w.h1, l.ln2_beta, l.ln2_gamma,
                last ? output : static_cast<void*>(w.x), l.b_ffn2));
        if (!i8)
            amax(last ? output : static_cast<void*>(w.x), T * E, li, 7);
    }
    if (i8)
    {
        int64_t const n16 = T * E / 16;
        int const grid = static_cast<int>(n16 / 256 + 1 < smCount() * 8 ? n16 / 256 + 1 : smCount() * 8);
        auto dequant = [&]() -> int32_t {
            dequantKernel<<<grid, 256, 0, stream>>>(
                n16, reinterpret_cast<int8_t const*>(w.x), static_cast<__half*>(output), enc->layers.back().s_out);
            return checkLaunch("dequantKernel");
        };
        B200_STEP(BERT_B200_KIND_OTHER, dequant());
    }
#undef B200_STEP
    enc->lastLaunches = launches;
    return BERT_B200_OK;
}

static int32_t checkForward(bert_b200_encoder* enc, int32_t B, int32_t total, int32_t maxSeqlen, void const* a,
    void const* b, void const* c, void* workspace, int64_t workspaceBytes, void* output, Workspace* w)
{
    B200_REQUIRE(enc != nullptr, "encoder_forward: null encoder");
    B200_REQUIRE(B > 0 && total > 0 && maxSeqlen > 0 && maxSeqlen <= 512, "encoder_forward: bad sizes B=%d total=%d S=%d", B,
        total, maxSeqlen);
    B200_REQUIRE(maxSeqlen <= enc->cfg.max_positions, "encoder_forward: max_seqlen %d exceeds the position table (%d)",
        maxSeqlen, enc->cfg.max_positions);
    B200_REQUIRE(a && b && c && workspace && output, "encoder_forward: null pointer");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 1023u) == 0, "encoder_forward: workspace must be 1024-byte aligned");
    *w = carve(enc->cfg, total, B, workspace);
    B200_REQUIRE(w->bytes <= workspaceBytes, "encoder_forward: workspace too small (%lld < %lld)",
        static_cast<long long>(workspaceBytes), static_cast<long long>(w->bytes));
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_encoder_forward(bert_b200_encoder* enc, void* stream, int32_t B, int32_t total,
    int32_t max_seqlen, int32_t const* input_ids, int32_t const* segment_ids, int32_t const* cu_seqlens, void* workspace,
    int64_t workspace_bytes, void* output)
{
    Workspace w{};
    int32_t const st
        = checkForward(enc, B, total, max_seqlen, input_ids, segment_ids, cu_seqlens, workspace, workspace_bytes, output, &w);
    if (st != BERT_B200_OK)
        return st;
    return forwardImpl(enc, static_cast<cudaStream_t>(stream), B, total, max_seqlen, input_ids, segment_ids, cu_seqlens, w,
        output);
}

extern "C" int32_t bert_b200_encoder_forward_host(bert_b200_encoder* enc, void* stream, int32_t B, int32_t total,
    int32_t max_seqlen, int32_t const* input_ids_host, int32_t const* segment_ids_host, int32_t const* cu_seqlens_host,
    void* workspace, int64_t workspace_bytes, void* output_dev, void* output_host)
{
    Workspace w{};
    int32_t st = checkForward(enc, B, total, max_seqlen, input_ids_host, segment_ids_host, cu_seqlens_host, workspace,
        workspace_bytes, output_dev, &w);
    if (st != BERT_B200_OK)
        return st;
    B200_REQUIRE(output_host != nullptr, "encoder_forward_host: null output_host");
    auto s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(w.ids, input_ids_host, sizeof(int32_t) * total, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(w.seg, segment_ids_host, sizeof(int32_t) * total, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(w.cu, cu_seqlens_host, sizeof(int32_t) * (B + 1), cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward_host: H2D copy: %s", cudaGetErrorString(e));
    st = forwardImpl(enc, s, B, total, max_seqlen, w.ids, w.seg, w.cu, w, output_dev);
    if (st != BERT_B200_OK)
        return st;
    e = cudaMemcpyAsync(output_host, output_dev, sizeof(__half) * static_cast<size_t>(total) * enc->cfg.hidden_size,
        cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess)
        e = cudaStreamSynchronize(s);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward_host: D2H copy: %s", cudaGetErrorString(e));
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_encoder_forward_host_async(bert_b200_encoder* enc, void* stream, void* copy_stream,
    int32_t slot, int32_t B, int32_t total, int32_t max_seqlen, int32_t const* input_ids_host,
    int32_t const* segment_ids_host, int32_t const* cu_seqlens_host, void* workspace, int64_t workspace_bytes,
    void* output_dev, void* output_host)
{
    Workspace w{};
    int32_t st = checkForward(enc, B, total, max_seqlen, input_ids_host, segment_ids_host, cu_seqlens_host, workspace,
        workspace_bytes, output_dev, &w);
    if (st != BERT_B200_OK)
        return st;
    B200_REQUIRE(output_host != nullptr, "encoder_forward_host_async: null output_host");
    B200_REQUIRE(slot == 0 || slot == 1, "encoder_forward_host_async: slot %d (0 or 1)", slot);
    B200_REQUIRE(stream != copy_stream, "encoder_forward_host_async: the copy stream must differ from the compute stream");
    auto s = static_cast<cudaStream_t>(stream);
    auto cs = static_cast<cudaStream_t>(copy_stream);
    cudaError_t e = cudaSuccess;
    if (!enc->computeDone[slot])
    {
        e = cudaEventCreateWithFlags(&enc->computeDone[slot], cudaEventDisableTiming);
        if (e == cudaSuccess)
            e = cudaEventCreateWithFlags(&enc->copyDone[slot], cudaEventDisableTiming);
        if (e != cudaSuccess)
            B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward_host_async: event: %s", cudaGetErrorString(e));
    }
    // the previous copy out of this slot's device buffer must have finished before the encoder overwrites it
    if (enc->slotUsed[slot])
        e = cudaStreamWaitEvent(s, enc->copyDone[slot], 0);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(w.ids, input_ids_host, sizeof(int32_t) * total, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(w.seg, segment_ids_host, sizeof(int32_t) * total, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(w.cu, cu_seqlens_host, sizeof(int32_t) * (B + 1), cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward_host_async: H2D copy: %s", cudaGetErrorString(e));
    st = forwardImpl(enc, s, B, total, max_seqlen, w.ids, w.seg, w.cu, w, output_dev);
    if (st != BERT_B200_OK)
        return st;
    e = cudaEventRecord(enc->computeDone[slot], s);
    if (e == cudaSuccess)
        e = cudaStreamWaitEvent(cs, enc->computeDone[slot], 0);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(output_host, output_dev, sizeof(__half) * static_cast<size_t>(total) * enc->cfg.hidden_size,
            cudaMemcpyDeviceToHost, cs);
    if (e == cudaSuccess)
        e = cudaEventRecord(enc->copyDone[slot], cs);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward_host_async: D2H copy: %s", cudaGetErrorString(e));
    enc->slotUsed[slot] = true;
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_encoder_wait_host(bert_b200_encoder* enc, int32_t slot)
{
    B200_REQUIRE(enc != nullptr, "encoder_wait_host: null encoder");
    B200_REQUIRE(slot == 0 || slot == 1, "encoder_wait_host: slot %d (0 or 1)", slot);
    if (!enc->slotUsed[slot])
        return BERT_B200_OK;
    cudaError_t const e = cudaEventSynchronize(enc->copyDone[slot]);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_wait_host: %s", cudaGetErrorString(e));
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_encoder_enable_timing(bert_b200_encoder* enc, int32_t on)
{
    B200_REQUIRE(enc != nullptr, "encoder_enable_timing: null encoder");
    enc->timing = on != 0;
    enc->timedLaunches = 0;
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_encoder_read_timing(bert_b200_encoder* enc, float* ms, int32_t* launches)
{
    B200_REQUIRE(enc && ms && launches, "encoder_read_timing: null pointer");
    for (int32_t i = 0; i < enc->timedLaunches; ++i)
    {
        cudaError_t e = cudaEventSynchronize(enc->events[2 * i + 1]);
        float t = 0.f;
        if (e == cudaSuccess)
            e = cudaEventElapsedTime(&t, enc->events[2 * i], enc->events[2 * i + 1]);
        if (e != cudaSuccess)
            B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_read_timing: %s", cudaGetErrorString(e));
        int32_t const k = enc->kinds[i];
        ms[k] += t;
        launches[k] += 1;
    }
    return BERT_B200_OK;
}

extern "C" int32_t bert_b200_encoder_calibrate(bert_b200_encoder* enc, void* stream, int32_t B, int32_t total,
    int32_t max_seqlen, int32_t const* input_ids, int32_t const* segment_ids, int32_t const* cu_seqlens, void* workspace,
    int64_t workspace_bytes, void* output, float* amax_dev, float* amax_host)
{
    Workspace w{};
    int32_t st
        = checkForward(enc, B, total, max_seqlen, input_ids, segment_ids, cu_seqlens, workspace, workspace_bytes, output, &w);
    if (st != BERT_B200_OK)
        return st;
    B200_REQUIRE(enc->cfg.type_id == BERT_B200_FP16, "encoder_calibrate: needs the FP16 encoder");
    B200_REQUIRE(amax_dev && amax_host, "encoder_calibrate: null pointer");
    auto s = static_cast<cudaStream_t>(stream);
    size_t const bytes = sizeof(float) * 8 * static_cast<size_t>(enc->cfg.num_layers);
    if (cudaMemsetAsync(amax_dev, 0, bytes, s) != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_calibrate: memset failed");
    enc->amaxDev = amax_dev;
    st = forwardImpl(enc, s, B, total, max_seqlen, input_ids, segment_ids, cu_seqlens, w, output);
    enc->amaxDev = nullptr;
    if (st != BERT_B200_OK)
        return st;
    cudaError_t e = cudaMemcpyAsync(amax_host, amax_dev, bytes, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess)
        e = cudaStreamSynchronize(s);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_calibrate: %s", cudaGetErrorString(e));
    return BERT_B200_OK;
}

// ------------------------------------------------------------------------------------------------
// Forward pass that needs no caller-provided scratch memory
// ------------------------------------------------------------------------------------------------
namespace
{
// Scratch for bert_b200_encoder_forward_static. It is part of the library image: every GPU that loads the
// library reserves these bytes until the process exits, whether the entry point is used or not.
constexpr int64_t kStaticWorkspaceBytes = BERT_B200_STATIC_WORKSPACE_BYTES;
static __device__ __align__(256) uint8_t gStaticWorkspace[kStaticWorkspaceBytes + 1024];

// In host code `gStaticWorkspace` is only a handle for the symbol, not a device address: the address the kernels
// can use has to be asked from the runtime, once per device, with that device current.
int32_t staticWorkspace(void** out)
{
    static std::mutex mtx;
    static void* perDevice[64] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64)
        B200_FAIL(BERT_B200_NOT_SUPPORTED, "encoder_forward_static: device ordinal %d is outside the 64 this entry point keeps an address for", dev);
    std::lock_guard<std::mutex> lock(mtx);
    if (!perDevice[dev])
    {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, gStaticWorkspace);
        if (e != cudaSuccess || p == nullptr)
            B200_FAIL(BERT_B200_CUDA_ERROR, "encoder_forward_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        // the layer loop wants 1024-byte alignment; the array carries 1 KiB of slack for rounding up
        perDevice[dev] = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
    }
    *out = perDevice[dev];
    return BERT_B200_OK;
}
} // namespace

extern "C" int64_t bert_b200_encoder_static_workspace_limit(void)
{
    return kStaticWorkspaceBytes;
}

extern "C" int32_t bert_b200_encoder_forward_static(bert_b200_encoder* enc, void* stream, int32_t B, int32_t total,
    int32_t max_seqlen, int32_t const* input_ids, int32_t const* segment_ids, int32_t const* cu_seqlens, void* output)
{
    B200_REQUIRE(enc != nullptr, "encoder_forward_static: null encoder");
    B200_REQUIRE(!enc->timing, "encoder_forward_static: per-kernel timing creates CUDA events; disable it for this entry point");
    B200_REQUIRE(B > 0 && total > 0, "encoder_forward_static: bad sizes B=%d total=%d", B, total);
    int64_t const need = carve(enc->cfg, total, B, nullptr).bytes;
    if (need > kStaticWorkspaceBytes)
        B200_FAIL(BERT_B200_NOT_SUPPORTED,
            "encoder_forward_static: %d tokens / %d sequences need %lld bytes of scratch, the built-in buffer holds %lld; "
            "use bert_b200_encoder_forward with a caller-allocated workspace",
            total, B, static_cast<long long>(need), static_cast<long long>(kStaticWorkspaceBytes));
    void* ws = nullptr;
    int32_t st = staticWorkspace(&ws);
    if (st != BERT_B200_OK)
        return st;
    Workspace w{};
    st = checkForward(enc, B, total, max_seqlen, input_ids, segment_ids, cu_seqlens, ws, kStaticWorkspaceBytes, output, &w);
    if (st != BERT_B200_OK)
        return st;
    // Every buffer carved from the scratch is written before it is read in one forward; the only word that has
    // to start from zero, the device-wait status word, is cleared by forwardImpl.
    return forwardImpl(enc, static_cast<cudaStream_t>(stream), B, total, max_seqlen, input_ids, segment_ids, cu_seqlens, w,
        output);
}

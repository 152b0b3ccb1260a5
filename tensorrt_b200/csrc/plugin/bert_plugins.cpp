// IPluginV3 adapters for the four BERT encoder plugins, same creator names / versions / PluginFields as the
// reference library:
//   CustomEmbLayerNormPluginDynamic   "4" (packed, HFace), "5" (packed + pre-LN output, MTron), "6" (fixed + mask)
//       ref: plugin/embLayerNormPlugin/embLayerNormVarSeqlenPlugin.cpp, embLayerNormPlugin.cpp
//   CustomQKVToContextPluginDynamic   "4" (fixed), "5" (var-seqlen), "6" (INT8 CHW32-interleaved)
//       ref: plugin/bertQKVToContextPlugin/qkvToContextPlugin.cpp, qkvToContextInt8InterleavedPlugin.cpp
//   CustomSkipLayerNormPluginDynamic  "5" (fixed), "6" (any rank), "7" / "8" (INT8 CHW32-interleaved HFace / MTron)
//       ref: plugin/skipLayerNormPlugin/skipLayerNormPlugin.cpp, skipLayerNormInt8InterleavedPlugin.cpp
//   CustomFCPluginDynamic             "2"  the fields of the reference's version 1 (plugin/fcPlugin/fcPlugin.cpp, an
//       IPluginV2DynamicExt) on the V3 interfaces, plus optional bias / activation / INT8 extension fields. Version 1
//       itself, with the reference's interface kind and serialisation buffer, is the adapter in legacy_plugins.cpp.
// Every enqueue() only translates descriptors into C-ABI calls (include/bert_b200.h).
#include "plugin_common.h"

#include <dlfcn.h>

#include <cmath>
#include <cstdio>
#include <mutex>

namespace bert_b200_plugin
{

// ------------------------------------------------------------------------------------------------
// logging / errors
// ------------------------------------------------------------------------------------------------
namespace
{
std::mutex gLogMutex;
ILogger* gLogger = nullptr;
ILoggerFinder* gLoggerFinder = nullptr;
} // namespace

void setLogger(ILogger* logger)
{
    std::lock_guard<std::mutex> lock(gLogMutex);
    gLogger = logger;
}

void logMessage(ILogger::Severity severity, char const* fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    std::lock_guard<std::mutex> lock(gLogMutex);
    if (!gLogger && gLoggerFinder)
        gLogger = gLoggerFinder->findLogger();
    if (gLogger)
        gLogger->log(severity, buf);
    else if (severity <= ILogger::Severity::kWARNING)
        fprintf(stderr, "[bert_b200_plugin] %s\n", buf);
}

void caughtError(std::exception const& e)
{
    logMessage(ILogger::Severity::kERROR, "%s", e.what());
}

static int32_t abiStatus(int32_t st, char const* what)
{
    if (st != BERT_B200_OK)
        logMessage(ILogger::Severity::kERROR, "%s: %s", what, bert_b200_last_error());
    return st;
}

// ------------------------------------------------------------------------------------------------
// weights
// ------------------------------------------------------------------------------------------------
void HostWeights::assign(void const* src, DataType srcType, int64_t n, DataType dst)
{
    PLG_VALIDATE(src != nullptr && n > 0);
    PLG_VALIDATE(srcType == DataType::kFLOAT || srcType == DataType::kHALF);
    PLG_VALIDATE(dst == DataType::kFLOAT || dst == DataType::kHALF);
    type = dst;
    count = n;
    size_t const elem = dst == DataType::kHALF ? 2 : 4;
    bytes.resize(static_cast<size_t>(n) * elem);
    if (srcType == dst)
    {
        std::memcpy(bytes.data(), src, bytes.size());
    }
    else if (dst == DataType::kHALF)
    {
        auto const* s = static_cast<float const*>(src);
        auto* d = reinterpret_cast<__half*>(bytes.data());
        for (int64_t i = 0; i < n; ++i)
            d[i] = __float2half(s[i]);
    }
    else
    {
        auto const* s = static_cast<__half const*>(src);
        auto* d = reinterpret_cast<float*>(bytes.data());
        for (int64_t i = 0; i < n; ++i)
            d[i] = __half2float(s[i]);
    }
}

void HostWeights::assign(PluginField const& f, DataType dst)
{
    PLG_VALIDATE(f.type == PluginFieldType::kFLOAT32 || f.type == PluginFieldType::kFLOAT16);
    assign(f.data, f.type == PluginFieldType::kFLOAT16 ? DataType::kHALF : DataType::kFLOAT, f.length, dst);
}

float HostWeights::at(int64_t i) const
{
    return type == DataType::kHALF ? __half2float(reinterpret_cast<__half const*>(bytes.data())[i])
                                   : reinterpret_cast<float const*>(bytes.data())[i];
}

DeviceBuffer::~DeviceBuffer()
{
    if (ptr)
        cudaFree(ptr);
}

bool DeviceBuffer::upload(void const* host, size_t n)
{
    if (ptr)
    {
        cudaFree(ptr);
        ptr = nullptr;
    }
    if (cudaMalloc(&ptr, n) != cudaSuccess)
    {
        ptr = nullptr;
        (void) cudaGetLastError(); // no usable device (host-only build / test phase): enqueue will refuse to run
        return false;
    }
    if (cudaMemcpy(ptr, host, n, cudaMemcpyHostToDevice) != cudaSuccess)
    {
        cudaFree(ptr);
        ptr = nullptr;
        (void) cudaGetLastError();
        return false;
    }
    return true;
}

// ------------------------------------------------------------------------------------------------
// PluginBase / CreatorBase
// ------------------------------------------------------------------------------------------------
IPluginCapability* PluginBase::getCapabilityInterface(PluginCapabilityType type) noexcept
{
    if (type == PluginCapabilityType::kBUILD)
        return static_cast<IPluginV3OneBuild*>(this);
    if (type == PluginCapabilityType::kRUNTIME)
        return static_cast<IPluginV3OneRuntime*>(this);
    return static_cast<IPluginV3OneCore*>(this);
}

PluginFieldCollection const* PluginBase::getFieldsToSerialize() noexcept
{
    try
    {
        mFields.clear();
        serialize(mFields);
        mFC.nbFields = static_cast<int32_t>(mFields.size());
        mFC.fields = mFields.data();
        return &mFC;
    }
    catch (std::exception const& e)
    {
        caughtError(e);
    }
    return nullptr;
}

IPluginV3* CreatorBase::createPlugin(AsciiChar const* name, PluginFieldCollection const* fc, TensorRTPhase phase) noexcept
{
    try
    {
        PLG_VALIDATE(fc != nullptr);
        PluginBase* p = make(name ? name : "", *fc, phase);
        if (p)
            p->setPluginNamespace(mNamespace.c_str());
        return p;
    }
    catch (std::exception const& e)
    {
        caughtError(e);
    }
    return nullptr;
}

namespace
{

constexpr char const* kEmbName = "CustomEmbLayerNormPluginDynamic";
constexpr char const* kQkvName = "CustomQKVToContextPluginDynamic";
constexpr char const* kSkipName = "CustomSkipLayerNormPluginDynamic";
constexpr char const* kFcName = "CustomFCPluginDynamic";

inline int32_t typeId(DataType t)
{
    return static_cast<int32_t>(t);
}

// INT8 tensors of these plugins have H = W = 1, so CHW32 / CHW4 equal the linear layout
// (ref: plugin/skipLayerNormPlugin/skipLayerNormPlugin.cpp:143-159, qkvToContextPlugin.cpp:233-243).
inline TensorFormat int8Format(int64_t channels)
{
    return channels % 32 == 0 ? TensorFormat::kCHW32 : TensorFormat::kCHW4;
}

// ================================================================================================
// EmbLayerNorm: shared weights
// ================================================================================================
struct EmbWeights
{
    DataType type{DataType::kFLOAT}; // output / table type
    HostWeights beta, gamma, word, pos, tok;
    DeviceBuffer dBeta, dGamma, dWord, dPos, dTok;
    int32_t ld{0}, wordVocab{0}, posVocab{0}, tokVocab{0};

    // ref: plugin/embLayerNormPlugin/embLayerNormPlugin.cpp:49-73 (constructor)
    void init(PluginFieldCollection const& fc, bool outputFp16)
    {
        requireFields(fc,
            {"bert_embeddings_layernorm_beta", "bert_embeddings_layernorm_gamma", "bert_embeddings_word_embeddings",
                "bert_embeddings_token_type_embeddings", "bert_embeddings_position_embeddings"});
        type = outputFp16 ? DataType::kHALF : DataType::kFLOAT;
        beta.assign(*findField(fc, "bert_embeddings_layernorm_beta"), DataType::kFLOAT);
        gamma.assign(*findField(fc, "bert_embeddings_layernorm_gamma"), DataType::kFLOAT);
        word.assign(*findField(fc, "bert_embeddings_word_embeddings"), type);
        tok.assign(*findField(fc, "bert_embeddings_token_type_embeddings"), type);
        pos.assign(*findField(fc, "bert_embeddings_position_embeddings"), type);
        finish();
    }
    void copyFrom(EmbWeights const& o)
    {
        type = o.type;
        beta = o.beta;
        gamma = o.gamma;
        word = o.word;
        pos = o.pos;
        tok = o.tok;
        finish();
    }
    void finish()
    {
        ld = static_cast<int32_t>(beta.count);
        PLG_VALIDATE(ld > 0 && gamma.count == ld);
        PLG_VALIDATE(word.count % ld == 0 && pos.count % ld == 0 && tok.count % ld == 0);
        wordVocab = static_cast<int32_t>(word.count / ld);
        posVocab = static_cast<int32_t>(pos.count / ld);
        tokVocab = static_cast<int32_t>(tok.count / ld);
        dBeta.upload(beta.data(), beta.sizeBytes());
        dGamma.upload(gamma.data(), gamma.sizeBytes());
        dWord.upload(word.data(), word.sizeBytes());
        dPos.upload(pos.data(), pos.sizeBytes());
        dTok.upload(tok.data(), tok.sizeBytes());
    }
    bool onDevice() const
    {
        return dBeta.ptr && dGamma.ptr && dWord.ptr && dPos.ptr && dTok.ptr;
    }
    void serialize(std::vector<PluginField>& f) const
    {
        f.emplace_back("bert_embeddings_layernorm_beta", beta.data(), PluginFieldType::kFLOAT32, static_cast<int32_t>(beta.count));
        f.emplace_back("bert_embeddings_layernorm_gamma", gamma.data(), PluginFieldType::kFLOAT32, static_cast<int32_t>(gamma.count));
        f.emplace_back("bert_embeddings_word_embeddings", word.data(), word.fieldType(), static_cast<int32_t>(word.count));
        f.emplace_back("bert_embeddings_token_type_embeddings", tok.data(), tok.fieldType(), static_cast<int32_t>(tok.count));
        f.emplace_back("bert_embeddings_position_embeddings", pos.data(), pos.fieldType(), static_cast<int32_t>(pos.count));
    }
};

// ================================================================================================
// CustomEmbLayerNormPluginDynamic version 6: fixed length, emits the packed mask or the mask index
// ref: plugin/embLayerNormPlugin/embLayerNormPlugin.cpp
// ================================================================================================
class EmbLayerNormFixed : public PluginBase
{
public:
    EmbLayerNormFixed(std::string const& name)
        : PluginBase(name, kEmbName, "6")
    {
    }
    EmbWeights w;
    int32_t outputFp16{0};
    int32_t fullMask{0};
    int32_t mhaTypeId{0};

    IPluginV3* clone() noexcept override
    {
        try
        {
            auto p = std::make_unique<EmbLayerNormFixed>(mLayerName);
            p->outputFp16 = outputFp16;
            p->fullMask = fullMask;
            p->mhaTypeId = mhaTypeId;
            p->w.copyFrom(w);
            p->setPluginNamespace(mNamespace.c_str());
            return p.release();
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    int32_t getNbOutputs() const noexcept override
    {
        return 2;
    }
    bool supportsFormatCombination(int32_t pos, DynamicPluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs) noexcept override
    {
        if (!inOut || nbInputs != 3 || nbOutputs != 2 || pos < 0 || pos >= 5)
            return false;
        PluginTensorDesc const& d = inOut[pos].desc;
        if (d.format != TensorFormat::kLINEAR)
            return false;
        if (pos == 0)
            return d.type == DataType::kINT32 && d.dims.nbDims == 2;
        PluginTensorDesc const& prev = inOut[pos - 1].desc;
        if (pos == 1 || pos == 2)
            return d.type == DataType::kINT32 && d.dims.nbDims == 2 && d.dims.d[BDIM] == prev.dims.d[BDIM]
                && d.dims.d[SDIM] == prev.dims.d[SDIM];
        if (pos == 3)
            return d.type == w.type && d.dims.nbDims == 5 && d.dims.d[BDIM] == prev.dims.d[BDIM]
                && d.dims.d[SDIM] == prev.dims.d[SDIM] && d.dims.d[3] == 1 && d.dims.d[4] == 1;
        return d.type == DataType::kINT32;
    }
    int32_t getOutputShapes(DimsExprs const* inputs, int32_t nbInputs, DimsExprs const*, int32_t, DimsExprs* outputs,
        int32_t nbOutputs, IExprBuilder& eb) noexcept override
    {
        try
        {
            PLG_VALIDATE(inputs && outputs && nbInputs == 3 && nbOutputs == 2);
            PLG_VALIDATE(inputs[0].nbDims == 2 && inputs[1].nbDims == 2 && inputs[2].nbDims == 2);
            outputs[0].nbDims = 5;
            outputs[0].d[0] = inputs[0].d[0];
            outputs[0].d[1] = inputs[0].d[1];
            outputs[0].d[2] = eb.constant(w.ld);
            outputs[0].d[3] = eb.constant(1);
            outputs[0].d[4] = eb.constant(1);
            outputs[1].nbDims = 2;
            outputs[1].d[0] = inputs[0].d[BDIM];
            auto const* one = eb.constant(kUnfusedMaskSize);
            DataType const mhaType = static_cast<DataType>(mhaTypeId);
            bool const precisionOk = mhaType == DataType::kHALF || mhaType == DataType::kINT8;
            if (fullMask || precisionOk)
            {
                // size = 512 for S in {64, 96, 128}, 6144 for S = 384, else 1 - written as an expression of S
                // (ref: embLayerNormPlugin.cpp:414-451)
                auto const& S = *inputs[0].d[SDIM];
                auto sel = [&](int64_t s, int64_t size) {
                    return eb.operation(DimensionOperation::kPROD,
                        *eb.operation(DimensionOperation::kEQUAL, S, *eb.constant(s)), *eb.constant(size));
                };
                auto const* sum = eb.operation(DimensionOperation::kSUM, *sel(384, kPackedMaskSize384), *sel(128, kPackedMaskSize128));
                auto const* sum2 = eb.operation(DimensionOperation::kSUM, *sel(64, kPackedMaskSize128), *sel(96, kPackedMaskSize128));
                sum = eb.operation(DimensionOperation::kSUM, *sum, *sum2);
                auto const* isZero = eb.operation(DimensionOperation::kEQUAL, *sum, *eb.constant(0));
                outputs[1].d[1] = eb.operation(
                    DimensionOperation::kSUM, *sum, *eb.operation(DimensionOperation::kPROD, *isZero, *one));
            }
            else
            {
                outputs[1].d[1] = one;
            }
            return STATUS_SUCCESS;
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }
    int32_t getOutputDataTypes(DataType* out, int32_t nbOutputs, DataType const*, int32_t nbInputs) const noexcept override
    {
        if (!out || nbOutputs != 2 || nbInputs != 3)
            return STATUS_FAILURE;
        out[0] = w.type;
        out[1] = DataType::kINT32;
        return STATUS_SUCCESS;
    }
    int32_t enqueue(PluginTensorDesc const* inDesc, PluginTensorDesc const*, void const* const* inputs, void* const* outputs,
        void*, cudaStream_t stream) noexcept override
    {
        try
        {
            PLG_VALIDATE(inDesc && inputs && outputs);
            PLG_VALIDATE(w.onDevice());
            int32_t const B = static_cast<int32_t>(inDesc[0].dims.d[BDIM]);
            int32_t const S = static_cast<int32_t>(inDesc[0].dims.d[SDIM]);
            auto const* mask = static_cast<int32_t const*>(inputs[2]);
            uint32_t wm = 0, wn = 0;
            bool const packed = (fullMask || mhaMaskPackedSize(static_cast<DataType>(mhaTypeId), S) != kUnfusedMaskSize)
                && packedMaskWarps(S, wm, wn);
            // the mask index comes out of the embedding launch itself; only the packed fused-attention mask is a second kernel
            int32_t const st = abiStatus(
                bert_b200_emb_layer_norm_mask_idx(stream, typeId(w.type), w.ld, B, S, static_cast<int32_t const*>(inputs[0]),
                    static_cast<int32_t const*>(inputs[1]), static_cast<float const*>(w.dBeta.ptr),
                    static_cast<float const*>(w.dGamma.ptr), w.dWord.ptr, w.dPos.ptr, w.dTok.ptr, w.wordVocab, w.tokVocab,
                    w.posVocab, outputs[0], nullptr, 0.f, packed ? nullptr : mask,
                    packed ? nullptr : static_cast<int32_t*>(outputs[1])),
                "emb_layer_norm");
            if (st != BERT_B200_OK || !packed)
                return st;
            return abiStatus(bert_b200_convert_mask(S, B, wm, wn, 1, mask, static_cast<uint32_t*>(outputs[1]), stream),
                "convert_mask");
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }

protected:
    void serialize(std::vector<PluginField>& f) override
    {
        f.emplace_back("output_fp16", &outputFp16, PluginFieldType::kINT32, 1);
        f.emplace_back("full_mask", &fullMask, PluginFieldType::kINT32, 1);
        f.emplace_back("mha_type_id", &mhaTypeId, PluginFieldType::kINT32, 1);
        w.serialize(f);
    }
};

class EmbLayerNormFixedCreator : public CreatorBase
{
public:
    EmbLayerNormFixedCreator()
        : CreatorBase(kEmbName, "6",
            {PluginField("bert_embeddings_layernorm_beta"), PluginField("bert_embeddings_layernorm_gamma"),
                PluginField("bert_embeddings_word_embeddings"), PluginField("bert_embeddings_token_type_embeddings"),
                PluginField("bert_embeddings_position_embeddings"), PluginField("output_fp16"), PluginField("full_mask"),
                PluginField("mha_type_id")})
    {
    }
    PluginBase* make(char const* name, PluginFieldCollection const& fc, TensorRTPhase) override
    {
        auto p = std::make_unique<EmbLayerNormFixed>(name);
        getInt(fc, "output_fp16", p->outputFp16);
        p->outputFp16 = p->outputFp16 != 0;
        getInt(fc, "full_mask", p->fullMask);
        p->fullMask = p->fullMask != 0;
        getInt(fc, "mha_type_id", p->mhaTypeId);
        PLG_VALIDATE(p->mhaTypeId >= 0 && p->mhaTypeId <= 3);
        p->w.init(fc, p->outputFp16 != 0);
        return p.release();
    }
};

// ================================================================================================
// CustomEmbLayerNormPluginDynamic versions 4 (HFace) and 5 (MTron): packed variable-length input
// ref: plugin/embLayerNormPlugin/embLayerNormVarSeqlenPlugin.cpp
// ================================================================================================
class EmbLayerNormVarSeqlen : public PluginBase
{
public:
    EmbLayerNormVarSeqlen(std::string const& name, bool mtron)
        : PluginBase(name, kEmbName, mtron ? "5" : "4")
        , mtron(mtron)
    {
    }
    EmbWeights w;
    bool mtron;

    DataType maskType() const
    {
        return mtron ? w.type : DataType::kINT32;
    }
    IPluginV3* clone() noexcept override
    {
        try
        {
            auto p = std::make_unique<EmbLayerNormVarSeqlen>(mLayerName, mtron);
            p->w.copyFrom(w);
            p->setPluginNamespace(mNamespace.c_str());
            return p.release();
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    int32_t getNbOutputs() const noexcept override
    {
        return 2;
    }
    bool supportsFormatCombination(int32_t pos, DynamicPluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs) noexcept override
    {
        if (!inOut || nbInputs != 4 || nbOutputs != 2 || pos < 0 || pos >= 6)
            return false;
        PluginTensorDesc const& d = inOut[pos].desc;
        if (d.format != TensorFormat::kLINEAR)
            return false;
        if (pos == 0 || pos == 2) // input_ids, cu_seqlens
            return d.type == DataType::kINT32 && d.dims.nbDims == 1;
        if (pos == 1) // segment ids
            return d.type == DataType::kINT32 && d.dims.nbDims == 1 && d.dims.d[0] == inOut[0].desc.dims.d[0];
        if (pos == 3) // dummy tensor whose length is the maximum sequence length
            return d.dims.nbDims == 1;
        if (pos == 4)
            return d.type == w.type && d.dims.nbDims == 4 && d.dims.d[0] == inOut[0].desc.dims.d[0] && d.dims.d[2] == 1
                && d.dims.d[3] == 1;
        return d.type == maskType();
    }
    int32_t getOutputShapes(DimsExprs const* inputs, int32_t nbInputs, DimsExprs const*, int32_t, DimsExprs* outputs,
        int32_t nbOutputs, IExprBuilder& eb) noexcept override
    {
        try
        {
            PLG_VALIDATE(inputs && outputs && nbInputs == 4 && nbOutputs == 2);
            PLG_VALIDATE(inputs[0].nbDims == 1 && inputs[1].nbDims == 1 && inputs[2].nbDims == 1);
            outputs[0].nbDims = 4;
            outputs[0].d[0] = inputs[0].d[0];
            outputs[0].d[1] = eb.constant(w.ld);
            outputs[0].d[2] = eb.constant(1);
            outputs[0].d[3] = eb.constant(1);
            if (mtron)
                outputs[1] = outputs[0]; // pre-LayerNorm sum
            else
                outputs[1].nbDims = 0; // empty placeholder where version 6 has the mask
            return STATUS_SUCCESS;
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }
    int32_t getOutputDataTypes(DataType* out, int32_t nbOutputs, DataType const*, int32_t) const noexcept override
    {
        if (!out || nbOutputs != 2)
            return STATUS_FAILURE;
        out[0] = w.type;
        out[1] = maskType();
        return STATUS_SUCCESS;
    }
    int32_t enqueue(PluginTensorDesc const* inDesc, PluginTensorDesc const*, void const* const* inputs, void* const* outputs,
        void*, cudaStream_t stream) noexcept override
    {
        try
        {
            PLG_VALIDATE(inDesc && inputs && outputs);
            PLG_VALIDATE(w.onDevice());
            int32_t const total = static_cast<int32_t>(inDesc[0].dims.d[0]);
            int32_t const B = static_cast<int32_t>(inDesc[2].dims.d[0]) - 1;
            int32_t const maxS = static_cast<int32_t>(inDesc[3].dims.d[0]);
            PLG_VALIDATE(B >= 0);
            return abiStatus(bert_b200_emb_layer_norm_var_seqlen(stream, typeId(w.type), w.ld, B, maxS, total,
                                 static_cast<int32_t const*>(inputs[0]), static_cast<int32_t const*>(inputs[1]),
                                 static_cast<int32_t const*>(inputs[2]), static_cast<float const*>(w.dBeta.ptr),
                                 static_cast<float const*>(w.dGamma.ptr), w.dWord.ptr, w.dPos.ptr, w.dTok.ptr, w.wordVocab,
                                 w.tokVocab, w.posVocab, outputs[0], mtron ? outputs[1] : nullptr, nullptr, 0.f),
                "emb_layer_norm_var_seqlen");
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }

protected:
    int32_t mOutputFp16{0};
    void serialize(std::vector<PluginField>& f) override
    {
        mOutputFp16 = w.type == DataType::kHALF;
        f.emplace_back("output_fp16", &mOutputFp16, PluginFieldType::kINT32, 1);
        w.serialize(f);
    }
};

class EmbLayerNormVarSeqlenCreator : public CreatorBase
{
public:
    explicit EmbLayerNormVarSeqlenCreator(bool mtron)
        : CreatorBase(kEmbName, mtron ? "5" : "4",
            {PluginField("bert_embeddings_layernorm_beta"), PluginField("bert_embeddings_layernorm_gamma"),
                PluginField("bert_embeddings_word_embeddings"), PluginField("bert_embeddings_token_type_embeddings"),
                PluginField("bert_embeddings_position_embeddings"), PluginField("output_fp16")})
        , mMtron(mtron)
    {
    }
    PluginBase* make(char const* name, PluginFieldCollection const& fc, TensorRTPhase) override
    {
        auto p = std::make_unique<EmbLayerNormVarSeqlen>(name, mMtron);
        int32_t fp16 = 0;
        getInt(fc, "output_fp16", fp16);
        p->w.init(fc, fp16 != 0);
        return p.release();
    }

private:
    bool mMtron;
};

// ================================================================================================
// CustomQKVToContextPluginDynamic versions 4 / 5 / 6
// ================================================================================================
enum class QkvKind
{
    kFixed,      // version 4
    kVarSeqlen,  // version 5
    kInterleaved // version 6
};

class QkvToContext : public PluginBase
{
public:
    QkvToContext(std::string const& name, QkvKind kind)
        : PluginBase(name, kQkvName, kind == QkvKind::kFixed ? "4" : (kind == QkvKind::kVarSeqlen ? "5" : "6"))
        , kind(kind)
    {
    }
    QkvKind kind;
    int32_t type{1}; // nvinfer1::DataType as int32 (serialised as such)
    int32_t hiddenSize{0}, numHeads{0}, headSize{0};
    int32_t hasMask{0}, varSeqlen{0}, useInt8ScaleMax{1}, useExplicitInt8{0};
    float dqProbs{-1.f}, qkvScale{1.f}, ctxScale{1.f};
    int32_t S{0}, B{0}, sm{100}, hasUnfusedDispatcher{0};

    DataType dtype() const
    {
        return static_cast<DataType>(type);
    }
    int32_t hdim() const
    {
        return kind == QkvKind::kVarSeqlen && varSeqlen ? 1 : HDIM;
    }
    int32_t nbInputsExpected() const
    {
        if (kind == QkvKind::kInterleaved)
            return 3;
        if (kind == QkvKind::kVarSeqlen)
            return 1 + hasMask + 2 * varSeqlen;
        return 1 + hasMask;
    }
    void finish()
    {
        PLG_VALIDATE(hiddenSize > 0 && numHeads > 0 && hiddenSize % numHeads == 0);
        headSize = hiddenSize / numHeads;
        if (kind == QkvKind::kInterleaved)
            type = typeId(DataType::kINT8);
        PLG_VALIDATE(dtype() == DataType::kFLOAT || dtype() == DataType::kHALF || dtype() == DataType::kINT8);
        if (dtype() == DataType::kINT8 && dqProbs < 0)
            dqProbs = 1.f / 127.f; // ref: qkvToContextPlugin.cpp:715-719
        if (dtype() == DataType::kINT8) // FP16 outside these shapes takes the SIMT kernel
            PLG_VALIDATE(headSize <= 64 && headSize % (kind == QkvKind::kInterleaved ? 32 : 16) == 0
                && "INT8 attention takes head sizes 16, 32, 48, 64 (32, 64 interleaved)");
        if (kind == QkvKind::kVarSeqlen && varSeqlen)
            PLG_VALIDATE(dtype() != DataType::kFLOAT && hasMask); // ref: qkvToContextPlugin.cpp:877-881
    }
    IPluginV3* clone() noexcept override
    {
        try
        {
            auto p = std::make_unique<QkvToContext>(mLayerName, kind);
            p->type = type;
            p->hiddenSize = hiddenSize;
            p->numHeads = numHeads;
            p->headSize = headSize;
            p->hasMask = hasMask;
            p->varSeqlen = varSeqlen;
            p->useInt8ScaleMax = useInt8ScaleMax;
            p->useExplicitInt8 = useExplicitInt8;
            p->dqProbs = dqProbs;
            p->qkvScale = qkvScale;
            p->ctxScale = ctxScale;
            p->S = S;
            p->B = B;
            p->sm = sm;
            p->hasUnfusedDispatcher = hasUnfusedDispatcher;
            p->setPluginNamespace(mNamespace.c_str());
            return p.release();
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    int32_t getNbOutputs() const noexcept override
    {
        return 1;
    }
    bool supportsFormatCombination(int32_t pos, DynamicPluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs) noexcept override
    {
        if (!inOut || nbInputs != nbInputsExpected() || nbOutputs != 1 || pos < 0 || pos > nbInputs)
            return false;
        PluginTensorDesc const& d = inOut[pos].desc;
        PluginTensorDesc const& in = inOut[0].desc;
        PluginTensorDesc const& out = inOut[nbInputs].desc;
        if (kind == QkvKind::kInterleaved)
        {
            // ref: qkvToContextInt8InterleavedPlugin.cpp:131-170: qkv [1, 3E, total, 1] CHW32, cu_seqlens, dummy
            if (pos == 0 || pos == nbInputs)
                return d.type == DataType::kINT8 && d.format == TensorFormat::kCHW32 && d.dims.nbDims == 4 && d.dims.d[0] == 1
                    && d.dims.d[3] == 1 && d.dims.d[1] == (pos == 0 ? 3 : 1) * static_cast<int64_t>(hiddenSize);
            if (pos == 1)
                return d.type == DataType::kINT32 && d.format == TensorFormat::kLINEAR && d.dims.nbDims == 1;
            return d.dims.nbDims == 1;
        }
        int32_t const h = hdim();
        bool const packed = kind == QkvKind::kVarSeqlen && varSeqlen;
        if (pos == 0 || pos == nbInputs)
        {
            TensorFormat fmt = TensorFormat::kLINEAR;
            if (dtype() == DataType::kINT8)
                fmt = int8Format(in.dims.d[h]);
            int32_t const rank = packed ? 4 : 5;
            if (d.type != dtype() || d.format != fmt || d.dims.nbDims != rank || d.dims.d[h + 1] != 1 || d.dims.d[h + 2] != 1)
                return false;
            if (pos == 0)
                return in.dims.d[h] % 3 == 0;
            if (in.dims.d[h] / 3 != out.dims.d[h])
                return false;
            if (!packed)
                return out.dims.d[BDIM] == in.dims.d[BDIM] && out.dims.d[SDIM] == in.dims.d[SDIM];
            return true;
        }
        if (pos == 1)
        {
            if (packed)
                return true; // dummy mask input
            if (d.type != DataType::kINT32 || d.format != TensorFormat::kLINEAR)
                return false;
            if (kind == QkvKind::kFixed) // [B, packed size] or [B, 1] (ref: qkvToContextPlugin.cpp:259-277)
                return d.dims.nbDims == 2 && d.dims.d[0] == in.dims.d[BDIM];
            return d.dims.nbDims == 1; // version 5 without var_seqlen: maskIdx[B]
        }
        if (pos == 2)
            return d.type == DataType::kINT32 && d.format == TensorFormat::kLINEAR;
        return d.dims.nbDims == 1;
    }
    int32_t getOutputShapes(DimsExprs const* inputs, int32_t nbInputs, DimsExprs const*, int32_t, DimsExprs* outputs,
        int32_t nbOutputs, IExprBuilder& eb) noexcept override
    {
        try
        {
            PLG_VALIDATE(inputs && outputs && nbInputs == nbInputsExpected() && nbOutputs == 1);
            outputs[0] = inputs[0];
            int32_t const h = kind == QkvKind::kInterleaved ? 1 : hdim();
            outputs[0].d[h] = eb.operation(DimensionOperation::kFLOOR_DIV, *inputs[0].d[h], *eb.constant(3));
            return STATUS_SUCCESS;
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }
    int32_t getOutputDataTypes(DataType* out, int32_t nbOutputs, DataType const*, int32_t) const noexcept override
    {
        if (!out || nbOutputs != 1)
            return STATUS_FAILURE;
        out[0] = dtype();
        return STATUS_SUCCESS;
    }
    int32_t configurePlugin(DynamicPluginTensorDesc const* in, int32_t nbInputs, DynamicPluginTensorDesc const*, int32_t) noexcept override
    {
        if (in && nbInputs >= 1 && kind != QkvKind::kInterleaved && !(kind == QkvKind::kVarSeqlen && varSeqlen))
        {
            S = static_cast<int32_t>(in[0].max.d[SDIM]);
            B = static_cast<int32_t>(in[0].max.d[BDIM]);
        }
        return STATUS_SUCCESS;
    }
    int32_t onShapeChange(PluginTensorDesc const* in, int32_t nbInputs, PluginTensorDesc const*, int32_t) noexcept override
    {
        if (in && nbInputs >= 1 && kind != QkvKind::kInterleaved && !(kind == QkvKind::kVarSeqlen && varSeqlen))
        {
            S = static_cast<int32_t>(in[0].dims.d[SDIM]);
            B = static_cast<int32_t>(in[0].dims.d[BDIM]);
        }
        return STATUS_SUCCESS;
    }
    // Workspace of the fixed-length versions: the lengths recovered from a packed mask. (The reference's unfused runner
    // also keeps its score matrix there, qkvToContextPlugin.cpp:430-438; these kernels need no scratch memory.)
    static int64_t maskBytes(int64_t b)
    {
        return (b * 4 + 255) / 256 * 256;
    }
    size_t getWorkspaceSize(DynamicPluginTensorDesc const* in, int32_t nbInputs, DynamicPluginTensorDesc const*, int32_t) const noexcept override
    {
        if (kind != QkvKind::kFixed || !in || nbInputs < 1)
            return 0;
        int64_t const b = in[0].max.d[BDIM] > 0 ? in[0].max.d[BDIM] : 1;
        return static_cast<size_t>(hasMask ? maskBytes(b) : 0);
    }
    int32_t enqueue(PluginTensorDesc const* inDesc, PluginTensorDesc const* outDesc, void const* const* inputs,
        void* const* outputs, void* workspace, cudaStream_t stream) noexcept override
    {
        try
        {
            PLG_VALIDATE(inDesc && outDesc && inputs && outputs);
            bert_b200_mha_params p{};
            p.type_id = type;
            p.num_heads = numHeads;
            p.head_size = headSize;
            p.qkv = inputs[0];
            p.out = outputs[0];
            float const rsqrtD = 1.f / std::sqrt(static_cast<float>(headSize));
            float sQkv = inDesc[0].scale, sCtx = outDesc[0].scale;
            if (kind == QkvKind::kInterleaved && useExplicitInt8)
            {
                sQkv = qkvScale;
                sCtx = ctxScale;
            }
            if (dtype() == DataType::kINT8)
            {
                // ref: mhaRunner.cu:1178-1190, qkvToContextInt8InterleavedPlugin.cpp:269-278
                PLG_VALIDATE(sCtx != 0.f && dqProbs > 0.f);
                p.scale_bmm1 = sQkv * sQkv * rsqrtD;
                p.scale_softmax = 1.f / dqProbs;
                p.scale_bmm2 = dqProbs * sQkv / sCtx;
            }
            else
            {
                p.scale_bmm1 = rsqrtD;
                p.scale_softmax = 1.f;
                p.scale_bmm2 = 1.f;
            }
            if (kind == QkvKind::kInterleaved)
            {
                p.total = static_cast<int32_t>(inDesc[0].dims.d[2]);
                p.B = static_cast<int32_t>(inDesc[1].dims.d[0]) - 1;
                p.S = static_cast<int32_t>(inDesc[2].dims.d[0]);
                p.cu_seqlens = static_cast<int32_t const*>(inputs[1]);
                p.interleaved = 1;
                PLG_VALIDATE(p.S <= 384 && "version 6 supports sequence lengths up to 384");
            }
            else if (kind == QkvKind::kVarSeqlen && varSeqlen)
            {
                p.total = static_cast<int32_t>(inDesc[0].dims.d[0]);
                p.B = static_cast<int32_t>(inDesc[2].dims.d[0]) - 1;
                p.S = static_cast<int32_t>(inDesc[3].dims.d[0]);
                p.cu_seqlens = static_cast<int32_t const*>(inputs[2]);
                PLG_VALIDATE(p.S <= 512 && "no variable sequence length attention beyond 512"); // ref: :1220-1221
            }
            else
            {
                p.S = static_cast<int32_t>(inDesc[0].dims.d[SDIM]);
                p.B = static_cast<int32_t>(inDesc[0].dims.d[BDIM]);
                if (hasMask)
                {
                    int64_t const maskWidth = inDesc[1].dims.nbDims == 2 ? inDesc[1].dims.d[1] : 1;
                    if (kind == QkvKind::kFixed && maskWidth != kUnfusedMaskSize)
                    {
                        uint32_t wm = 0, wn = 0;
                        PLG_VALIDATE(packedMaskWarps(p.S, wm, wn) && workspace != nullptr);
                        int32_t const st = abiStatus(
                            bert_b200_packed_mask_to_lengths(stream, p.S, p.B, wm, wn, static_cast<uint32_t>(maskWidth),
                                static_cast<uint32_t const*>(inputs[1]), static_cast<int32_t*>(workspace)),
                            "packed_mask_to_lengths");
                        if (st != BERT_B200_OK)
                            return st;
                        p.mask_idx = static_cast<int32_t const*>(workspace);
                    }
                    else
                    {
                        p.mask_idx = static_cast<int32_t const*>(inputs[1]);
                    }
                }
            }
            return abiStatus(bert_b200_mha(&p, stream), "mha");
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }

protected:
    void serialize(std::vector<PluginField>& f) override
    {
        if (kind != QkvKind::kInterleaved)
            f.emplace_back("type_id", &type, PluginFieldType::kINT32, 1);
        f.emplace_back("hidden_size", &hiddenSize, PluginFieldType::kINT32, 1);
        f.emplace_back("num_heads", &numHeads, PluginFieldType::kINT32, 1);
        if (kind != QkvKind::kInterleaved)
            f.emplace_back("has_mask", &hasMask, PluginFieldType::kINT32, 1);
        if (kind == QkvKind::kFixed)
        {
            // ref: qkvToContextPlugin.cpp:543-579. The runner state of the reference is not needed here.
            f.emplace_back("S", &S, PluginFieldType::kINT32, 1);
            f.emplace_back("B", &B, PluginFieldType::kINT32, 1);
            f.emplace_back("SM", &sm, PluginFieldType::kINT32, 1);
            f.emplace_back("hasUnfusedDispatcher", &hasUnfusedDispatcher, PluginFieldType::kINT32, 1);
        }
        if (kind == QkvKind::kVarSeqlen)
        {
            f.emplace_back("var_seqlen", &varSeqlen, PluginFieldType::kINT32, 1);
            f.emplace_back("use_int8_scale_max", &useInt8ScaleMax, PluginFieldType::kINT32, 1);
            f.emplace_back("S", &S, PluginFieldType::kINT32, 1);
            f.emplace_back("B", &B, PluginFieldType::kINT32, 1);
        }
        if (kind == QkvKind::kInterleaved)
        {
            f.emplace_back("use_int8_scale_max", &useInt8ScaleMax, PluginFieldType::kINT32, 1);
            f.emplace_back("use_explicit_int8", &useExplicitInt8, PluginFieldType::kINT32, 1);
            f.emplace_back("input_qkv_scale", &qkvScale, PluginFieldType::kFLOAT32, 1);
            f.emplace_back("output_ctx_scale", &ctxScale, PluginFieldType::kFLOAT32, 1);
        }
        if (dqProbs >= 0)
            f.emplace_back("dq_probs", &dqProbs, PluginFieldType::kFLOAT32, 1);
    }
};

class QkvToContextCreator : public CreatorBase
{
public:
    explicit QkvToContextCreator(QkvKind kind)
        : CreatorBase(kQkvName, kind == QkvKind::kFixed ? "4" : (kind == QkvKind::kVarSeqlen ? "5" : "6"), attributes(kind))
        , mKind(kind)
    {
    }
    static std::vector<PluginField> attributes(QkvKind kind)
    {
        if (kind == QkvKind::kInterleaved)
            return {PluginField("hidden_size", nullptr, PluginFieldType::kINT32, 1),
                PluginField("num_heads", nullptr, PluginFieldType::kINT32, 1),
                PluginField("dq_probs", nullptr, PluginFieldType::kFLOAT32, 1),
                PluginField("use_int8_scale_max", nullptr, PluginFieldType::kINT32, 1),
                PluginField("use_explicit_int8", nullptr, PluginFieldType::kINT32, 1),
                PluginField("input_qkv_scale", nullptr, PluginFieldType::kFLOAT32, 1),
                PluginField("output_ctx_scale", nullptr, PluginFieldType::kFLOAT32, 1)};
        std::vector<PluginField> a{PluginField("type_id", nullptr, PluginFieldType::kINT32, 1),
            PluginField("hidden_size", nullptr, PluginFieldType::kINT32, 1),
            PluginField("num_heads", nullptr, PluginFieldType::kINT32, 1),
            PluginField("has_mask", nullptr, PluginFieldType::kINT32, 1),
            PluginField("dq_probs", nullptr, PluginFieldType::kFLOAT32, 1)};
        if (kind == QkvKind::kVarSeqlen)
        {
            a.emplace_back("var_seqlen", nullptr, PluginFieldType::kINT32, 1);
            a.emplace_back("use_int8_scale_max", nullptr, PluginFieldType::kINT32, 1);
        }
        return a;
    }
    PluginBase* make(char const* name, PluginFieldCollection const& fc, TensorRTPhase phase) override
    {
        auto p = std::make_unique<QkvToContext>(name, mKind);
        if (mKind == QkvKind::kInterleaved)
            requireFields(fc, {"hidden_size", "num_heads"});
        else
            requireFields(fc, {"type_id", "hidden_size", "num_heads", "has_mask"});
        getInt(fc, "type_id", p->type);
        PLG_VALIDATE(p->type >= 0 && p->type <= 2);
        getInt(fc, "hidden_size", p->hiddenSize);
        getInt(fc, "num_heads", p->numHeads);
        getInt(fc, "has_mask", p->hasMask);
        PLG_VALIDATE(p->hasMask == 0 || p->hasMask == 1);
        getFloat(fc, "dq_probs", p->dqProbs);
        getInt(fc, "var_seqlen", p->varSeqlen);
        getInt(fc, "use_int8_scale_max", p->useInt8ScaleMax);
        getInt(fc, "use_explicit_int8", p->useExplicitInt8);
        getFloat(fc, "input_qkv_scale", p->qkvScale);
        getFloat(fc, "output_ctx_scale", p->ctxScale);
        if (phase == TensorRTPhase::kRUNTIME)
        {
            // serialised engines also carry S, B, SM, hasUnfusedDispatcher and the reference's runner state
            getInt(fc, "S", p->S);
            getInt(fc, "B", p->B);
            getInt(fc, "SM", p->sm);
            getInt(fc, "hasUnfusedDispatcher", p->hasUnfusedDispatcher);
        }
        p->finish();
        return p.release();
    }

private:
    QkvKind mKind;
};

// ================================================================================================
// CustomSkipLayerNormPluginDynamic versions 5 / 6 (linear) and 7 / 8 (INT8 CHW32-interleaved)
// ================================================================================================
class SkipLayerNorm : public PluginBase
{
public:
    SkipLayerNorm(std::string const& name, bool withLdField)
        : PluginBase(name, kSkipName, withLdField ? "5" : "6")
        , withLdField(withLdField)
    {
    }
    bool withLdField;
    int32_t type{0};
    int32_t ld{0};
    HostWeights beta, gamma, bias;
    DeviceBuffer dBeta, dGamma, dBias;

    DataType dtype() const
    {
        return static_cast<DataType>(type);
    }
    DataType cfgType() const // parameters are FP16 for INT8 I/O (ref: skipLayerNormPlugin.cpp:55-67)
    {
        return dtype() == DataType::kINT8 ? DataType::kHALF : dtype();
    }
    void finish()
    {
        PLG_VALIDATE(dtype() == DataType::kFLOAT || dtype() == DataType::kHALF || dtype() == DataType::kINT8);
        if (!withLdField)
            ld = static_cast<int32_t>(beta.count);
        PLG_VALIDATE(ld > 0 && beta.count == ld && gamma.count == ld && (bias.empty() || bias.count == ld));
        dBeta.upload(beta.data(), beta.sizeBytes());
        dGamma.upload(gamma.data(), gamma.sizeBytes());
        if (!bias.empty())
            dBias.upload(bias.data(), bias.sizeBytes());
    }
    IPluginV3* clone() noexcept override
    {
        try
        {
            auto p = std::make_unique<SkipLayerNorm>(mLayerName, withLdField);
            p->type = type;
            p->ld = ld;
            p->beta = beta;
            p->gamma = gamma;
            p->bias = bias;
            p->finish();
            p->setPluginNamespace(mNamespace.c_str());
            return p.release();
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    int32_t getNbOutputs() const noexcept override
    {
        return 1;
    }
    bool supportsFormatCombination(int32_t pos, DynamicPluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs) noexcept override
    {
        if (!inOut || nbInputs != 2 || nbOutputs != 1 || pos < 0 || pos >= 3)
            return false;
        PluginTensorDesc const& d = inOut[pos].desc;
        if (pos == 0)
        {
            if (dtype() == DataType::kINT8)
                return d.type == dtype() && d.format == (ld < 32 ? TensorFormat::kCHW4 : TensorFormat::kCHW32);
            return d.type == dtype() && d.format == TensorFormat::kLINEAR;
        }
        PluginTensorDesc const& prev = inOut[pos - 1].desc;
        return d.type == prev.type && d.format == prev.format;
    }
    int32_t getOutputShapes(DimsExprs const* inputs, int32_t nbInputs, DimsExprs const*, int32_t, DimsExprs* outputs,
        int32_t nbOutputs, IExprBuilder&) noexcept override
    {
        if (!inputs || !outputs || nbInputs != 2 || nbOutputs != 1 || inputs[0].nbDims != inputs[1].nbDims)
            return STATUS_FAILURE;
        outputs[0] = inputs[0];
        return STATUS_SUCCESS;
    }
    int32_t getOutputDataTypes(DataType* out, int32_t nbOutputs, DataType const* in, int32_t nbInputs) const noexcept override
    {
        if (!out || !in || nbOutputs != 1 || nbInputs != 2)
            return STATUS_FAILURE;
        out[0] = in[0];
        return STATUS_SUCCESS;
    }
    int32_t enqueue(PluginTensorDesc const* inDesc, PluginTensorDesc const* outDesc, void const* const* inputs,
        void* const* outputs, void*, cudaStream_t stream) noexcept override
    {
        try
        {
            PLG_VALIDATE(inDesc && outDesc && inputs && outputs);
            PLG_VALIDATE(dBeta.ptr && dGamma.ptr && (bias.empty() || dBias.ptr));
            int64_t const n = volume(inDesc[0].dims);
            if (inDesc[0].type == DataType::kINT8)
            {
                PLG_VALIDATE(outDesc[0].scale != 0.f);
                return abiStatus(bert_b200_skip_layer_norm_dqq(stream, ld, n, static_cast<int8_t const*>(inputs[0]),
                                     static_cast<int8_t const*>(inputs[1]), dBeta.ptr, dGamma.ptr,
                                     static_cast<int8_t*>(outputs[0]), dBias.ptr, inDesc[0].scale, inDesc[1].scale,
                                     1.f / outDesc[0].scale),
                    "skip_layer_norm_dqq");
            }
            return abiStatus(bert_b200_skip_layer_norm(stream, typeId(inDesc[0].type), ld, n, inputs[0], inputs[1], dBeta.ptr,
                                 dGamma.ptr, outputs[0], dBias.ptr),
                "skip_layer_norm");
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }

protected:
    void serialize(std::vector<PluginField>& f) override
    {
        f.emplace_back("type_id", &type, PluginFieldType::kINT32, 1);
        if (withLdField)
            f.emplace_back("ld", &ld, PluginFieldType::kINT32, 1);
        f.emplace_back("beta", beta.data(), beta.fieldType(), static_cast<int32_t>(beta.count));
        f.emplace_back("gamma", gamma.data(), gamma.fieldType(), static_cast<int32_t>(gamma.count));
        if (!bias.empty())
            f.emplace_back("bias", bias.data(), bias.fieldType(), static_cast<int32_t>(bias.count));
    }
};

class SkipLayerNormCreator : public CreatorBase
{
public:
    explicit SkipLayerNormCreator(bool withLdField)
        : CreatorBase(kSkipName, withLdField ? "5" : "6", attributes(withLdField))
        , mWithLd(withLdField)
    {
    }
    static std::vector<PluginField> attributes(bool withLd)
    {
        std::vector<PluginField> a;
        if (withLd)
            a.emplace_back("ld");
        a.emplace_back("type_id");
        a.emplace_back("beta");
        a.emplace_back("gamma");
        a.emplace_back("bias");
        return a;
    }
    PluginBase* make(char const* name, PluginFieldCollection const& fc, TensorRTPhase) override
    {
        auto p = std::make_unique<SkipLayerNorm>(name, mWithLd);
        if (mWithLd)
            requireFields(fc, {"type_id", "ld", "beta", "gamma"});
        else
            requireFields(fc, {"type_id", "beta", "gamma"});
        getInt(fc, "type_id", p->type);
        PLG_VALIDATE(p->type >= 0 && p->type <= 2);
        getInt(fc, "ld", p->ld);
        DataType const cfg = p->cfgType();
        p->beta.assign(*findField(fc, "beta"), cfg);
        p->gamma.assign(*findField(fc, "gamma"), cfg);
        if (PluginField const* b = findField(fc, "bias"); b && b->data)
            p->bias.assign(*b, cfg);
        p->finish();
        return p.release();
    }

private:
    bool mWithLd;
};

class SkipLayerNormInterleaved : public PluginBase
{
public:
    SkipLayerNormInterleaved(std::string const& name, bool mtron)
        : PluginBase(name, kSkipName, mtron ? "8" : "7")
        , mtron(mtron)
    {
    }
    bool mtron;
    HostWeights beta, gamma; // always FP16 (ref: skipLayerNormInt8InterleavedPlugin.cpp:95, 108-111)
    DeviceBuffer dBeta, dGamma;
    int32_t ld{0};

    void finish()
    {
        ld = static_cast<int32_t>(beta.count);
        PLG_VALIDATE(ld > 0 && gamma.count == ld);
        dBeta.upload(beta.data(), beta.sizeBytes());
        dGamma.upload(gamma.data(), gamma.sizeBytes());
    }
    IPluginV3* clone() noexcept override
    {
        try
        {
            auto p = std::make_unique<SkipLayerNormInterleaved>(mLayerName, mtron);
            p->beta = beta;
            p->gamma = gamma;
            p->finish();
            p->setPluginNamespace(mNamespace.c_str());
            return p.release();
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    int32_t getNbOutputs() const noexcept override
    {
        return mtron ? 2 : 1;
    }
    bool supportsFormatCombination(int32_t pos, DynamicPluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs) noexcept override
    {
        if (!inOut || nbInputs != 2 || nbOutputs != getNbOutputs() || pos < 0 || pos >= nbInputs + nbOutputs)
            return false;
        return inOut[pos].desc.type == DataType::kINT8 && inOut[pos].desc.format == TensorFormat::kCHW32;
    }
    int32_t getOutputShapes(DimsExprs const* inputs, int32_t nbInputs, DimsExprs const*, int32_t, DimsExprs* outputs,
        int32_t nbOutputs, IExprBuilder&) noexcept override
    {
        if (!inputs || !outputs || nbInputs != 2 || nbOutputs != getNbOutputs() || inputs[0].nbDims != inputs[1].nbDims)
            return STATUS_FAILURE;
        for (int32_t i = 0; i < nbOutputs; ++i)
            outputs[i] = inputs[0];
        return STATUS_SUCCESS;
    }
    int32_t getOutputDataTypes(DataType* out, int32_t nbOutputs, DataType const* in, int32_t nbInputs) const noexcept override
    {
        if (!out || !in || nbOutputs != getNbOutputs() || nbInputs != 2)
            return STATUS_FAILURE;
        for (int32_t i = 0; i < nbOutputs; ++i)
            out[i] = in[0];
        return STATUS_SUCCESS;
    }
    int32_t enqueue(PluginTensorDesc const* inDesc, PluginTensorDesc const* outDesc, void const* const* inputs,
        void* const* outputs, void*, cudaStream_t stream) noexcept override
    {
        try
        {
            PLG_VALIDATE(inDesc && outDesc && inputs && outputs);
            PLG_VALIDATE(dBeta.ptr && dGamma.ptr);
            // input shape 1 x E x total x 1 (ref: skipLayerNormInt8InterleavedPlugin.cpp:284-291)
            PLG_VALIDATE(inDesc[0].dims.nbDims == 4 && inDesc[0].dims.d[0] == 1 && inDesc[0].dims.d[3] == 1);
            PLG_VALIDATE(inDesc[0].dims.d[1] == ld);
            int32_t const total = static_cast<int32_t>(inDesc[0].dims.d[2]);
            PLG_VALIDATE(outDesc[0].scale != 0.f);
            float const qScale = 1.f / outDesc[0].scale;
            auto const* in = static_cast<int8_t const*>(inputs[0]);
            auto const* skip = static_cast<int8_t const*>(inputs[1]);
            if (!mtron)
                return abiStatus(bert_b200_skip_layer_norm_interleaved_hface(stream, ld, total, in, skip, dBeta.ptr, dGamma.ptr,
                                     static_cast<int8_t*>(outputs[0]), inDesc[0].scale, inDesc[1].scale, qScale),
                    "skip_layer_norm_interleaved_hface");
            PLG_VALIDATE(outDesc[1].scale != 0.f);
            return abiStatus(bert_b200_skip_layer_norm_interleaved_mtron(stream, ld, total, in, skip, dBeta.ptr, dGamma.ptr,
                                 static_cast<int8_t*>(outputs[0]), static_cast<int8_t*>(outputs[1]), inDesc[0].scale,
                                 inDesc[1].scale, qScale, 1.f / outDesc[1].scale),
                "skip_layer_norm_interleaved_mtron");
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }

protected:
    void serialize(std::vector<PluginField>& f) override
    {
        f.emplace_back("beta", beta.data(), PluginFieldType::kFLOAT16, static_cast<int32_t>(beta.count));
        f.emplace_back("gamma", gamma.data(), PluginFieldType::kFLOAT16, static_cast<int32_t>(gamma.count));
    }
};

class SkipLayerNormInterleavedCreator : public CreatorBase
{
public:
    explicit SkipLayerNormInterleavedCreator(bool mtron)
        : CreatorBase(kSkipName, mtron ? "8" : "7", {PluginField("beta"), PluginField("gamma")})
        , mMtron(mtron)
    {
    }
    PluginBase* make(char const* name, PluginFieldCollection const& fc, TensorRTPhase) override
    {
        requireFields(fc, {"beta", "gamma"});
        auto p = std::make_unique<SkipLayerNormInterleaved>(name, mMtron);
        p->beta.assign(*findField(fc, "beta"), DataType::kHALF);
        p->gamma.assign(*findField(fc, "gamma"), DataType::kHALF);
        p->finish();
        return p.release();
    }

private:
    bool mMtron;
};

// ================================================================================================
// CustomFCPluginDynamic version 1
// ================================================================================================
class FullyConnected : public PluginBase
{
public:
    explicit FullyConnected(std::string const& name)
        : PluginBase(name, kFcName, "2")
    {
    }
    int32_t type{0};
    int32_t outDim{0};
    int32_t K{0};
    int32_t activation{0};
    HostWeights W;    // [K][out] as given (FP32 or FP16, the I/O type; FP32 master copy for INT8)
    HostWeights bias; // FP32, optional extension
    float wScale{1.f};
    DeviceBuffer dWt, dBias;

    DataType dtype() const
    {
        return static_cast<DataType>(type);
    }
    // Transposes W [K][out] to Wt [out][K] (the layout the tensor-core tiles read) and uploads it.
    void finish()
    {
        PLG_VALIDATE(dtype() == DataType::kFLOAT || dtype() == DataType::kHALF || dtype() == DataType::kINT8);
        PLG_VALIDATE(outDim > 0 && W.count >= outDim && W.count % outDim == 0); // ref: fcPlugin.cpp:776-781
        K = static_cast<int32_t>(W.count / outDim);
        PLG_VALIDATE(bias.empty() || bias.count == outDim);
        size_t const n = static_cast<size_t>(W.count);
        if (dtype() == DataType::kINT8)
        {
            float amax = 0.f;
            for (size_t i = 0; i < n; ++i)
                amax = std::fmax(amax, std::fabs(W.at(static_cast<int64_t>(i))));
            wScale = (amax > 0.f ? amax : 1.f) / 127.f;
            std::vector<int8_t> wt(n);
            for (int32_t k = 0; k < K; ++k)
                for (int32_t o = 0; o < outDim; ++o)
                {
                    float const q = std::nearbyint(W.at(static_cast<int64_t>(k) * outDim + o) / wScale);
                    wt[static_cast<size_t>(o) * K + k] = static_cast<int8_t>(std::fmax(-127.f, std::fmin(127.f, q)));
                }
            dWt.upload(wt.data(), n);
        }
        else
        {
            size_t const elem = dtype() == DataType::kHALF ? 2 : 4;
            std::vector<uint8_t> wt(n * elem);
            auto const* src = static_cast<uint8_t const*>(W.data());
            for (int32_t k = 0; k < K; ++k)
                for (int32_t o = 0; o < outDim; ++o)
                    std::memcpy(&wt[(static_cast<size_t>(o) * K + k) * elem], &src[(static_cast<size_t>(k) * outDim + o) * elem], elem);
            dWt.upload(wt.data(), wt.size());
        }
        if (!bias.empty())
            dBias.upload(bias.data(), bias.sizeBytes());
    }
    IPluginV3* clone() noexcept override
    {
        try
        {
            auto p = std::make_unique<FullyConnected>(mLayerName);
            p->type = type;
            p->outDim = outDim;
            p->activation = activation;
            p->W = W;
            p->bias = bias;
            p->finish();
            p->setPluginNamespace(mNamespace.c_str());
            return p.release();
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    int32_t getNbOutputs() const noexcept override
    {
        return 1;
    }
    bool supportsFormatCombination(int32_t pos, DynamicPluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs) noexcept override
    {
        if (!inOut || nbInputs != 1 || nbOutputs != 1 || pos < 0 || pos >= 2)
            return false;
        PluginTensorDesc const& d = inOut[pos].desc;
        if (pos == 0)
        {
            TensorFormat const fmt = dtype() == DataType::kINT8 ? int8Format(d.dims.d[HDIM]) : TensorFormat::kLINEAR;
            return d.type == dtype() && d.format == fmt;
        }
        if (dtype() == DataType::kINT8) // INT8 extension: INT8 or FP16 result
            return (d.type == DataType::kINT8 && d.format == int8Format(outDim))
                || (d.type == DataType::kHALF && d.format == TensorFormat::kLINEAR);
        return d.type == inOut[0].desc.type && d.format == inOut[0].desc.format;
    }
    int32_t getOutputShapes(DimsExprs const* inputs, int32_t nbInputs, DimsExprs const*, int32_t, DimsExprs* outputs,
        int32_t nbOutputs, IExprBuilder& eb) noexcept override
    {
        try
        {
            PLG_VALIDATE(inputs && outputs && nbInputs == 1 && nbOutputs == 1);
            outputs[0].nbDims = 5; // ref: fcPlugin.cpp:410-425
            outputs[0].d[0] = inputs[0].d[0];
            outputs[0].d[1] = inputs[0].d[1];
            outputs[0].d[2] = eb.constant(outDim);
            outputs[0].d[3] = eb.constant(1);
            outputs[0].d[4] = eb.constant(1);
            return STATUS_SUCCESS;
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }
    int32_t getOutputDataTypes(DataType* out, int32_t nbOutputs, DataType const* in, int32_t nbInputs) const noexcept override
    {
        if (!out || !in || nbOutputs != 1 || nbInputs != 1)
            return STATUS_FAILURE;
        out[0] = in[0];
        return STATUS_SUCCESS;
    }
    int32_t configurePlugin(DynamicPluginTensorDesc const* in, int32_t nbInputs, DynamicPluginTensorDesc const*, int32_t) noexcept override
    {
        try
        {
            PLG_VALIDATE(in && nbInputs == 1);
            PLG_VALIDATE(in[0].desc.type == dtype() && in[0].desc.dims.nbDims == 5);
            PLG_VALIDATE(in[0].desc.dims.d[HDIM] == K && in[0].desc.dims.d[3] == 1 && in[0].desc.dims.d[4] == 1);
            return STATUS_SUCCESS;
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }
    int32_t enqueue(PluginTensorDesc const* inDesc, PluginTensorDesc const* outDesc, void const* const* inputs,
        void* const* outputs, void*, cudaStream_t stream) noexcept override
    {
        try
        {
            PLG_VALIDATE(inDesc && outDesc && inputs && outputs);
            PLG_VALIDATE(dWt.ptr && (bias.empty() || dBias.ptr));
            bert_b200_fc_params p{};
            p.type_id = type;
            p.out_type_id = typeId(outDesc[0].type);
            p.m = inDesc[0].dims.d[SDIM] * inDesc[0].dims.d[BDIM];
            p.n = outDim;
            p.k = K;
            p.a = inputs[0];
            p.lda = K;
            p.wt = dWt.ptr;
            p.c = outputs[0];
            p.ldc = outDim;
            p.bias = static_cast<float const*>(dBias.ptr);
            p.activation = activation;
            p.alpha = 1.f;
            p.out_scale = 1.f;
            if (dtype() == DataType::kINT8)
            {
                p.alpha = inDesc[0].scale * wScale;
                if (outDesc[0].type == DataType::kINT8)
                {
                    PLG_VALIDATE(outDesc[0].scale != 0.f);
                    p.out_scale = 1.f / outDesc[0].scale;
                }
            }
            return abiStatus(bert_b200_fc(&p, stream), "fc");
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return STATUS_FAILURE;
    }

protected:
    void serialize(std::vector<PluginField>& f) override
    {
        f.emplace_back("out_dims", &outDim, PluginFieldType::kINT32, 1);
        f.emplace_back("type_id", &type, PluginFieldType::kINT32, 1);
        f.emplace_back("W", W.data(), W.fieldType(), static_cast<int32_t>(W.count));
        if (!bias.empty())
            f.emplace_back("bias", bias.data(), PluginFieldType::kFLOAT32, static_cast<int32_t>(bias.count));
        if (activation != 0)
            f.emplace_back("activation", &activation, PluginFieldType::kINT32, 1);
    }
};

class FullyConnectedCreator : public CreatorBase
{
public:
    FullyConnectedCreator()
        : CreatorBase(kFcName, "2",
            {PluginField("out_dims", nullptr, PluginFieldType::kINT32, 1), PluginField("type_id", nullptr, PluginFieldType::kINT32, 1),
                PluginField("W", nullptr, PluginFieldType::kFLOAT32, 1), PluginField("bias", nullptr, PluginFieldType::kFLOAT32, 1),
                PluginField("activation", nullptr, PluginFieldType::kINT32, 1)})
    {
    }
    PluginBase* make(char const* name, PluginFieldCollection const& fc, TensorRTPhase) override
    {
        requireFields(fc, {"out_dims", "type_id", "W"});
        auto p = std::make_unique<FullyConnected>(name);
        getInt(fc, "out_dims", p->outDim);
        getInt(fc, "type_id", p->type);
        PLG_VALIDATE(p->type >= 0 && p->type <= 2);
        getInt(fc, "activation", p->activation);
        PLG_VALIDATE(p->activation == BERT_B200_ACT_NONE || p->activation == BERT_B200_ACT_GELU_ERF);
        // W is stored in the I/O type (ref: fcPlugin.cpp:356-357); INT8 keeps an FP32 master copy
        DataType const wType = p->dtype() == DataType::kHALF ? DataType::kHALF : DataType::kFLOAT;
        p->W.assign(*findField(fc, "W"), wType);
        if (PluginField const* b = findField(fc, "bias"); b && b->data)
            p->bias.assign(*b, DataType::kFLOAT);
        p->finish();
        return p.release();
    }
};

} // namespace

std::vector<CreatorBase*> const& allCreators()
{
    static EmbLayerNormVarSeqlenCreator emb4(false);
    static EmbLayerNormVarSeqlenCreator emb5(true);
    static EmbLayerNormFixedCreator emb6;
    static QkvToContextCreator qkv4(QkvKind::kFixed);
    static QkvToContextCreator qkv5(QkvKind::kVarSeqlen);
    static QkvToContextCreator qkv6(QkvKind::kInterleaved);
    static SkipLayerNormCreator skip5(true);
    static SkipLayerNormCreator skip6(false);
    static SkipLayerNormInterleavedCreator skip7(false);
    static SkipLayerNormInterleavedCreator skip8(true);
    static FullyConnectedCreator fc1;
    static std::vector<CreatorBase*> const all{&emb4, &emb5, &emb6, &qkv4, &qkv5, &qkv6, &skip5, &skip6, &skip7, &skip8, &fc1};
    return all;
}

} // namespace bert_b200_plugin

using namespace bert_b200_plugin;

#define PLUGIN_API extern "C" __attribute__((visibility("default")))

// ref: plugin/vc/vfcCommon.cpp:68-81 (entry points used by IPluginRegistry::loadLibrary / trtexec --dynamicPlugins)
PLUGIN_API nvinfer1::IPluginCreatorInterface* const* getCreators(int32_t& nbCreators)
{
    static std::vector<nvinfer1::IPluginCreatorInterface*> list;
    static std::once_flag once;
    std::call_once(once, [] {
        for (CreatorBase* c : allCreators())
            list.push_back(c);
        for (nvinfer1::IPluginCreatorInterface* c : allLegacyCreators())
            list.push_back(c);
    });
    nbCreators = static_cast<int32_t>(list.size());
    return list.data();
}

PLUGIN_API void setLoggerFinder(nvinfer1::ILoggerFinder* finder)
{
    std::lock_guard<std::mutex> lock(gLogMutex);
    gLoggerFinder = finder;
}

// ref: plugin/api/inferPlugin.cpp:169-210. Registers the creators with the TensorRT registry when libnvinfer is
// loaded in the process (the symbol is looked up at run time; this library does not link libnvinfer).
PLUGIN_API bool initLibNvInferPlugins(void* logger, char const* libNamespace)
{
    if (logger)
        setLogger(static_cast<nvinfer1::ILogger*>(logger));
    using RegistryFn = nvinfer1::IPluginRegistry* (*) ();
    auto const fn = reinterpret_cast<RegistryFn>(dlsym(RTLD_DEFAULT, "getPluginRegistry"));
    bool ok = true;
    for (CreatorBase* c : allCreators())
    {
        c->setPluginNamespace(libNamespace ? libNamespace : "");
        if (fn && fn())
            ok = fn()->registerCreator(*c, libNamespace ? libNamespace : "") && ok;
    }
    for (nvinfer1::IPluginCreatorInterface* c : allLegacyCreators())
    {
        static_cast<nvinfer1::IPluginCreator*>(c)->setPluginNamespace(libNamespace ? libNamespace : "");
        if (fn && fn())
            ok = fn()->registerCreator(*c, libNamespace ? libNamespace : "") && ok;
    }
    return ok;
}

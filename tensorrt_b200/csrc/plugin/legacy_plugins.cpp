// Legacy IPluginV2DynamicExt versions of the BERT plugins:
//   CustomQKVToContextPluginDynamic   1 (fixed), 2 (variable sequence length), 3 (INT8 interleaved)
//   CustomEmbLayerNormPluginDynamic   1 (fixed), 2 / 3 (variable sequence length, HFace / MTron)
//   CustomSkipLayerNormPluginDynamic  1 / 2 (linear), 3 / 4 (INT8 interleaved, HFace / MTron)
//   CustomFCPluginDynamic             1 (the only version the reference has)
// Networks and serialised engines that still name these versions load them from this library. Each legacy version has
// the same inputs, outputs, formats and fields as one IPluginV3 version (QKV 1/2/3 = 4/5/6, Emb 1/2/3 = 6/4/5,
// SkipLN 1/2/3/4 = 5/6/7/8, FC 1 = this library's 2), so an adapter object owns the IPluginV3 object of that version
// and forwards every call; what is specific to the legacy versions is the flat serialisation buffer, written and read
// here in the reference's field order and field widths:
//   ref: plugin/bertQKVToContextPlugin/qkvToContextPluginLegacy.cpp:399-422, 909-925 (+ mhaRunner.cu:461-466, 494-499),
//        plugin/bertQKVToContextPlugin/qkvToContextInt8InterleavedPluginLegacy.cpp:203-216,
//        plugin/embLayerNormPlugin/embLayerNormPluginLegacy.cpp:451-470,
//        plugin/embLayerNormPlugin/embLayerNormVarSeqlenPluginLegacy.cpp:545-562,
//        plugin/skipLayerNormPlugin/skipLayerNormPluginLegacy.cpp:381-397, 900-916,
//        plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedPluginLegacy.cpp:426-435,
//        plugin/fcPlugin/fcPlugin.cpp:661-673 (the cuBLASLt algorithm blob is written as zeros; optional bias /
//        activation of this library follow the weights in a tagged extension block the reference never reads).
// The reference's runner state at the end of the attention buffers (cuBLAS algorithm ids, S, B, head size) is written
// with neutral values and skipped on reading: no kernel here has tunable state.
#include "plugin_common.h"

#include <cstring>
#include <memory>

#if defined(__GNUC__)
#pragma GCC diagnostic ignored "-Wdeprecated-declarations"
#endif

namespace bert_b200_plugin
{
namespace
{

enum class LegacyKind
{
    kQkvFixed,
    kQkvVarSeqlen,
    kQkvInterleaved,
    kEmbFixed,
    kEmbVarSeqlen,
    kSkip,
    kSkipInterleaved,
    kFc
};

struct LegacySpec
{
    char const* name;
    char const* legacyVersion;
    char const* coreVersion; // the IPluginV3 version with the same behaviour
    LegacyKind kind;
};

constexpr char const* kQkv = "CustomQKVToContextPluginDynamic";
constexpr char const* kEmb = "CustomEmbLayerNormPluginDynamic";
constexpr char const* kSkip = "CustomSkipLayerNormPluginDynamic";
constexpr char const* kFc = "CustomFCPluginDynamic";
constexpr uint32_t kFcExtensionTag = 0x30303242u; // "B200"
constexpr size_t kLtAlgoBytes = 64;              // sizeof(cublasLtMatmulAlgo_t): uint64_t data[8]

LegacySpec const kSpecs[] = {
    {kQkv, "1", "4", LegacyKind::kQkvFixed},
    {kQkv, "2", "5", LegacyKind::kQkvVarSeqlen},
    {kQkv, "3", "6", LegacyKind::kQkvInterleaved},
    {kEmb, "1", "6", LegacyKind::kEmbFixed},
    {kEmb, "2", "4", LegacyKind::kEmbVarSeqlen},
    {kEmb, "3", "5", LegacyKind::kEmbVarSeqlen},
    {kSkip, "1", "5", LegacyKind::kSkip},
    {kSkip, "2", "6", LegacyKind::kSkip},
    {kSkip, "3", "7", LegacyKind::kSkipInterleaved},
    {kSkip, "4", "8", LegacyKind::kSkipInterleaved},
    {kFc, "1", "2", LegacyKind::kFc},
};

CreatorBase* coreCreator(LegacySpec const& spec)
{
    for (CreatorBase* c : allCreators())
        if (std::strcmp(c->getPluginName(), spec.name) == 0 && std::strcmp(c->getPluginVersion(), spec.coreVersion) == 0)
            return c;
    return nullptr;
}

// ---- flat buffer helpers ---------------------------------------------------------------------
struct Writer
{
    std::vector<uint8_t> bytes;
    template <typename T>
    void put(T v)
    {
        auto const* p = reinterpret_cast<uint8_t const*>(&v);
        bytes.insert(bytes.end(), p, p + sizeof(T));
    }
    void putBool(bool v)
    {
        put<uint8_t>(v ? 1 : 0); // the reference writes sizeof(bool) = 1 byte
    }
    void putRaw(void const* p, size_t n)
    {
        auto const* b = static_cast<uint8_t const*>(p);
        bytes.insert(bytes.end(), b, b + n);
    }
};

struct Reader
{
    uint8_t const* p;
    size_t left;
    template <typename T>
    T get()
    {
        if (left < sizeof(T))
            throw PluginError("legacy plugin: serialised buffer is too short");
        T v;
        std::memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        left -= sizeof(T);
        return v;
    }
    bool getBool()
    {
        return get<uint8_t>() != 0;
    }
    void const* raw(size_t n)
    {
        if (left < n)
            throw PluginError("legacy plugin: serialised buffer is too short");
        void const* r = p;
        p += n;
        left -= n;
        return r;
    }
};

int32_t fieldInt(PluginFieldCollection const& fc, char const* name, int32_t fallback)
{
    int32_t v = fallback;
    getInt(fc, name, v);
    return v;
}

float fieldFloat(PluginFieldCollection const& fc, char const* name, float fallback)
{
    float v = fallback;
    getFloat(fc, name, v);
    return v;
}

size_t fieldElemSize(PluginField const& f)
{
    return f.type == PluginFieldType::kFLOAT16 ? 2 : 4;
}

// Fields handed to a core creator; the ints / floats live in the deque-like storage of this object.
struct FieldList
{
    std::vector<PluginField> fields;
    std::vector<std::unique_ptr<int32_t>> ints;
    std::vector<std::unique_ptr<float>> floats;
    void addInt(char const* name, int32_t v)
    {
        ints.push_back(std::make_unique<int32_t>(v));
        fields.emplace_back(name, ints.back().get(), PluginFieldType::kINT32, 1);
    }
    void addFloat(char const* name, float v)
    {
        floats.push_back(std::make_unique<float>(v));
        fields.emplace_back(name, floats.back().get(), PluginFieldType::kFLOAT32, 1);
    }
    void addArray(char const* name, void const* data, bool half, int64_t count)
    {
        fields.emplace_back(name, data, half ? PluginFieldType::kFLOAT16 : PluginFieldType::kFLOAT32, static_cast<int32_t>(count));
    }
    PluginFieldCollection collection()
    {
        PluginFieldCollection fc{};
        fc.nbFields = static_cast<int32_t>(fields.size());
        fc.fields = fields.data();
        return fc;
    }
};

constexpr int32_t kHalf = static_cast<int32_t>(DataType::kHALF);
constexpr int32_t kInt8 = static_cast<int32_t>(DataType::kINT8);
constexpr int32_t kSmVersion = 100;

// ---- core fields -> flat buffer ----------------------------------------------------------------
void writeFlat(LegacyKind kind, PluginFieldCollection const& fc, Writer& w)
{
    auto array = [&](char const* name) -> PluginField const& {
        PluginField const* f = findField(fc, name);
        if (!f || !f->data)
            throw PluginError(std::string("legacy plugin: field missing for serialisation: ") + name);
        return *f;
    };
    auto putArray = [&](PluginField const& f) { w.putRaw(f.data, static_cast<size_t>(f.length) * fieldElemSize(f)); };
    switch (kind)
    {
    case LegacyKind::kQkvFixed:
    case LegacyKind::kQkvVarSeqlen:
    {
        int32_t const hidden = fieldInt(fc, "hidden_size", 0);
        int32_t const heads = fieldInt(fc, "num_heads", 1);
        int32_t const headSize = heads > 0 ? hidden / heads : 0;
        int32_t const S = fieldInt(fc, "S", 0);
        int32_t const B = fieldInt(fc, "B", 0);
        w.put<int32_t>(fieldInt(fc, "type_id", 0));
        w.put<int32_t>(heads);
        w.put<int32_t>(headSize);
        w.putBool(fieldInt(fc, "has_mask", 0) != 0);
        w.put<int32_t>(hidden);
        w.put<int32_t>(fieldInt(fc, "SM", kSmVersion));
        w.put<int32_t>(S);
        w.put<int32_t>(B);
        w.put<float>(fieldFloat(fc, "dq_probs", -1.f));
        if (kind == LegacyKind::kQkvFixed)
        {
            w.put<int32_t>(0); // no unfused runner state follows
        }
        else
        {
            w.putBool(fieldInt(fc, "var_seqlen", 0) != 0);
            w.put<int32_t>(headSize); // padded head size of the reference; no padding here
            w.putBool(fieldInt(fc, "use_int8_scale_max", 1) != 0);
            w.put<int32_t>(S); // runner state: S, B, head size
            w.put<int32_t>(B);
            w.put<int32_t>(headSize);
        }
        break;
    }
    case LegacyKind::kQkvInterleaved:
    {
        int32_t const hidden = fieldInt(fc, "hidden_size", 0);
        int32_t const heads = fieldInt(fc, "num_heads", 1);
        w.put<int32_t>(heads);
        w.put<int32_t>(heads > 0 ? hidden / heads : 0);
        w.put<int32_t>(hidden);
        w.put<int32_t>(kSmVersion);
        w.put<int32_t>(fieldInt(fc, "S", 0));
        w.put<int32_t>(fieldInt(fc, "B", 0));
        w.put<float>(fieldFloat(fc, "dq_probs", -1.f));
        w.putBool(fieldInt(fc, "use_int8_scale_max", 1) != 0);
        w.putBool(fieldInt(fc, "use_explicit_int8", 0) != 0);
        w.put<float>(fieldFloat(fc, "input_qkv_scale", 1.f));
        w.put<float>(fieldFloat(fc, "output_ctx_scale", 1.f));
        break;
    }
    case LegacyKind::kEmbFixed:
    case LegacyKind::kEmbVarSeqlen:
    {
        PluginField const& beta = array("bert_embeddings_layernorm_beta");
        PluginField const& gamma = array("bert_embeddings_layernorm_gamma");
        PluginField const& word = array("bert_embeddings_word_embeddings");
        PluginField const& tok = array("bert_embeddings_token_type_embeddings");
        PluginField const& pos = array("bert_embeddings_position_embeddings");
        uint64_t const ld = static_cast<uint64_t>(beta.length);
        PLG_VALIDATE(ld > 0 && beta.type == PluginFieldType::kFLOAT32 && gamma.type == PluginFieldType::kFLOAT32);
        bool const half = fieldInt(fc, "output_fp16", 0) != 0;
        w.put<int32_t>(half ? kHalf : 0);
        if (kind == LegacyKind::kEmbFixed)
            w.put<int32_t>(fieldInt(fc, "mha_type_id", 0));
        w.put<uint64_t>(ld);
        if (kind == LegacyKind::kEmbFixed)
            w.put<uint64_t>(0); // configured sequence length: not needed to rebuild the object
        w.put<uint64_t>(static_cast<uint64_t>(word.length) / ld);
        w.put<uint64_t>(static_cast<uint64_t>(pos.length) / ld);
        w.put<uint64_t>(static_cast<uint64_t>(tok.length) / ld);
        if (kind == LegacyKind::kEmbFixed)
        {
            w.putBool(fieldInt(fc, "full_mask", 0) != 0);
            w.put<int32_t>(kSmVersion);
        }
        else
        {
            w.put<int32_t>(half ? kHalf : 0); // mask type of the reference: follows the output type
        }
        putArray(beta);
        putArray(gamma);
        putArray(word);
        putArray(pos);
        putArray(tok);
        break;
    }
    case LegacyKind::kSkip:
    {
        PluginField const& beta = array("beta");
        PluginField const& gamma = array("gamma");
        PluginField const* bias = findField(fc, "bias");
        int32_t const type = fieldInt(fc, "type_id", 0);
        w.put<int32_t>(type);
        w.put<int32_t>(type == kInt8 ? kHalf : type); // parameter type: FP32 or FP16
        w.put<uint64_t>(static_cast<uint64_t>(beta.length));
        w.putBool(bias != nullptr && bias->data != nullptr);
        putArray(beta);
        putArray(gamma);
        if (bias && bias->data)
            putArray(*bias);
        break;
    }
    case LegacyKind::kSkipInterleaved:
    {
        PluginField const& beta = array("beta");
        PluginField const& gamma = array("gamma");
        w.put<uint64_t>(static_cast<uint64_t>(beta.length));
        putArray(beta);
        putArray(gamma);
        break;
    }
    case LegacyKind::kFc:
    {
        PluginField const& W = array("W");
        PluginField const* bias = findField(fc, "bias");
        int32_t const outDim = fieldInt(fc, "out_dims", 0);
        int32_t const activation = fieldInt(fc, "activation", 0);
        PLG_VALIDATE(outDim > 0);
        w.put<int32_t>(fieldInt(fc, "type_id", 0));
        w.put<uint64_t>(static_cast<uint64_t>(outDim));
        w.put<uint64_t>(static_cast<uint64_t>(W.length));
        w.put<int32_t>(0);                        // Nmax: only used by the reference's algorithm search
        w.put<int32_t>(W.length / outDim);        // K
        uint8_t const noAlgo[kLtAlgoBytes] = {};
        w.putRaw(noAlgo, sizeof(noAlgo));
        putArray(W);
        bool const hasBias = bias != nullptr && bias->data != nullptr;
        if (hasBias || activation != 0)
        {
            w.put<uint32_t>(kFcExtensionTag);
            w.put<int32_t>(activation);
            w.putBool(hasBias);
            if (hasBias)
                putArray(*bias);
        }
        break;
    }
    }
}

// ---- flat buffer -> fields for the core creator (arrays point into the buffer) ----------------------
void readFlat(LegacySpec const& spec, Reader& r, FieldList& f)
{
    switch (spec.kind)
    {
    case LegacyKind::kQkvFixed:
    case LegacyKind::kQkvVarSeqlen:
    {
        int32_t const type = r.get<int32_t>();
        int32_t const heads = r.get<int32_t>();
        r.get<int32_t>(); // head size
        bool const hasMask = r.getBool();
        int32_t const hidden = r.get<int32_t>();
        int32_t const sm = r.get<int32_t>();
        int32_t const S = r.get<int32_t>();
        int32_t const B = r.get<int32_t>();
        float const dqProbs = r.get<float>();
        f.addInt("type_id", type);
        f.addInt("hidden_size", hidden);
        f.addInt("num_heads", heads);
        f.addInt("has_mask", hasMask ? 1 : 0);
        if (dqProbs >= 0.f)
            f.addFloat("dq_probs", dqProbs);
        f.addInt("S", S);
        f.addInt("B", B);
        f.addInt("SM", sm);
        if (spec.kind == LegacyKind::kQkvVarSeqlen)
        {
            f.addInt("var_seqlen", r.getBool() ? 1 : 0);
            r.get<int32_t>(); // padded head size
            f.addInt("use_int8_scale_max", r.getBool() ? 1 : 0);
        }
        // whatever follows is the reference's runner state
        break;
    }
    case LegacyKind::kQkvInterleaved:
    {
        int32_t const heads = r.get<int32_t>();
        r.get<int32_t>(); // head size
        int32_t const hidden = r.get<int32_t>();
        r.get<int32_t>(); // SM
        int32_t const S = r.get<int32_t>();
        int32_t const B = r.get<int32_t>();
        float const dqProbs = r.get<float>();
        f.addInt("hidden_size", hidden);
        f.addInt("num_heads", heads);
        if (dqProbs >= 0.f)
            f.addFloat("dq_probs", dqProbs);
        f.addInt("use_int8_scale_max", r.getBool() ? 1 : 0);
        f.addInt("use_explicit_int8", r.getBool() ? 1 : 0);
        f.addFloat("input_qkv_scale", r.get<float>());
        f.addFloat("output_ctx_scale", r.get<float>());
        f.addInt("S", S);
        f.addInt("B", B);
        break;
    }
    case LegacyKind::kEmbFixed:
    case LegacyKind::kEmbVarSeqlen:
    {
        int32_t const type = r.get<int32_t>();
        PLG_VALIDATE(type == 0 || type == kHalf);
        bool const half = type == kHalf;
        int32_t mhaType = 0;
        if (spec.kind == LegacyKind::kEmbFixed)
            mhaType = r.get<int32_t>();
        uint64_t const ld = r.get<uint64_t>();
        if (spec.kind == LegacyKind::kEmbFixed)
            r.get<uint64_t>(); // configured sequence length
        uint64_t const wordVocab = r.get<uint64_t>();
        uint64_t const posVocab = r.get<uint64_t>();
        uint64_t const tokVocab = r.get<uint64_t>();
        PLG_VALIDATE(ld > 0 && ld < (1ull << 20) && wordVocab < (1ull << 31) / ld && posVocab < (1ull << 31) / ld
            && tokVocab < (1ull << 31) / ld);
        f.addInt("output_fp16", half ? 1 : 0);
        if (spec.kind == LegacyKind::kEmbFixed)
        {
            f.addInt("full_mask", r.getBool() ? 1 : 0);
            r.get<int32_t>(); // SM
            f.addInt("mha_type_id", mhaType);
        }
        else
        {
            r.get<int32_t>(); // mask type
        }
        size_t const wordSize = half ? 2 : 4;
        f.addArray("bert_embeddings_layernorm_beta", r.raw(ld * 4), false, static_cast<int64_t>(ld));
        f.addArray("bert_embeddings_layernorm_gamma", r.raw(ld * 4), false, static_cast<int64_t>(ld));
        f.addArray("bert_embeddings_word_embeddings", r.raw(ld * wordVocab * wordSize), half, static_cast<int64_t>(ld * wordVocab));
        f.addArray("bert_embeddings_position_embeddings", r.raw(ld * posVocab * wordSize), half, static_cast<int64_t>(ld * posVocab));
        f.addArray("bert_embeddings_token_type_embeddings", r.raw(ld * tokVocab * wordSize), half, static_cast<int64_t>(ld * tokVocab));
        break;
    }
    case LegacyKind::kSkip:
    {
        int32_t const type = r.get<int32_t>();
        int32_t const cfgType = r.get<int32_t>();
        uint64_t const ld = r.get<uint64_t>();
        bool const hasBias = r.getBool();
        PLG_VALIDATE((cfgType == 0 || cfgType == kHalf) && ld > 0 && ld < (1ull << 24));
        bool const half = cfgType == kHalf;
        size_t const bytes = ld * (half ? 2 : 4);
        f.addInt("type_id", type);
        if (std::strcmp(spec.coreVersion, "5") == 0)
            f.addInt("ld", static_cast<int32_t>(ld));
        f.addArray("beta", r.raw(bytes), half, static_cast<int64_t>(ld));
        f.addArray("gamma", r.raw(bytes), half, static_cast<int64_t>(ld));
        if (hasBias)
            f.addArray("bias", r.raw(bytes), half, static_cast<int64_t>(ld));
        break;
    }
    case LegacyKind::kSkipInterleaved:
    {
        uint64_t const ld = r.get<uint64_t>();
        PLG_VALIDATE(ld > 0 && ld < (1ull << 24));
        f.addArray("beta", r.raw(ld * 2), true, static_cast<int64_t>(ld));
        f.addArray("gamma", r.raw(ld * 2), true, static_cast<int64_t>(ld));
        break;
    }
    case LegacyKind::kFc:
    {
        int32_t const type = r.get<int32_t>();
        uint64_t const outDim = r.get<uint64_t>();
        uint64_t const numParams = r.get<uint64_t>();
        r.get<int32_t>(); // Nmax
        r.get<int32_t>(); // K
        r.raw(kLtAlgoBytes);
        PLG_VALIDATE(type >= 0 && type <= kInt8 && outDim > 0 && outDim < (1ull << 31) && numParams < (1ull << 31));
        bool const half = type == kHalf; // FP32 and (this library's) INT8 objects keep FP32 weights
        f.addInt("out_dims", static_cast<int32_t>(outDim));
        f.addInt("type_id", type);
        f.addArray("W", r.raw(numParams * (half ? 2 : 4)), half, static_cast<int64_t>(numParams));
        if (r.left >= 9)
        {
            Reader ext = r;
            if (ext.get<uint32_t>() == kFcExtensionTag)
            {
                int32_t const activation = ext.get<int32_t>();
                bool const hasBias = ext.getBool();
                if (activation != 0)
                    f.addInt("activation", activation);
                if (hasBias)
                    f.addArray("bias", ext.raw(outDim * 4), false, static_cast<int64_t>(outDim));
            }
        }
        break;
    }
    }
}

// ---- the adapter -----------------------------------------------------------------------------
class LegacyAdapter final : public nvinfer1::IPluginV2DynamicExt
{
public:
    LegacyAdapter(LegacySpec const& spec, PluginBase* core)
        : mSpec(spec)
        , mCore(core)
    {
    }
    ~LegacyAdapter() noexcept override = default;

    // IPluginV2DynamicExt
    nvinfer1::IPluginV2DynamicExt* clone() const noexcept override
    {
        try
        {
            auto* c = static_cast<PluginBase*>(mCore->clone());
            if (!c)
                return nullptr;
            auto* a = new LegacyAdapter(mSpec, c);
            a->mNamespace = mNamespace;
            return a;
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    nvinfer1::DimsExprs getOutputDimensions(
        int32_t outputIndex, nvinfer1::DimsExprs const* inputs, int32_t nbInputs, nvinfer1::IExprBuilder& exprBuilder) noexcept override
    {
        nvinfer1::DimsExprs outs[kMaxOutputs]{};
        int32_t const n = getNbOutputs();
        if (outputIndex < 0 || outputIndex >= n || n > kMaxOutputs
            || build()->getOutputShapes(inputs, nbInputs, nullptr, 0, outs, n, exprBuilder) != 0)
        {
            nvinfer1::DimsExprs bad{};
            bad.nbDims = -1;
            return bad;
        }
        return outs[outputIndex];
    }
    bool supportsFormatCombination(
        int32_t pos, nvinfer1::PluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs) noexcept override
    {
        try
        {
            std::vector<DynamicPluginTensorDesc> d = dynamic(inOut, nbInputs + nbOutputs);
            return build()->supportsFormatCombination(pos, d.data(), nbInputs, nbOutputs);
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return false;
    }
    void configurePlugin(DynamicPluginTensorDesc const* in, int32_t nbInputs, DynamicPluginTensorDesc const* out,
        int32_t nbOutputs) noexcept override
    {
        build()->configurePlugin(in, nbInputs, out, nbOutputs);
    }
    size_t getWorkspaceSize(nvinfer1::PluginTensorDesc const* inputs, int32_t nbInputs, nvinfer1::PluginTensorDesc const* outputs,
        int32_t nbOutputs) const noexcept override
    {
        try
        {
            std::vector<DynamicPluginTensorDesc> i = dynamic(inputs, nbInputs), o = dynamic(outputs, nbOutputs);
            return build()->getWorkspaceSize(i.data(), nbInputs, o.data(), nbOutputs);
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return 0;
    }
    int32_t enqueue(nvinfer1::PluginTensorDesc const* inputDesc, nvinfer1::PluginTensorDesc const* outputDesc,
        void const* const* inputs, void* const* outputs, void* workspace, cudaStream_t stream) noexcept override
    {
        auto* rt = static_cast<IPluginV3OneRuntime*>(mCore->getCapabilityInterface(PluginCapabilityType::kRUNTIME));
        return rt->enqueue(inputDesc, outputDesc, inputs, outputs, workspace, stream);
    }

    // IPluginV2Ext
    nvinfer1::DataType getOutputDataType(int32_t index, nvinfer1::DataType const* inputTypes, int32_t nbInputs) const noexcept override
    {
        nvinfer1::DataType outs[kMaxOutputs]{};
        int32_t const n = getNbOutputs();
        if (index < 0 || index >= n || n > kMaxOutputs || build()->getOutputDataTypes(outs, n, inputTypes, nbInputs) != 0)
            return nvinfer1::DataType::kFLOAT;
        return outs[index];
    }
    void attachToContext(cudnnContext*, cublasContext*, nvinfer1::IGpuAllocator*) noexcept override {}
    void detachFromContext() noexcept override {}

    // IPluginV2
    char const* getPluginType() const noexcept override
    {
        return mSpec.name;
    }
    char const* getPluginVersion() const noexcept override
    {
        return mSpec.legacyVersion;
    }
    int32_t getNbOutputs() const noexcept override
    {
        return build()->getNbOutputs();
    }
    int32_t initialize() noexcept override
    {
        return 0;
    }
    void terminate() noexcept override {}
    size_t getSerializationSize() const noexcept override
    {
        try
        {
            return flat().size();
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return 0;
    }
    void serialize(void* buffer) const noexcept override
    {
        try
        {
            std::vector<uint8_t> const b = flat();
            std::memcpy(buffer, b.data(), b.size());
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
    }
    void destroy() noexcept override
    {
        delete this;
    }
    void setPluginNamespace(char const* ns) noexcept override
    {
        mNamespace = ns ? ns : "";
    }
    char const* getPluginNamespace() const noexcept override
    {
        return mNamespace.c_str();
    }

private:
    static constexpr int32_t kMaxOutputs = 4;

    IPluginV3OneBuild* build() const
    {
        return static_cast<IPluginV3OneBuild*>(mCore->getCapabilityInterface(PluginCapabilityType::kBUILD));
    }
    static std::vector<DynamicPluginTensorDesc> dynamic(nvinfer1::PluginTensorDesc const* descs, int32_t n)
    {
        std::vector<DynamicPluginTensorDesc> d(static_cast<size_t>(n > 0 ? n : 0));
        for (int32_t i = 0; i < n; ++i)
        {
            d[i].desc = descs[i];
            d[i].min = descs[i].dims;
            d[i].max = descs[i].dims;
            d[i].opt = descs[i].dims;
        }
        return d;
    }
    std::vector<uint8_t> flat() const
    {
        auto* rt = static_cast<IPluginV3OneRuntime*>(mCore->getCapabilityInterface(PluginCapabilityType::kRUNTIME));
        PluginFieldCollection const* fc = rt->getFieldsToSerialize();
        if (!fc)
            throw PluginError("legacy plugin: the core object did not report its fields");
        Writer w;
        writeFlat(mSpec.kind, *fc, w);
        return std::move(w.bytes);
    }

    LegacySpec mSpec;
    std::unique_ptr<PluginBase> mCore;
    std::string mNamespace;
};

class LegacyCreator final : public nvinfer1::IPluginCreator
{
public:
    explicit LegacyCreator(LegacySpec const& spec)
        : mSpec(spec)
    {
    }
    char const* getPluginName() const noexcept override
    {
        return mSpec.name;
    }
    char const* getPluginVersion() const noexcept override
    {
        return mSpec.legacyVersion;
    }
    PluginFieldCollection const* getFieldNames() noexcept override
    {
        CreatorBase* c = coreCreator(mSpec);
        return c ? c->getFieldNames() : nullptr;
    }
    nvinfer1::IPluginV2* createPlugin(char const* name, PluginFieldCollection const* fc) noexcept override
    {
        try
        {
            PLG_VALIDATE(fc != nullptr);
            return wrap(name, *fc, TensorRTPhase::kBUILD);
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    nvinfer1::IPluginV2* deserializePlugin(char const* name, void const* serialData, size_t serialLength) noexcept override
    {
        try
        {
            PLG_VALIDATE(serialData != nullptr);
            Reader r{static_cast<uint8_t const*>(serialData), serialLength};
            FieldList fields;
            readFlat(mSpec, r, fields);
            PluginFieldCollection const fc = fields.collection();
            return wrap(name, fc, TensorRTPhase::kRUNTIME);
        }
        catch (std::exception const& e)
        {
            caughtError(e);
        }
        return nullptr;
    }
    void setPluginNamespace(char const* ns) noexcept override
    {
        mNamespace = ns ? ns : "";
    }
    char const* getPluginNamespace() const noexcept override
    {
        return mNamespace.c_str();
    }

private:
    nvinfer1::IPluginV2* wrap(char const* name, PluginFieldCollection const& fc, TensorRTPhase phase)
    {
        CreatorBase* c = coreCreator(mSpec);
        if (!c)
            throw PluginError("legacy plugin: no core creator for this version");
        auto* core = static_cast<PluginBase*>(c->createPlugin(name ? name : "", &fc, phase));
        if (!core)
            return nullptr;
        auto* a = new LegacyAdapter(mSpec, core);
        a->setPluginNamespace(mNamespace.c_str());
        return a;
    }

    LegacySpec mSpec;
    std::string mNamespace;
};

} // namespace

std::vector<nvinfer1::IPluginCreatorInterface*> const& allLegacyCreators()
{
    static std::vector<nvinfer1::IPluginCreatorInterface*> const list = [] {
        std::vector<nvinfer1::IPluginCreatorInterface*> v;
        for (LegacySpec const& s : kSpecs)
            v.push_back(new LegacyCreator(s));
        return v;
    }();
    return list;
}

} // namespace bert_b200_plugin

// Minimal host standing in for the TensorRT builder / runtime, so that the plugin objects can be driven through
// their real IPluginV3 interfaces without libnvinfer: createPlugin -> supportsFormatCombination -> getOutputShapes
// -> getOutputDataTypes -> configurePlugin -> getWorkspaceSize -> onShapeChange -> enqueue -> getFieldsToSerialize
// -> createPlugin(kRUNTIME) -> clone / attachToContext. All arguments are the POD structs of the public headers
// (PluginFieldCollection, DynamicPluginTensorDesc, PluginTensorDesc, Dims), so ctypes can build them.
#include "plugin_common.h"

#include <NvInferImpl.h>

#include <deque>

using namespace bert_b200_plugin;

namespace
{

// Constant-folding stand-in for the builder's dimension expressions.
struct ConstExprImpl : public nvinfer1::apiv::VDimensionExpr
{
    int64_t value{0};
    bool isConstant() const override
    {
        return true;
    }
    int64_t getConstantValue() const override
    {
        return value;
    }
    bool isSizeTensor() const override
    {
        return false;
    }
};

struct ConstExpr : public nvinfer1::IDimensionExpr
{
    ConstExprImpl impl;
    explicit ConstExpr(int64_t v)
    {
        impl.value = v;
        mImpl = &impl;
    }
    ~ConstExpr() noexcept override = default;
};

struct ExprBuilderImpl : public nvinfer1::apiv::VExprBuilder
{
    std::deque<std::unique_ptr<ConstExpr>> pool;
    nvinfer1::IDimensionExpr const* constant(int64_t value) override
    {
        pool.push_back(std::make_unique<ConstExpr>(value));
        return pool.back().get();
    }
    nvinfer1::IDimensionExpr const* operation(
        nvinfer1::DimensionOperation op, nvinfer1::IDimensionExpr const& a, nvinfer1::IDimensionExpr const& b) override
    {
        int64_t const x = a.getConstantValue();
        int64_t const y = b.getConstantValue();
        int64_t r = 0;
        switch (op)
        {
        case nvinfer1::DimensionOperation::kSUM: r = x + y; break;
        case nvinfer1::DimensionOperation::kPROD: r = x * y; break;
        case nvinfer1::DimensionOperation::kMAX: r = x > y ? x : y; break;
        case nvinfer1::DimensionOperation::kMIN: r = x < y ? x : y; break;
        case nvinfer1::DimensionOperation::kSUB: r = x - y; break;
        case nvinfer1::DimensionOperation::kEQUAL: r = x == y; break;
        case nvinfer1::DimensionOperation::kLESS: r = x < y; break;
        case nvinfer1::DimensionOperation::kFLOOR_DIV: r = y ? x / y : 0; break;
        case nvinfer1::DimensionOperation::kCEIL_DIV: r = y ? (x + y - 1) / y : 0; break;
        }
        return constant(r);
    }
    nvinfer1::IDimensionExpr const* declareSizeTensor(int32_t, nvinfer1::IDimensionExpr const& opt, nvinfer1::IDimensionExpr const&) override
    {
        return &opt;
    }
};

struct ExprBuilder : public nvinfer1::IExprBuilder
{
    ExprBuilderImpl impl;
    ExprBuilder()
    {
        mImpl = &impl;
    }
    ~ExprBuilder() noexcept override = default;
};

template <typename T>
T* capability(nvinfer1::IPluginV3* p, nvinfer1::PluginCapabilityType type)
{
    return p ? static_cast<T*>(p->getCapabilityInterface(type)) : nullptr;
}

} // namespace

#define HARNESS_API extern "C" __attribute__((visibility("default")))

HARNESS_API nvinfer1::IPluginCreatorInterface* const* getCreators(int32_t& nbCreators);

namespace
{
bool isLegacy(nvinfer1::IPluginCreatorInterface* c)
{
    return std::strcmp(c->getInterfaceInfo().kind, "PLUGIN CREATOR_V1") == 0;
}

nvinfer1::IPluginCreator* legacyCreator(char const* name, char const* version)
{
    int32_t n = 0;
    auto* const* list = getCreators(n);
    for (int32_t i = 0; i < n; ++i)
    {
        if (!isLegacy(list[i]))
            continue;
        auto* c = static_cast<nvinfer1::IPluginCreator*>(list[i]);
        if (std::strcmp(c->getPluginName(), name) == 0 && std::strcmp(c->getPluginVersion(), version) == 0)
            return c;
    }
    return nullptr;
}
} // namespace

HARNESS_API int32_t bert_b200_harness_num_creators()
{
    int32_t n = 0;
    getCreators(n);
    return n;
}

// name / version / namespace / number of advertised fields of creator i
HARNESS_API int32_t bert_b200_harness_creator_info(int32_t i, char const** name, char const** version, char const** ns, int32_t* nbFields)
{
    int32_t n = 0;
    auto* const* list = getCreators(n);
    if (i < 0 || i >= n)
        return 1;
    if (isLegacy(list[i]))
    {
        auto* c = static_cast<nvinfer1::IPluginCreator*>(list[i]);
        *name = c->getPluginName();
        *version = c->getPluginVersion();
        *ns = c->getPluginNamespace();
        *nbFields = c->getFieldNames()->nbFields;
        return 0;
    }
    auto* c = static_cast<nvinfer1::IPluginCreatorV3One*>(list[i]);
    *name = c->getPluginName();
    *version = c->getPluginVersion();
    *ns = c->getPluginNamespace();
    *nbFields = c->getFieldNames()->nbFields;
    return 0;
}

// 1 if creator i is an IPluginCreator (legacy IPluginV2DynamicExt plugins), 0 if IPluginCreatorV3One
HARNESS_API int32_t bert_b200_harness_creator_is_legacy(int32_t i)
{
    int32_t n = 0;
    auto* const* list = getCreators(n);
    return i >= 0 && i < n ? (isLegacy(list[i]) ? 1 : 0) : -1;
}

HARNESS_API char const* bert_b200_harness_creator_field_name(int32_t i, int32_t f)
{
    int32_t n = 0;
    auto* const* list = getCreators(n);
    if (i < 0 || i >= n)
        return nullptr;
    auto const* fc = isLegacy(list[i]) ? static_cast<nvinfer1::IPluginCreator*>(list[i])->getFieldNames()
                                       : static_cast<nvinfer1::IPluginCreatorV3One*>(list[i])->getFieldNames();
    return f >= 0 && f < fc->nbFields ? fc->fields[f].name : nullptr;
}

HARNESS_API nvinfer1::IPluginV3* bert_b200_harness_create(
    char const* name, char const* version, nvinfer1::PluginFieldCollection const* fc, int32_t phase)
{
    int32_t n = 0;
    auto* const* list = getCreators(n);
    for (int32_t i = 0; i < n; ++i)
    {
        if (isLegacy(list[i]))
            continue;
        auto* c = static_cast<nvinfer1::IPluginCreatorV3One*>(list[i]);
        if (std::strcmp(c->getPluginName(), name) == 0 && std::strcmp(c->getPluginVersion(), version) == 0)
            return c->createPlugin("harness_layer", fc, static_cast<nvinfer1::TensorRTPhase>(phase));
    }
    return nullptr;
}

HARNESS_API void bert_b200_harness_destroy(nvinfer1::IPluginV3* p)
{
    delete p;
}

HARNESS_API nvinfer1::IPluginV3* bert_b200_harness_clone(nvinfer1::IPluginV3* p)
{
    return p ? p->clone() : nullptr;
}

HARNESS_API nvinfer1::IPluginV3* bert_b200_harness_attach(nvinfer1::IPluginV3* p)
{
    auto* rt = capability<nvinfer1::IPluginV3OneRuntime>(p, nvinfer1::PluginCapabilityType::kRUNTIME);
    return rt ? rt->attachToContext(nullptr) : nullptr;
}

HARNESS_API int32_t bert_b200_harness_core_info(nvinfer1::IPluginV3* p, char const** name, char const** version, char const** ns)
{
    auto* core = capability<nvinfer1::IPluginV3OneCore>(p, nvinfer1::PluginCapabilityType::kCORE);
    if (!core)
        return 1;
    *name = core->getPluginName();
    *version = core->getPluginVersion();
    *ns = core->getPluginNamespace();
    return 0;
}

HARNESS_API int32_t bert_b200_harness_nb_outputs(nvinfer1::IPluginV3* p)
{
    auto* b = capability<nvinfer1::IPluginV3OneBuild>(p, nvinfer1::PluginCapabilityType::kBUILD);
    return b ? b->getNbOutputs() : -1;
}

HARNESS_API int32_t bert_b200_harness_supports_format(
    nvinfer1::IPluginV3* p, int32_t pos, nvinfer1::DynamicPluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs)
{
    auto* b = capability<nvinfer1::IPluginV3OneBuild>(p, nvinfer1::PluginCapabilityType::kBUILD);
    return b ? (b->supportsFormatCombination(pos, inOut, nbInputs, nbOutputs) ? 1 : 0) : -1;
}

// Input shapes are concrete Dims; output shapes come back as concrete Dims.
HARNESS_API int32_t bert_b200_harness_output_shapes(
    nvinfer1::IPluginV3* p, nvinfer1::Dims const* inputs, int32_t nbInputs, nvinfer1::Dims* outputs, int32_t nbOutputs)
{
    auto* b = capability<nvinfer1::IPluginV3OneBuild>(p, nvinfer1::PluginCapabilityType::kBUILD);
    if (!b || nbInputs > 8 || nbOutputs > 8)
        return 1;
    ExprBuilder eb;
    nvinfer1::DimsExprs in[8], out[8];
    for (int32_t i = 0; i < nbInputs; ++i)
    {
        in[i].nbDims = inputs[i].nbDims;
        for (int32_t k = 0; k < inputs[i].nbDims; ++k)
            in[i].d[k] = eb.constant(inputs[i].d[k]);
    }
    int32_t const st = b->getOutputShapes(in, nbInputs, nullptr, 0, out, nbOutputs, eb);
    if (st != 0)
        return st;
    for (int32_t i = 0; i < nbOutputs; ++i)
    {
        outputs[i].nbDims = out[i].nbDims;
        for (int32_t k = 0; k < out[i].nbDims; ++k)
            outputs[i].d[k] = out[i].d[k]->getConstantValue();
    }
    return 0;
}

HARNESS_API int32_t bert_b200_harness_output_types(
    nvinfer1::IPluginV3* p, int32_t* outTypes, int32_t nbOutputs, int32_t const* inTypes, int32_t nbInputs)
{
    auto* b = capability<nvinfer1::IPluginV3OneBuild>(p, nvinfer1::PluginCapabilityType::kBUILD);
    return b ? b->getOutputDataTypes(reinterpret_cast<nvinfer1::DataType*>(outTypes), nbOutputs,
                   reinterpret_cast<nvinfer1::DataType const*>(inTypes), nbInputs)
             : 1;
}

HARNESS_API int32_t bert_b200_harness_configure(nvinfer1::IPluginV3* p, nvinfer1::DynamicPluginTensorDesc const* in, int32_t nbInputs,
    nvinfer1::DynamicPluginTensorDesc const* out, int32_t nbOutputs)
{
    auto* b = capability<nvinfer1::IPluginV3OneBuild>(p, nvinfer1::PluginCapabilityType::kBUILD);
    return b ? b->configurePlugin(in, nbInputs, out, nbOutputs) : 1;
}

HARNESS_API int64_t bert_b200_harness_workspace_size(nvinfer1::IPluginV3* p, nvinfer1::DynamicPluginTensorDesc const* in,
    int32_t nbInputs, nvinfer1::DynamicPluginTensorDesc const* out, int32_t nbOutputs)
{
    auto* b = capability<nvinfer1::IPluginV3OneBuild>(p, nvinfer1::PluginCapabilityType::kBUILD);
    return b ? static_cast<int64_t>(b->getWorkspaceSize(in, nbInputs, out, nbOutputs)) : -1;
}

HARNESS_API int32_t bert_b200_harness_on_shape_change(nvinfer1::IPluginV3* p, nvinfer1::PluginTensorDesc const* in, int32_t nbInputs,
    nvinfer1::PluginTensorDesc const* out, int32_t nbOutputs)
{
    auto* rt = capability<nvinfer1::IPluginV3OneRuntime>(p, nvinfer1::PluginCapabilityType::kRUNTIME);
    return rt ? rt->onShapeChange(in, nbInputs, out, nbOutputs) : 1;
}

HARNESS_API int32_t bert_b200_harness_enqueue(nvinfer1::IPluginV3* p, nvinfer1::PluginTensorDesc const* inDesc,
    nvinfer1::PluginTensorDesc const* outDesc, void const* const* inputs, void* const* outputs, void* workspace, void* stream)
{
    auto* rt = capability<nvinfer1::IPluginV3OneRuntime>(p, nvinfer1::PluginCapabilityType::kRUNTIME);
    return rt ? rt->enqueue(inDesc, outDesc, inputs, outputs, workspace, static_cast<cudaStream_t>(stream)) : 1;
}

HARNESS_API nvinfer1::PluginFieldCollection const* bert_b200_harness_serialize(nvinfer1::IPluginV3* p)
{
    auto* rt = capability<nvinfer1::IPluginV3OneRuntime>(p, nvinfer1::PluginCapabilityType::kRUNTIME);
    return rt ? rt->getFieldsToSerialize() : nullptr;
}

// ---- legacy IPluginV2DynamicExt objects: the calls the builder and the runtime make on them ----------------------

using LegacyPlugin = nvinfer1::IPluginV2DynamicExt;

HARNESS_API LegacyPlugin* bert_b200_harness_legacy_create(char const* name, char const* version, nvinfer1::PluginFieldCollection const* fc)
{
    auto* c = legacyCreator(name, version);
    return c ? static_cast<LegacyPlugin*>(c->createPlugin("harness_layer", fc)) : nullptr;
}

HARNESS_API LegacyPlugin* bert_b200_harness_legacy_deserialize(char const* name, char const* version, void const* data, int64_t length)
{
    auto* c = legacyCreator(name, version);
    return c ? static_cast<LegacyPlugin*>(c->deserializePlugin("harness_layer", data, static_cast<size_t>(length))) : nullptr;
}

HARNESS_API void bert_b200_harness_legacy_destroy(LegacyPlugin* p)
{
    if (p)
        p->destroy();
}

HARNESS_API LegacyPlugin* bert_b200_harness_legacy_clone(LegacyPlugin* p)
{
    return p ? p->clone() : nullptr;
}

HARNESS_API int32_t bert_b200_harness_legacy_info(LegacyPlugin* p, char const** type, char const** version, char const** ns)
{
    if (!p)
        return 1;
    *type = p->getPluginType();
    *version = p->getPluginVersion();
    *ns = p->getPluginNamespace();
    return 0;
}

HARNESS_API int32_t bert_b200_harness_legacy_nb_outputs(LegacyPlugin* p)
{
    return p ? p->getNbOutputs() : -1;
}

HARNESS_API int32_t bert_b200_harness_legacy_supports_format(
    LegacyPlugin* p, int32_t pos, nvinfer1::PluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs)
{
    return p ? (p->supportsFormatCombination(pos, inOut, nbInputs, nbOutputs) ? 1 : 0) : -1;
}

HARNESS_API int32_t bert_b200_harness_legacy_output_dims(
    LegacyPlugin* p, int32_t outputIndex, nvinfer1::Dims const* inputs, int32_t nbInputs, nvinfer1::Dims* output)
{
    if (!p || nbInputs > 8)
        return 1;
    ExprBuilder eb;
    nvinfer1::DimsExprs in[8];
    for (int32_t i = 0; i < nbInputs; ++i)
    {
        in[i].nbDims = inputs[i].nbDims;
        for (int32_t k = 0; k < inputs[i].nbDims; ++k)
            in[i].d[k] = eb.constant(inputs[i].d[k]);
    }
    nvinfer1::DimsExprs const out = p->getOutputDimensions(outputIndex, in, nbInputs, eb);
    if (out.nbDims < 0)
        return 2;
    output->nbDims = out.nbDims;
    for (int32_t k = 0; k < out.nbDims; ++k)
        output->d[k] = out.d[k]->getConstantValue();
    return 0;
}

HARNESS_API int32_t bert_b200_harness_legacy_output_type(LegacyPlugin* p, int32_t index, int32_t const* inTypes, int32_t nbInputs)
{
    return p ? static_cast<int32_t>(p->getOutputDataType(index, reinterpret_cast<nvinfer1::DataType const*>(inTypes), nbInputs)) : -1;
}

HARNESS_API int32_t bert_b200_harness_legacy_configure(LegacyPlugin* p, nvinfer1::DynamicPluginTensorDesc const* in, int32_t nbInputs,
    nvinfer1::DynamicPluginTensorDesc const* out, int32_t nbOutputs)
{
    if (!p)
        return 1;
    p->configurePlugin(in, nbInputs, out, nbOutputs);
    return 0;
}

HARNESS_API int64_t bert_b200_harness_legacy_workspace_size(LegacyPlugin* p, nvinfer1::PluginTensorDesc const* in, int32_t nbInputs,
    nvinfer1::PluginTensorDesc const* out, int32_t nbOutputs)
{
    return p ? static_cast<int64_t>(p->getWorkspaceSize(in, nbInputs, out, nbOutputs)) : -1;
}

HARNESS_API int32_t bert_b200_harness_legacy_enqueue(LegacyPlugin* p, nvinfer1::PluginTensorDesc const* inDesc,
    nvinfer1::PluginTensorDesc const* outDesc, void const* const* inputs, void* const* outputs, void* workspace, void* stream)
{
    return p ? p->enqueue(inDesc, outDesc, inputs, outputs, workspace, static_cast<cudaStream_t>(stream)) : 1;
}

HARNESS_API int64_t bert_b200_harness_legacy_serialization_size(LegacyPlugin* p)
{
    return p ? static_cast<int64_t>(p->getSerializationSize()) : -1;
}

HARNESS_API int32_t bert_b200_harness_legacy_serialize(LegacyPlugin* p, void* buffer)
{
    if (!p || !buffer)
        return 1;
    p->serialize(buffer);
    return 0;
}

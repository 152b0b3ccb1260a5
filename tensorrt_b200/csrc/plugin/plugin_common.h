// Shared pieces of the IPluginV3 adapters: error convention, field parsing, weight storage.
//
// The adapters keep the reference's plugin surface (creator names, versions, PluginFields, I/O ranks and
// formats) and forward enqueue() to the C ABI of libbert_b200.so. They compile against the public TensorRT
// headers only and do not link libnvinfer: the registry and logger are looked up at run time.
#pragma once

#include <NvInferRuntime.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstring>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

#include "bert_b200.h"

namespace bert_b200_plugin
{
using namespace nvinfer1;

// ref: plugin/common/plugin.h:34-41
enum pluginStatus_t : int32_t
{
    STATUS_SUCCESS = 0,
    STATUS_FAILURE = 1,
    STATUS_BAD_PARAM = 2,
    STATUS_NOT_SUPPORTED = 3,
    STATUS_NOT_INITIALIZED = 4
};

// Dimension roles of the fixed-length tensors (ref: plugin/common/bertCommon.h:55-57)
constexpr int32_t SDIM = 0;
constexpr int32_t BDIM = 1;
constexpr int32_t HDIM = 2;

// Packed-mask row sizes (ref: plugin/common/bertCommon.h:71-84)
constexpr int32_t kUnfusedMaskSize = 1;
constexpr int32_t kPackedMaskSize128 = 4 * (2 * 2 * 32);
constexpr int32_t kPackedMaskSize384 = 24 * (1 * 8 * 32);

// ref: plugin/common/bertCommon.h:114-140 (getMHAMaskPackedSize); the SM test is always true on sm_100a
inline int32_t mhaMaskPackedSize(DataType mhaType, int64_t S)
{
    bool const precisionOk = mhaType == DataType::kINT8 || mhaType == DataType::kHALF;
    if (precisionOk && (S == 64 || S == 96 || S == 128))
        return kPackedMaskSize128;
    if (precisionOk && S == 384)
        return kPackedMaskSize384;
    return kUnfusedMaskSize;
}

// warps_m, warps_n of the packed mask for sequence length S (ref: plugin/embLayerNormPlugin/embLayerNormPlugin.cpp:308-318)
inline bool packedMaskWarps(int64_t S, uint32_t& warpsM, uint32_t& warpsN)
{
    if (S == 64 || S == 96 || S == 128)
    {
        warpsM = 2;
        warpsN = 2;
        return true;
    }
    if (S == 384)
    {
        warpsM = 1;
        warpsN = 8;
        return true;
    }
    return false;
}

struct PluginError : std::runtime_error
{
    using std::runtime_error::runtime_error;
};

#define PLG_VALIDATE(cond)                                                                                             \
    do                                                                                                                 \
    {                                                                                                                  \
        if (!(cond))                                                                                                   \
            throw ::bert_b200_plugin::PluginError(std::string("validation failed: ") + #cond + " (" + __FILE__ + ":"   \
                + std::to_string(__LINE__) + ")");                                                                     \
    } while (0)

// Reports through the ILogger given to initLibNvInferPlugins / found by the ILoggerFinder, else stderr.
void logMessage(ILogger::Severity severity, char const* fmt, ...);
void setLogger(ILogger* logger);
// No exception crosses the plugin boundary: every API method catches and calls this.
void caughtError(std::exception const& e);

inline int64_t volume(Dims const& d)
{
    int64_t v = 1;
    for (int32_t i = 0; i < d.nbDims; ++i)
        v *= d.d[i];
    return v;
}

inline PluginField const* findField(PluginFieldCollection const& fc, char const* name)
{
    for (int32_t i = 0; i < fc.nbFields; ++i)
        if (fc.fields[i].name && std::strcmp(fc.fields[i].name, name) == 0)
            return &fc.fields[i];
    return nullptr;
}

// ref: plugin/common/plugin.cpp (validateRequiredAttributesExist)
inline void requireFields(PluginFieldCollection const& fc, std::initializer_list<char const*> names)
{
    for (char const* n : names)
        if (!findField(fc, n))
            throw PluginError(std::string("PluginFieldCollection missing required field: {") + n + "}");
}

inline bool getInt(PluginFieldCollection const& fc, char const* name, int32_t& out)
{
    PluginField const* f = findField(fc, name);
    if (!f || !f->data)
        return false;
    PLG_VALIDATE(f->type == PluginFieldType::kINT32 && f->length >= 1);
    out = static_cast<int32_t const*>(f->data)[0];
    return true;
}

inline bool getFloat(PluginFieldCollection const& fc, char const* name, float& out)
{
    PluginField const* f = findField(fc, name);
    if (!f || !f->data)
        return false;
    PLG_VALIDATE(f->type == PluginFieldType::kFLOAT32 && f->length >= 1);
    out = static_cast<float const*>(f->data)[0];
    return true;
}

// Host copy of a weight tensor, converted to FP32 or FP16 (ref: WeightsWithOwnership::convertAndCopy,
// plugin/common/bertCommon.h:358-445).
struct HostWeights
{
    DataType type{DataType::kFLOAT};
    int64_t count{0};
    std::vector<uint8_t> bytes;

    bool empty() const
    {
        return count == 0;
    }
    void const* data() const
    {
        return bytes.data();
    }
    size_t sizeBytes() const
    {
        return bytes.size();
    }
    PluginFieldType fieldType() const
    {
        return type == DataType::kHALF ? PluginFieldType::kFLOAT16 : PluginFieldType::kFLOAT32;
    }
    // src is FP32 or FP16 plugin-field data
    void assign(PluginField const& f, DataType dst);
    void assign(void const* src, DataType srcType, int64_t n, DataType dst);
    float at(int64_t i) const;
};

// Device copy owned by a plugin object (ref: copyToDevice, plugin/common/bertCommon.h:447-457). Creating a
// plugin on a machine without a GPU leaves the pointer null; enqueue then reports an error.
struct DeviceBuffer
{
    void* ptr{nullptr};
    DeviceBuffer() = default;
    DeviceBuffer(DeviceBuffer const&) = delete;
    DeviceBuffer& operator=(DeviceBuffer const&) = delete;
    ~DeviceBuffer();
    bool upload(void const* host, size_t bytes);
};

// Common base of all adapters.
class PluginBase : public IPluginV3, public IPluginV3OneCore, public IPluginV3OneBuild, public IPluginV3OneRuntime
{
public:
    PluginBase(std::string layerName, char const* pluginName, char const* version)
        : mLayerName(std::move(layerName))
        , mPluginName(pluginName)
        , mVersion(version)
    {
    }
    ~PluginBase() override = default;

    IPluginCapability* getCapabilityInterface(PluginCapabilityType type) noexcept override;
    AsciiChar const* getPluginName() const noexcept override
    {
        return mPluginName;
    }
    AsciiChar const* getPluginVersion() const noexcept override
    {
        return mVersion;
    }
    AsciiChar const* getPluginNamespace() const noexcept override
    {
        return mNamespace.c_str();
    }
    void setPluginNamespace(char const* ns)
    {
        mNamespace = ns ? ns : "";
    }

    int32_t configurePlugin(DynamicPluginTensorDesc const*, int32_t, DynamicPluginTensorDesc const*, int32_t) noexcept override
    {
        return STATUS_SUCCESS;
    }
    size_t getWorkspaceSize(DynamicPluginTensorDesc const*, int32_t, DynamicPluginTensorDesc const*, int32_t) const noexcept override
    {
        return 0;
    }
    int32_t onShapeChange(PluginTensorDesc const*, int32_t, PluginTensorDesc const*, int32_t) noexcept override
    {
        return STATUS_SUCCESS;
    }
    IPluginV3* attachToContext(IPluginResourceContext*) noexcept override
    {
        return clone();
    }
    PluginFieldCollection const* getFieldsToSerialize() noexcept override;

protected:
    // Appends the fields that reproduce this object through createPlugin(..., kRUNTIME).
    virtual void serialize(std::vector<PluginField>& fields) = 0;

    std::string mLayerName;
    std::string mNamespace;
    char const* mPluginName;
    char const* mVersion;
    std::vector<PluginField> mFields;
    PluginFieldCollection mFC{};
};

class CreatorBase : public IPluginCreatorV3One
{
public:
    CreatorBase(char const* name, char const* version, std::vector<PluginField> attributes)
        : mName(name)
        , mVersion(version)
        , mAttributes(std::move(attributes))
    {
        mFC.nbFields = static_cast<int32_t>(mAttributes.size());
        mFC.fields = mAttributes.data();
    }
    AsciiChar const* getPluginName() const noexcept override
    {
        return mName;
    }
    AsciiChar const* getPluginVersion() const noexcept override
    {
        return mVersion;
    }
    AsciiChar const* getPluginNamespace() const noexcept override
    {
        return mNamespace.c_str();
    }
    PluginFieldCollection const* getFieldNames() noexcept override
    {
        return &mFC;
    }
    IPluginV3* createPlugin(AsciiChar const* name, PluginFieldCollection const* fc, TensorRTPhase phase) noexcept override;
    void setPluginNamespace(char const* ns)
    {
        mNamespace = ns ? ns : "";
    }

protected:
    virtual PluginBase* make(char const* name, PluginFieldCollection const& fc, TensorRTPhase phase) = 0;

    char const* mName;
    char const* mVersion;
    std::string mNamespace;
    std::vector<PluginField> mAttributes;
    PluginFieldCollection mFC{};
};

// Every creator of this library, in registration order.
std::vector<CreatorBase*> const& allCreators();

// The creators of the legacy IPluginV2DynamicExt versions (legacy_plugins.cpp), each an nvinfer1::IPluginCreator.
std::vector<nvinfer1::IPluginCreatorInterface*> const& allLegacyCreators();

} // namespace bert_b200_plugin

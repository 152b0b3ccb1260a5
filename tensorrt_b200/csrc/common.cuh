// Shared host/device helpers for the sm_100a BERT kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "bert_b200.h"

namespace b200
{

// ---- host-side error plumbing -------------------------------------------------------------
// No exception crosses the C ABI: every failure is a status code plus a thread-local message
// (the reference logs through ILogger and returns nullptr / STATUS_FAILURE,
// plugin/vc/checkMacrosPlugin.h:198-201, and may exit the process on assertion; this library never exits).
void setLastError(char const* fmt, ...);
char const* getLastError();

#define B200_FAIL(code, ...)                                                                                           \
    do                                                                                                                 \
    {                                                                                                                  \
        ::b200::setLastError(__VA_ARGS__);                                                                             \
        return (code);                                                                                                 \
    } while (0)

#define B200_REQUIRE(cond, ...)                                                                                        \
    do                                                                                                                 \
    {                                                                                                                  \
        if (!(cond))                                                                                                   \
        {                                                                                                              \
            ::b200::setLastError(__VA_ARGS__);                                                                         \
            return BERT_B200_BAD_PARAM;                                                                                \
        }                                                                                                              \
    } while (0)

inline int32_t checkLaunch(char const* what)
{
    cudaError_t const e = cudaPeekAtLastError();
    if (e != cudaSuccess)
    {
        setLastError("%s: %s", what, cudaGetErrorString(e));
        return BERT_B200_CUDA_ERROR;
    }
    return BERT_B200_OK;
}

inline bool aligned16(void const* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// Number of SMs of the current device (cached per device id).
int32_t smCount();

// Whether kernels are launched with programmatic stream serialisation (on unless BERT_B200_PDL=0): a kernel that
// follows another one in its stream may then start - set up its barriers, allocate tensor memory, fetch descriptors -
// while the earlier grid drains; it calls gridDependencyWait() before it touches global memory.
bool dependentLaunchEnabled();

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launchDependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependentLaunchEnabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

#ifdef __CUDACC__
// ---- device helpers -----------------------------------------------------------------------

// Programmatic dependent launch: let the next kernel of the stream start its set-up now ...
__device__ __forceinline__ void gridDependencyLaunch()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// ... and wait until the grids this one depends on have completed and their writes are visible. Every thread calls it
// before its first access to global memory; a no-op for a kernel launched without the attribute.
__device__ __forceinline__ void gridDependencyWait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float warpSum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warpMax(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// 128-bit global load through the read-only path, no L1 allocation (streamed once).
__device__ __forceinline__ uint4 ldgStream(void const* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// 128-bit global load kept in L1/L2 (parameters, re-used rows).
__device__ __forceinline__ uint4 ldgKeep(void const* p)
{
    return __ldg(reinterpret_cast<uint4 const*>(p));
}

__device__ __forceinline__ void stgStream(void* p, uint4 v)
{
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

// 64-bit forms of the two above (rows whose length is a multiple of 8 bytes but fills 16-byte chunks unevenly).
__device__ __forceinline__ uint2 ldgStream8(void const* p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ void stgStream8(void* p, uint2 v)
{
    asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

__device__ __forceinline__ void unpackHalf8(uint4 const& v, float (&f)[8])
{
    __half2 const* h = reinterpret_cast<__half2 const*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
        float2 const t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ uint4 packHalf8(float const (&f)[8])
{
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

// INT8 <-> FP32 without the conversion unit. cvt.f32.s32 / cvt.rni.sat.s8.f32 run at a sixteenth of the FMA rate and
// bound every INT8 kernel here; the same results come from the integer/FMA pipes:
//   byte -> float : flip the sign bit (b + 128 in 0..255), drop it into the low mantissa byte of 2^23 (one PRMT per
//                   value) and subtract 2^23 + 128 (exact).
//   float -> byte : clamp to [-128, 127], add 1.5 * 2^23 (the FP32 adder rounds to nearest even, like cvt.rni), take
//                   the low byte.
__device__ __forceinline__ void unpackChar4(uint32_t w, float (&f)[4])
{
    uint32_t const u = w ^ 0x80808080u;
    constexpr float kBias = 8388736.f; // 2^23 + 128
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - kBias;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - kBias;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - kBias;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - kBias;
}

// Round-to-nearest-even, saturate to [-128,127], pack four values into one word
// (same result as the reference's float4_to_char4, plugin/common/common.cuh:482-504).
__device__ __forceinline__ uint32_t packChar4(float a, float b, float c, float d)
{
    constexpr float kMagic = 12582912.f; // 1.5 * 2^23
    uint32_t const ua = __float_as_uint(fminf(fmaxf(a, -128.f), 127.f) + kMagic);
    uint32_t const ub = __float_as_uint(fminf(fmaxf(b, -128.f), 127.f) + kMagic);
    uint32_t const uc = __float_as_uint(fminf(fmaxf(c, -128.f), 127.f) + kMagic);
    uint32_t const ud = __float_as_uint(fminf(fmaxf(d, -128.f), 127.f) + kMagic);
    return __byte_perm(__byte_perm(ua, ub, 0x0040), __byte_perm(uc, ud, 0x0040), 0x5410);
}

// Same with the output scale folded into the rounding step: the values are clamped to [lo, hi] = [-128 / s, 127 / s]
// first, then one FMA computes x * s + 1.5 * 2^23 (a single rounding, to nearest even).
__device__ __forceinline__ uint32_t packChar4Scaled(float a, float b, float c, float d, float s, float lo, float hi)
{
    constexpr float kMagic = 12582912.f; // 1.5 * 2^23
    uint32_t const ua = __float_as_uint(fmaf(fminf(fmaxf(a, lo), hi), s, kMagic));
    uint32_t const ub = __float_as_uint(fmaf(fminf(fmaxf(b, lo), hi), s, kMagic));
    uint32_t const uc = __float_as_uint(fmaf(fminf(fmaxf(c, lo), hi), s, kMagic));
    uint32_t const ud = __float_as_uint(fmaf(fminf(fmaxf(d, lo), hi), s, kMagic));
    return __byte_perm(__byte_perm(ua, ub, 0x0040), __byte_perm(uc, ud, 0x0040), 0x5410);
}

// Variant on the conversion unit: one multiply and one saturating convert per value (the unit runs at a quarter of the
// FMA rate but is otherwise idle in a GEMM epilogue, where issue slots are the scarce resource).
__device__ __forceinline__ uint32_t packChar4Cvt(float a, float b, float c, float d, float s)
{
    int32_t ia, ib, ic, id;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(ia) : "f"(a * s));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(ib) : "f"(b * s));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(ic) : "f"(c * s));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(id) : "f"(d * s));
    return __byte_perm(__byte_perm(ia, ib, 0x0040), __byte_perm(ic, id, 0x0040), 0x5410);
}

// ... and without the multiply, for values that are already on the INT8 grid's scale.
__device__ __forceinline__ uint32_t packChar4Cvt(float a, float b, float c, float d)
{
    int32_t ia, ib, ic, id;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(ia) : "f"(a));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(ib) : "f"(b));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(ic) : "f"(c));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(id) : "f"(d));
    return __byte_perm(__byte_perm(ia, ib, 0x0040), __byte_perm(ic, id, 0x0040), 0x5410);
}

__device__ __forceinline__ int8_t quantChar(float a)
{
    int32_t ia;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(ia) : "f"(a));
    return static_cast<int8_t>(ia);
}
#endif // __CUDACC__

} // namespace b200

// Host-side runtime pieces shared by all kernels: error text, device properties, status word.
#include "common.cuh"

#include <cstdlib>

#include <mutex>

namespace b200
{
namespace
{
thread_local char gLastError[512] = {0};
}

void setLastError(char const* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(gLastError, sizeof(gLastError), fmt, ap);
    va_end(ap);
}

char const* getLastError()
{
    return gLastError;
}

int32_t smCount()
{
    // One process may drive several GPUs; cache per device id.
    static std::mutex mtx;
    static int32_t cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return 148;
    std::lock_guard<std::mutex> lock(mtx);
    if (cache[dev] == 0)
    {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

bool dependentLaunchEnabled()
{
    static int const on = [] {
        char const* e = std::getenv("BERT_B200_PDL");
        return (e != nullptr && e[0] == '0') ? 0 : 1;
    }();
    return on != 0;
}

} // namespace b200

extern "C" int32_t bert_b200_version(void)
{
    return 100;
}

extern "C" char const* bert_b200_last_error(void)
{
    return b200::getLastError();
}

extern "C" int32_t bert_b200_read_status_word(void const* status_word, void* stream, uint32_t* value_host)
{
    B200_REQUIRE(status_word && value_host, "read_status_word: null pointer");
    auto s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(value_host, status_word, sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess)
        e = cudaStreamSynchronize(s);
    if (e != cudaSuccess)
        B200_FAIL(BERT_B200_CUDA_ERROR, "read_status_word: %s", cudaGetErrorString(e));
    return BERT_B200_OK;
}

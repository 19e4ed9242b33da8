// Library-wide state: last error, launch counter, per-device status word.
#include "common.cuh"
#include <cstdarg>
#include <map>
#include <mutex>
#include <utility>

namespace ts2 {

thread_local std::string g_last_error;
std::atomic<long long> g_launch_count{0};
static std::string g_global_error; // last error of any thread, for ts2_last_error(NULL)
static std::mutex g_err_mu;

int fail(int code, const char *fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    {
        std::lock_guard<std::mutex> lk(g_err_mu);
        g_global_error = buf;
    }
    return code;
}

const char *global_error()
{
    std::lock_guard<std::mutex> lk(g_err_mu);
    static thread_local std::string copy;
    copy = g_global_error;
    return copy.c_str();
}

int sm_count(int device)
{
    static int cached[16] = {};
    int &c = cached[device & 15];
    if (c == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0)
            v = 148;
        c = v;
    }
    return c;
}

int resident_blocks(int device, const void *kernel, int threads)
{
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, int> cache;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find({kernel, threads * 16 + (device & 15)});
    if (it != cache.end())
        return it->second;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1)
        n = 1;
    cache[{kernel, threads * 16 + (device & 15)}] = n;
    return n;
}

int32_t *device_status_word(int device)
{
    static int32_t *words[16] = {};
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    int32_t *&w = words[device & 15];
    if (!w) {
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(device);
        if (cudaMalloc(&w, 256) != cudaSuccess) {
            w = nullptr;
        } else {
            cudaMemset(w, 0, 256);
        }
        cudaSetDevice(prev);
    }
    return w;
}

int collect_device_status(int device)
{
    int32_t *words[2] = {device_status_word(device), static_status_word_if_ready(device)};
    int32_t seen[2] = {0, 0};
    for (int i = 0; i < 2; ++i) {
        if (!words[i])
            continue;
        TS2_CUDA(cudaMemcpy(&seen[i], words[i], sizeof(int32_t), cudaMemcpyDeviceToHost));
        if (seen[i])
            cudaMemset(words[i], 0, sizeof(int32_t));
    }
    if (seen[0] | seen[1])
        return fail(TS2_ERR_DEVICE_STATUS,
                    "device status word = 0x%x%s (bit0: a bounded wait in a kernel timed out, bit1: a kernel refused its arguments)",
                    seen[0] | seen[1], seen[1] ? " (raised by ts2_gemm_dw_noalloc)" : "");
    return TS2_OK;
}

} // namespace ts2

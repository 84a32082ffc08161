// Error plumbing and struct-size queries of the C ABI.

#include "fmb_common.cuh"

#include <atomic>
#include <mutex>
#include <set>
#include <string>
#include <utility>

namespace fmb {

namespace {
std::mutex g_mutex;
std::string g_error;
std::atomic<long long> g_launches{0};
}  // namespace

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char* what, cudaError_t err, const char* file, int line) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_error = std::string(what) + ": " + cudaGetErrorString(err) + " (" + file + ":" + std::to_string(line) + ")";
}

cudaError_t opt_in_shared_memory(const void* kernel, int bytes) {
    static std::mutex mutex;
    static std::set<std::pair<int, const void*>> done;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    std::lock_guard<std::mutex> lock(mutex);
    if (done.count({dev, kernel})) return cudaSuccess;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (err == cudaSuccess) done.insert({dev, kernel});
    return err;
}

void set_error_text(const char* text) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_error = text;
}

}  // namespace fmb

extern "C" FMB_API int fmb_version(void) { return 100; }

extern "C" FMB_API const char* fmb_last_error(void) {
    static thread_local std::string copy;
    std::lock_guard<std::mutex> lock(fmb::g_mutex);
    copy = fmb::g_error;
    return copy.c_str();
}

extern "C" FMB_API int fmb_sizeof(int which) {
    switch (which) {
        case 0: return (int)sizeof(fmb_nl_t);
        case 1: return (int)sizeof(fmb_model_t);
        case 2: return (int)sizeof(fmb_work_t);
        case 3: return (int)sizeof(fmb_langevin_t);
        default: return -1;
    }
}

extern "C" FMB_API long long fmb_launch_count(void) { return fmb::g_launches.load(); }

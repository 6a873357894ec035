// Error plumbing and small helpers of the d3gs_b200 C ABI.
#include <atomic>
#include <cstring>

#include "common.cuh"

namespace d3gs {

static thread_local char g_last_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

int32_t cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return D3GS_ERR_CUDA;
}

static std::atomic<uint32_t> g_hook_polls{0};
static std::atomic<int32_t> g_hook_hold{-1};
TestHooks test_hooks() { return TestHooks{g_hook_polls.load(), g_hook_hold.load()}; }

static std::atomic<uint64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

}  // namespace d3gs

extern "C" void d3gs_test_hooks(uint32_t poll_limit, int32_t hold) {
    d3gs::g_hook_polls.store(poll_limit);
    d3gs::g_hook_hold.store(hold);
}

extern "C" uint64_t d3gs_kernel_launch_count(void) { return d3gs::g_launches.load(std::memory_order_relaxed); }

extern "C" const char* d3gs_version(void) { return "d3gs_b200 0.1.0 (sm_100a)"; }

extern "C" size_t d3gs_last_error(char* buf, size_t cap) {
    const size_t len = strlen(d3gs::g_last_error);
    if (buf != nullptr && cap > 0) {
        const size_t n = len < cap - 1 ? len : cap - 1;
        memcpy(buf, d3gs::g_last_error, n);
        buf[n] = '\0';
    }
    return len;
}

// DeviceSort.get_higher_msb (d3sim/csrc/devsort.py:129-149): position of the highest set bit + 1
extern "C" int32_t d3gs_bit_length(uint32_t n) {
    int32_t b = 0;
    while (n) {
        ++b;
        n >>= 1;
    }
    return b;
}

extern "C" size_t d3gs_struct_size(int32_t which) {
    switch (which) {
        case 0: return sizeof(D3gsCamera);
        case 1: return sizeof(D3gsOpConfig);
        case 2: return sizeof(D3gsModel);
        case 3: return sizeof(D3gsModelGrad);
        case 4: return sizeof(D3gsSplatContext);
        case 5: return sizeof(D3gsAdamSegment);
        case 6: return sizeof(D3gsDensifyStats);
        case 7: return sizeof(D3gsPeerSet);
        case 8: return sizeof(D3gsRefineConfig);
        case 9: return sizeof(D3gsRefineMoments);
        case 10: return sizeof(D3gsPeerViews);
        default: return 0;
    }
}

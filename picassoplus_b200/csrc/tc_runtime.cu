// Per-device asynchronous error words and the wait budget of the tensor-core kernels.
#include "tc_runtime.cuh"
#include "tc_ptx.cuh"

#include <atomic>
#include <mutex>

namespace pb {
namespace tc {

constexpr int MAX_DEVICES = 64;
static int* g_words = nullptr;             // MAX_DEVICES ints, pinned + mapped + portable
static std::mutex g_mu;
static std::atomic<int> g_budget{ptx::WAIT_BUDGET_KCLOCKS};
static std::atomic<int> g_skip_filter{0};

static int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) dev = 0;
    return dev;
}

int* async_error_word() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_words) {
        int* p = nullptr;
        if (cudaHostAlloc((void**)&p, sizeof(int) * MAX_DEVICES, cudaHostAllocMapped | cudaHostAllocPortable) !=
            cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        for (int i = 0; i < MAX_DEVICES; ++i) p[i] = 0;
        g_words = p;
    }
    return g_words + current_device();
}

int check_async_error(const char* where) {
    int* base = g_words;
    if (!base) return PB200_OK;
    const int code = *(volatile int*)(base + current_device());
    if (code != 0) {
        set_error("%s: an earlier tensor-core kernel of this library gave up waiting on this device (kernel %d: "
                  "1 facet2facet forward, 2 input gradient, 3 filter gradient, 4 pointwise fusion); the results of that call "
                  "are invalid. "
                  "pb200_clear_async_error() re-arms the device.", where, code);
        return PB200_ECUDA;
    }
    return PB200_OK;
}

int wait_budget_kclocks() { return g_budget.load(std::memory_order_relaxed); }
int test_skip_filter_stream() { return g_skip_filter.load(std::memory_order_relaxed); }

}  // namespace tc
}  // namespace pb

extern "C" {

int pb200_async_error(void) {
    int* base = pb::tc::g_words;
    return base ? *(volatile int*)(base + pb::tc::current_device()) : 0;
}

void pb200_clear_async_error(void) {
    int* base = pb::tc::g_words;
    if (base) *(volatile int*)(base + pb::tc::current_device()) = 0;
}

void pb200_set_wait_budget(int64_t clocks) {
    int k = clocks <= 0 ? pb::ptx::WAIT_BUDGET_KCLOCKS : (int)((clocks + 1023) >> 10);
    if (k < 1) k = 1;
    pb::tc::g_budget.store(k);
}

void pb200_test_silence_filter_stream(int on) { pb::tc::g_skip_filter.store(on ? 1 : 0); }

}  // extern "C"

// Error text, launch accounting, per-kernel CUDA-event timing and the shared
// fixed-order partial reduction.
#include "common.cuh"

#include <stdarg.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <string>
#include <vector>

namespace pb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
    return PB200_ECUDA;
}

static std::atomic<int64_t> g_launches{0};
static std::atomic<int> g_prof_on{0};

struct ProfPair { const char* name; cudaEvent_t a, b; };
static std::mutex g_prof_mu;
static std::vector<ProfPair> g_prof;

LaunchScope::LaunchScope(const char* n, cudaStream_t s) : name(n), stream(s), slot(nullptr) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (g_prof_on.load(std::memory_order_relaxed)) {
        ProfPair* p = new ProfPair{n, nullptr, nullptr};
        if (cudaEventCreate(&p->a) == cudaSuccess && cudaEventCreate(&p->b) == cudaSuccess) {
            cudaEventRecord(p->a, s);
            slot = p;
        } else {
            delete p;
        }
    }
}

LaunchScope::~LaunchScope() {
    if (slot) {
        ProfPair* p = (ProfPair*)slot;
        cudaEventRecord(p->b, stream);
        std::lock_guard<std::mutex> lk(g_prof_mu);
        g_prof.push_back(*p);
        delete p;
    }
}

int sm_count() {
    static int cached[64];
    static std::once_flag once;
    std::call_once(once, [] { memset(cached, 0, sizeof(cached)); });
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

__global__ void reduce_partials_kernel(const float* __restrict__ partial, int nparts, int64_t n,
                                       float* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (int b = 0; b < nparts; ++b) acc += partial[(int64_t)b * n + i];
    out[i] = acc;
}

// Many partials: 32 slices of them are summed side by side (each in ascending order, four loads in flight) and
// the 32 sums are added in slice order.
constexpr int RP_SLICES = 32, RP_WIDTH = 32;
__global__ void __launch_bounds__(RP_WIDTH * RP_SLICES)
reduce_partials_sliced_kernel(const float* __restrict__ partial, int nparts, int64_t n, float* __restrict__ out) {
    __shared__ float part[RP_SLICES][RP_WIDTH];
    const int64_t i = (int64_t)blockIdx.x * RP_WIDTH + threadIdx.x;
    const int y = threadIdx.y, per = (nparts + RP_SLICES - 1) / RP_SLICES;
    const int b0 = y * per, b1 = b0 + per < nparts ? b0 + per : nparts;
    float acc = 0.f;
    if (i < n) {
        int b = b0;
        for (; b + 4 <= b1; b += 4) {
            const float v0 = partial[(int64_t)b * n + i], v1 = partial[(int64_t)(b + 1) * n + i];
            const float v2 = partial[(int64_t)(b + 2) * n + i], v3 = partial[(int64_t)(b + 3) * n + i];
            acc += v0;
            acc += v1;
            acc += v2;
            acc += v3;
        }
        for (; b < b1; ++b) acc += partial[(int64_t)b * n + i];
    }
    part[y][threadIdx.x] = acc;
    __syncthreads();
    if (y == 0 && i < n) {
        float s = part[0][threadIdx.x];
        for (int k = 1; k < RP_SLICES; ++k) s += part[k][threadIdx.x];
        out[i] = s;
    }
}

int reduce_partials(const float* partial, int nparts, int64_t n, float* out, cudaStream_t stream) {
    if (n <= 0) return PB200_OK;
    if (nparts >= 256) {
        PB_LAUNCH("reduce_partials", reduce_partials_sliced_kernel, (unsigned)ceil_div(n, RP_WIDTH), dim3(RP_WIDTH, RP_SLICES), 0, stream,
                  partial, nparts, n, out);
        return PB200_OK;
    }
    PB_LAUNCH("reduce_partials", reduce_partials_kernel, (unsigned)ceil_div(n, 128), 128, 0, stream,
              partial, nparts, n, out);
    return PB200_OK;
}

}  // namespace pb

extern "C" {

int pb200_version(void) { return 100; }
const char* pb200_last_error(void) { return pb::g_err; }
int64_t pb200_launch_count(void) { return pb::g_launches.load(); }

void pb200_prof_enable(int on) { pb::g_prof_on.store(on ? 1 : 0); }

void pb200_prof_reset(void) {
    std::lock_guard<std::mutex> lk(pb::g_prof_mu);
    for (auto& p : pb::g_prof) { cudaEventDestroy(p.a); cudaEventDestroy(p.b); }
    pb::g_prof.clear();
}

int pb200_prof_read(pb200_prof_record* out, int cap) {
    std::lock_guard<std::mutex> lk(pb::g_prof_mu);
    std::vector<pb200_prof_record> recs;
    for (auto& p : pb::g_prof) {
        if (cudaEventSynchronize(p.b) != cudaSuccess) continue;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, p.a, p.b) != cudaSuccess) continue;
        size_t i = 0;
        for (; i < recs.size(); ++i)
            if (strncmp(recs[i].name, p.name, sizeof(recs[i].name) - 1) == 0) break;
        if (i == recs.size()) {
            pb200_prof_record r;
            memset(&r, 0, sizeof(r));
            strncpy(r.name, p.name, sizeof(r.name) - 1);
            recs.push_back(r);
        }
        recs[i].launches += 1;
        recs[i].total_ms += ms;
    }
    std::sort(recs.begin(), recs.end(),
              [](const pb200_prof_record& a, const pb200_prof_record& b) { return a.total_ms > b.total_ms; });
    int n = (int)recs.size();
    for (int i = 0; i < n && i < cap; ++i) out[i] = recs[i];
    return n;
}

}  // extern "C"

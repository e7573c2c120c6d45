// Shared plumbing of libpicasso_b200: status codes, per-thread error text, the launch
// wrapper (launch counter + optional CUDA-event bracketing) and small device helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/picasso_b200.h"

namespace pb {

void set_error(const char* fmt, ...);
int  cuda_fail(cudaError_t e, const char* what);

// Brackets one kernel launch: counts it and, when timing is enabled, records a CUDA event
// on the launch stream before and after it.
struct LaunchScope {
    const char* name;
    cudaStream_t stream;
    void* slot;
    LaunchScope(const char* name, cudaStream_t s);
    ~LaunchScope();
};

int sm_count();           // SMs of the current device (cached per device)

#define PB_REQUIRE(cond, code, ...)                      \
    do { if (!(cond)) { pb::set_error(__VA_ARGS__); return (code); } } while (0)

// launch + error check; `name` is the label the timing table reports
#define PB_LAUNCH(name, kern, grid, block, smem, stream, ...)                              \
    do {                                                                                   \
        { pb::LaunchScope _scope(name, stream);                                            \
          kern<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__); }                      \
        cudaError_t _e = cudaGetLastError();                                               \
        if (_e != cudaSuccess) return pb::cuda_fail(_e, name);                             \
    } while (0)

#define PB_CUDA(call)                                                                      \
    do { cudaError_t _e = (call); if (_e != cudaSuccess) return pb::cuda_fail(_e, #call); } while (0)

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline int pow2_ceil(int x) { int p = 1; while (p < x) p <<= 1; return p; }

// ---- vector helpers -------------------------------------------------------------------
__device__ __forceinline__ float4 ldg4(const float4* p) { return __ldg(p); }
__device__ __forceinline__ void fma4(float4& acc, const float4& a, const float4& b) {
    acc.x = fmaf(a.x, b.x, acc.x); acc.y = fmaf(a.y, b.y, acc.y);
    acc.z = fmaf(a.z, b.z, acc.z); acc.w = fmaf(a.w, b.w, acc.w);
}
__device__ __forceinline__ void fma4s(float4& acc, float s, const float4& b) {
    acc.x = fmaf(s, b.x, acc.x); acc.y = fmaf(s, b.y, acc.y);
    acc.z = fmaf(s, b.z, acc.z); acc.w = fmaf(s, b.w, acc.w);
}
__device__ __forceinline__ float4 mul4(const float4& a, const float4& b) {
    return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w);
}
__device__ __forceinline__ float4 scale4(const float4& a, float s) {
    return make_float4(a.x * s, a.y * s, a.z * s, a.w * s);
}
__device__ __forceinline__ void add4(float4& acc, const float4& a) {
    acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
}
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }

// The vectorised kernels give each item (a face or a vertex) to a team of TL threads
// (TL a power of two <= 32); a thread owns one float4 channel group of the item, and
// gridDim.y walks channel chunks of 32 groups (128 channels).
struct TeamGeom {
    int TL;            // threads per item
    int chunks;        // gridDim.y
    int teams;         // items per block (blockDim 256)
};
static inline TeamGeom team_geom(int CV) {
    TeamGeom g;
    g.TL = pow2_ceil(CV < 32 ? CV : 32);
    g.chunks = (int)ceil_div(CV, 32);
    g.teams = 256 / g.TL;
    return g;
}
static inline int persistent_blocks(int64_t items, int per_block, int blocks_per_sm) {
    int64_t need = ceil_div(items, per_block);
    int64_t cap = (int64_t)sm_count() * blocks_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

#define PB_DISPATCH_TL(TLv, ...)                                   \
    switch (TLv) {                                                 \
        case 1:  { constexpr int TL = 1;  __VA_ARGS__; } break;    \
        case 2:  { constexpr int TL = 2;  __VA_ARGS__; } break;    \
        case 4:  { constexpr int TL = 4;  __VA_ARGS__; } break;    \
        case 8:  { constexpr int TL = 8;  __VA_ARGS__; } break;    \
        case 16: { constexpr int TL = 16; __VA_ARGS__; } break;    \
        default: { constexpr int TL = 32; __VA_ARGS__; } break;    \
    }

// out[i] = sum_b partial[b*n + i], b ascending: the fixed-order second stage of every
// filter-gradient reduction.
int reduce_partials(const float* partial, int nparts, int64_t n, float* out, cudaStream_t stream);

}  // namespace pb

// Mesh pooling and unpooling over decimation clusters: max / average pool (fine -> coarse)
// and interpolation (coarse -> fine), forward and backward.  Every reduction is a pull over
// the cluster CSR (coarse vertex -> member fine vertices, ascending), every other kernel a
// plain gather: no floating-point atomics, no compare-and-swap loops, results independent of
// scheduling.  HBM-bound: one item = (vertex, float4 of channels), rows read 128 bits wide.
#include "common.cuh"

namespace pb {
namespace pool {

// item -> (row, channel group); VEC = 4: float4 items, VEC = 1: scalar items
template <int VEC> struct Vec;
template <> struct Vec<4> {
    using T = float4;
    static __device__ __forceinline__ T ld(const float* p, int64_t i) { return __ldg(reinterpret_cast<const float4*>(p) + i); }
    static __device__ __forceinline__ void st(float* p, int64_t i, const T& v) { reinterpret_cast<float4*>(p)[i] = v; }
};
template <> struct Vec<1> {
    using T = float;
    static __device__ __forceinline__ T ld(const float* p, int64_t i) { return __ldg(p + i); }
    static __device__ __forceinline__ void st(float* p, int64_t i, const T& v) { p[i] = v; }
};

__device__ __forceinline__ void upd(float& best, int& arg, float v, int m) { if (v > best) { best = v; arg = m; } }
__device__ __forceinline__ void set_zero(float& a) { a = 0.f; }
__device__ __forceinline__ void set_zero(float4& a) { a = zero4(); }
__device__ __forceinline__ float quot(float x, float c) { return x / c; }
__device__ __forceinline__ float4 quot(const float4& x, float c) { return make_float4(x.x / c, x.y / c, x.z / c, x.w / c); }
__device__ __forceinline__ void accum(float& a, float x) { a += x; }
__device__ __forceinline__ void accum(float4& a, const float4& x) { add4(a, x); }

// output[vo] = max over the cluster's members, maxIndex[vo] = the smallest member id that attains it
// (reference: max_pool3d_init / _forward / _index, mesh_pool3d_gpu.cu:20-88; ties there go to
// whichever thread writes last).  A coarse vertex without members gets 0 / index 0, the values
// the reference's zero-initialised outputs keep.
template <int VEC>
__global__ void max_pool_fwd_kernel(int64_t NvOut, int CVn, const float* __restrict__ in,
                                    const int32_t* __restrict__ rowptr, const int32_t* __restrict__ members,
                                    float* __restrict__ out, int32_t* __restrict__ max_index) {
    const int64_t total = NvOut * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t vo = i / CVn;
        const int c = (int)(i - vo * CVn);
        const int beg = rowptr[vo], end = rowptr[vo + 1];
        if (VEC == 4) {
            float4 best = zero4();
            int4 arg = make_int4(0, 0, 0, 0);
            if (beg < end) {
                const int m0 = members[beg];
                best = Vec<4>::ld(in, (int64_t)m0 * CVn + c);
                arg = make_int4(m0, m0, m0, m0);
                for (int e = beg + 1; e < end; ++e) {
                    const int m = members[e];
                    const float4 v = Vec<4>::ld(in, (int64_t)m * CVn + c);
                    upd(best.x, arg.x, v.x, m); upd(best.y, arg.y, v.y, m);
                    upd(best.z, arg.z, v.z, m); upd(best.w, arg.w, v.w, m);
                }
            }
            Vec<4>::st(out, i, best);
            reinterpret_cast<int4*>(max_index)[i] = arg;
        } else {
            float best = 0.f;
            int arg = 0;
            if (beg < end) {
                arg = members[beg];
                best = __ldg(in + (int64_t)arg * CVn + c);
                for (int e = beg + 1; e < end; ++e) {
                    const int m = members[e];
                    upd(best, arg, __ldg(in + (int64_t)m * CVn + c), m);
                }
            }
            out[i] = best;
            max_index[i] = arg;
        }
    }
}

// gradInput[maxIndex[vo,c], c] = gradOutput[vo,c] on a zeroed gradInput (reference:
// max_pool3d_backward, mesh_pool3d_gpu.cu:93-105).  Clusters are disjoint, so every target has one
// writer and plain stores suffice.
__global__ void max_pool_bwd_kernel(int64_t NvIn, int64_t NvOut, int C, const int32_t* __restrict__ max_index,
                                    const float* __restrict__ gout, float* __restrict__ gin) {
    const int64_t total = NvOut * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int vi = max_index[i];
        if (vi >= 0 && vi < NvIn) gin[(int64_t)vi * C + c] = gout[i];
    }
}

// The same gradient as a gather, for callers that hold the cluster structures: fine vertex v of cluster vo takes
// gradOutput[vo,c] where maxIndex[vo,c] == v, else 0. Whole rows are written once, in order, instead of a zero fill
// followed by 4-byte stores scattered over rows that have left the L2 (each of those is a read-modify-write of a
// sector in DRAM).
template <int VEC>
__global__ void max_pool_bwd_gather_kernel(int64_t NvIn, int CVn, const int32_t* __restrict__ max_index,
                                           const float* __restrict__ gout, const int32_t* __restrict__ key,
                                           float* __restrict__ gin) {
    const int64_t total = NvIn * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = i / CVn;
        const int c = (int)(i - v * CVn);
        const int vo = key[v];
        if (VEC == 4) {
            float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
            if (vo >= 0) {
                const int4 m = __ldg(reinterpret_cast<const int4*>(max_index) + (int64_t)vo * CVn + c);
                const float4 g = __ldg(reinterpret_cast<const float4*>(gout) + (int64_t)vo * CVn + c);
                r.x = m.x == v ? g.x : 0.f;
                r.y = m.y == v ? g.y : 0.f;
                r.z = m.z == v ? g.z : 0.f;
                r.w = m.w == v ? g.w : 0.f;
            }
            reinterpret_cast<float4*>(gin)[i] = r;
        } else {
            float r = 0.f;
            if (vo >= 0 && max_index[(int64_t)vo * CVn + c] == v) r = gout[(int64_t)vo * CVn + c];
            gin[i] = r;
        }
    }
}

// A coarse vertex without members records index 0 and the scatter hands its gradient to vertex 0: the gather
// cannot see it (no fine vertex has it as key), so those rows are stored afterwards.
__global__ void max_pool_bwd_empty_kernel(int64_t NvIn, int64_t NvOut, int C, const int32_t* __restrict__ rowptr,
                                          const int32_t* __restrict__ max_index, const float* __restrict__ gout,
                                          float* __restrict__ gin) {
    const int64_t vo = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vo >= NvOut || rowptr[vo] != rowptr[vo + 1]) return;
    for (int c = 0; c < C; ++c) {
        const int vi = max_index[vo * C + c];
        if (vi >= 0 && vi < NvIn) gin[(int64_t)vi * C + c] = gout[vo * C + c];
    }
}

// output[vo] = sum over members of input[m] / count, count = vtReplace[representative] + 1, terms
// added in ascending member order (reference: avg_pool3d_forward, mesh_pool3d_gpu.cu:112-132,
// which divides each term before its atomic add)
template <int VEC>
__global__ void avg_pool_fwd_kernel(int64_t NvIn, int64_t NvOut, int CVn, const float* __restrict__ in,
                                    const int32_t* __restrict__ vtReplace, const int32_t* __restrict__ rowptr,
                                    const int32_t* __restrict__ members, float* __restrict__ out) {
    const int64_t total = NvOut * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t vo = i / CVn;
        const int c = (int)(i - vo * CVn);
        const int beg = rowptr[vo], end = rowptr[vo + 1];
        typename Vec<VEC>::T acc;
        set_zero(acc);
        for (int e = beg; e < end; ++e) {
            const int m = members[e];
            const int rep = vtReplace[m];
            const int64_t mapid = rep < 0 ? -(int64_t)rep : m;
            const float count = (float)(vtReplace[mapid] + 1);
            accum(acc, quot(Vec<VEC>::ld(in, (int64_t)m * CVn + c), count));
        }
        Vec<VEC>::st(out, i, acc);
    }
}

// gradInput[v] = gradOutput[key[v]] / count for the members of a cluster, 0 for vertices outside
// every cluster (reference: avg_pool3d_backward, mesh_pool3d_gpu.cu:138-158)
template <int VEC>
__global__ void avg_pool_bwd_kernel(int64_t NvIn, int CVn, const float* __restrict__ gout,
                                    const int32_t* __restrict__ vtReplace, const int32_t* __restrict__ key,
                                    float* __restrict__ gin) {
    const int64_t total = NvIn * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = i / CVn;
        const int c = (int)(i - v * CVn);
        const int vo = key[v];
        typename Vec<VEC>::T r;
        set_zero(r);
        if (vo >= 0) {
            const int rep = vtReplace[v];
            const int64_t mapid = rep < 0 ? -(int64_t)rep : v;
            const float count = (float)(vtReplace[mapid] + 1);
            r = quot(Vec<VEC>::ld(gout, (int64_t)vo * CVn + c), count);
        }
        Vec<VEC>::st(gin, i, r);
    }
}

// output[v] = input[key[v]] for every fine vertex of a cluster, 0 elsewhere (reference:
// interpolate_forward, mesh_unpool3d_gpu.cu:5-26)
template <int VEC>
__global__ void unpool_fwd_kernel(int64_t NvFine, int CVn, const float* __restrict__ in, const int32_t* __restrict__ key,
                                  float* __restrict__ out) {
    const int64_t total = NvFine * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = i / CVn;
        const int c = (int)(i - v * CVn);
        const int vi = key[v];
        typename Vec<VEC>::T r;
        set_zero(r);
        if (vi >= 0) r = Vec<VEC>::ld(in, (int64_t)vi * CVn + c);
        Vec<VEC>::st(out, i, r);
    }
}

// gradInput[coarse] = sum over the cluster's members of gradOutput[m], ascending member order
// (reference: interpolate_backward, mesh_unpool3d_gpu.cu:29-46, float atomics there)
template <int VEC>
__global__ void unpool_bwd_kernel(int64_t NvCoarse, int CVn, const float* __restrict__ gout,
                                  const int32_t* __restrict__ rowptr, const int32_t* __restrict__ members,
                                  float* __restrict__ gin) {
    const int64_t total = NvCoarse * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t vo = i / CVn;
        const int c = (int)(i - vo * CVn);
        const int beg = rowptr[vo], end = rowptr[vo + 1];
        if (VEC == 4) {
            float4 acc = zero4();
            for (int e = beg; e < end; ++e) add4(acc, Vec<4>::ld(gout, (int64_t)members[e] * CVn + c));
            Vec<4>::st(gin, i, acc);
        } else {
            float acc = 0.f;
            for (int e = beg; e < end; ++e) acc += __ldg(gout + (int64_t)members[e] * CVn + c);
            gin[i] = acc;
        }
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool sizes_ok(int64_t a, int64_t b, int C) {
    return a >= 0 && b >= 0 && C > 0 && a < (1LL << 31) && b < (1LL << 31);
}

}  // namespace pool
}  // namespace pb

using namespace pb;
using namespace pb::pool;

#define PB_POOL_LAUNCH(label, kern, items, vec, ...)                                                    \
    do {                                                                                                \
        int grid_ = persistent_blocks((items), 256, 16);                                                \
        if (vec) PB_LAUNCH(label, kern<4>, grid_, 256, 0, stream, __VA_ARGS__);                         \
        else     PB_LAUNCH(label, kern<1>, grid_, 256, 0, stream, __VA_ARGS__);                         \
    } while (0)

extern "C" {

int pb200_mesh_max_pool_forward(int64_t NvIn, int64_t NvOut, int C, const float* input, const int32_t* rowptr,
                                const int32_t* members, float* output, int32_t* maxIndex, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(NvIn, NvOut, C), PB200_EINVAL, "mesh_max_pool_forward: bad sizes");
    if (NvOut == 0) return PB200_OK;
    PB_REQUIRE(rowptr && output && maxIndex && (NvIn == 0 || (input && members)), PB200_EINVAL,
               "mesh_max_pool_forward: null pointer");
    const bool vec = C % 4 == 0 && aligned16(input) && aligned16(output) && aligned16(maxIndex);
    const int CVn = vec ? C / 4 : C;
    PB_POOL_LAUNCH("mesh_max_pool_fwd", max_pool_fwd_kernel, NvOut * CVn, vec, NvOut, CVn, input, rowptr, members, output,
                   maxIndex);
    return PB200_OK;
}

int pb200_mesh_max_pool_backward(int64_t NvIn, int64_t NvOut, int C, const int32_t* maxIndex, const float* gradOutput,
                                 float* gradInput, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(NvIn, NvOut, C), PB200_EINVAL, "mesh_max_pool_backward: bad sizes");
    if (NvIn == 0) return PB200_OK;
    PB_REQUIRE(gradInput && (NvOut == 0 || (maxIndex && gradOutput)), PB200_EINVAL, "mesh_max_pool_backward: null pointer");
    PB_CUDA(cudaMemsetAsync(gradInput, 0, sizeof(float) * (size_t)NvIn * C, stream));
    if (NvOut == 0) return PB200_OK;
    PB_LAUNCH("mesh_max_pool_bwd", max_pool_bwd_kernel, persistent_blocks(NvOut * C, 256, 16), 256, 0, stream, NvIn, NvOut, C,
              maxIndex, gradOutput, gradInput);
    return PB200_OK;
}

int pb200_mesh_max_pool_backward_clusters(int64_t NvIn, int64_t NvOut, int C, const int32_t* maxIndex,
                                          const float* gradOutput, const int32_t* key, const int32_t* rowptr,
                                          float* gradInput, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(NvIn, NvOut, C), PB200_EINVAL, "mesh_max_pool_backward_clusters: bad sizes");
    if (NvIn == 0) return PB200_OK;
    PB_REQUIRE(gradInput && key && rowptr && (NvOut == 0 || (maxIndex && gradOutput)), PB200_EINVAL,
               "mesh_max_pool_backward_clusters: null pointer");
    const bool vec = C % 4 == 0 && aligned16(gradOutput) && aligned16(gradInput) && aligned16(maxIndex);
    const int CVn = vec ? C / 4 : C;
    PB_POOL_LAUNCH("mesh_max_pool_bwd", max_pool_bwd_gather_kernel, NvIn * CVn, vec, NvIn, CVn, maxIndex, gradOutput, key,
                   gradInput);
    if (NvOut > 0)
        PB_LAUNCH("mesh_max_pool_bwd_empty", max_pool_bwd_empty_kernel, (unsigned)ceil_div(NvOut, 256), 256, 0, stream, NvIn,
                  NvOut, C, rowptr, maxIndex, gradOutput, gradInput);
    return PB200_OK;
}

int pb200_mesh_avg_pool_forward(int64_t NvIn, int64_t NvOut, int C, const float* input, const int32_t* vtReplace,
                                const int32_t* rowptr, const int32_t* members, float* output, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(NvIn, NvOut, C), PB200_EINVAL, "mesh_avg_pool_forward: bad sizes");
    if (NvOut == 0) return PB200_OK;
    PB_REQUIRE(rowptr && output && (NvIn == 0 || (input && members && vtReplace)), PB200_EINVAL,
               "mesh_avg_pool_forward: null pointer");
    const bool vec = C % 4 == 0 && aligned16(input) && aligned16(output);
    const int CVn = vec ? C / 4 : C;
    PB_POOL_LAUNCH("mesh_avg_pool_fwd", avg_pool_fwd_kernel, NvOut * CVn, vec, NvIn, NvOut, CVn, input, vtReplace, rowptr,
                   members, output);
    return PB200_OK;
}

int pb200_mesh_avg_pool_backward(int64_t NvIn, int64_t NvOut, int C, const float* gradOutput, const int32_t* vtReplace,
                                 const int32_t* key, float* gradInput, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(NvIn, NvOut, C), PB200_EINVAL, "mesh_avg_pool_backward: bad sizes");
    if (NvIn == 0) return PB200_OK;
    PB_REQUIRE(gradInput && vtReplace && key && (NvOut == 0 || gradOutput), PB200_EINVAL,
               "mesh_avg_pool_backward: null pointer");
    const bool vec = C % 4 == 0 && aligned16(gradOutput) && aligned16(gradInput);
    const int CVn = vec ? C / 4 : C;
    PB_POOL_LAUNCH("mesh_avg_pool_bwd", avg_pool_bwd_kernel, NvIn * CVn, vec, NvIn, CVn, gradOutput, vtReplace, key,
                   gradInput);
    return PB200_OK;
}

int pb200_mesh_unpool_forward(int64_t NvCoarse, int64_t NvFine, int C, const float* input, const int32_t* key,
                              float* output, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(NvCoarse, NvFine, C), PB200_EINVAL, "mesh_unpool_forward: bad sizes");
    if (NvFine == 0) return PB200_OK;
    PB_REQUIRE(output && key && (NvCoarse == 0 || input), PB200_EINVAL, "mesh_unpool_forward: null pointer");
    const bool vec = C % 4 == 0 && aligned16(input) && aligned16(output);
    const int CVn = vec ? C / 4 : C;
    PB_POOL_LAUNCH("mesh_unpool_fwd", unpool_fwd_kernel, NvFine * CVn, vec, NvFine, CVn, input, key, output);
    return PB200_OK;
}

int pb200_mesh_unpool_backward(int64_t NvCoarse, int64_t NvFine, int C, const float* gradOutput, const int32_t* rowptr,
                               const int32_t* members, float* gradInput, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(NvCoarse, NvFine, C), PB200_EINVAL, "mesh_unpool_backward: bad sizes");
    if (NvCoarse == 0) return PB200_OK;
    PB_REQUIRE(gradInput && rowptr && (NvFine == 0 || (gradOutput && members)), PB200_EINVAL,
               "mesh_unpool_backward: null pointer");
    const bool vec = C % 4 == 0 && aligned16(gradOutput) && aligned16(gradInput);
    const int CVn = vec ? C / 4 : C;
    PB_POOL_LAUNCH("mesh_unpool_bwd", unpool_bwd_kernel, NvCoarse * CVn, vec, NvCoarse, CVn, gradOutput, rowptr, members,
                   gradInput);
    return PB200_OK;
}

}  // extern "C"

// vertex2facet: forward (pure gather) and backward (vertex-centred pull over the CSR that
// yields the input gradient and the filter gradient in one pass, no float atomics).
#include "common.cuh"

#include <mutex>

namespace pb {

// ------------------------------------------------------------------- forward, vectorised
// r == 1, C % 4 == 0.  A team of TL threads owns one face; a thread owns one float4 of
// channels.  HBM traffic per face: 12 B of indices, 16*CV B written; the three vertex rows
// are gathers that mostly hit L2 (every vertex row is shared by ~6 faces).
template <int TL>
__global__ void __launch_bounds__(256)
v2f_fwd_vec_kernel(int64_t Nf, int CV, const int32_t* __restrict__ face, const float4* __restrict__ in,
                   const float4* __restrict__ filt, float4* __restrict__ out) {
    const int lane = threadIdx.x % TL;
    const int team = threadIdx.x / TL;
    const int cg = blockIdx.y * 32 + lane;
    if (cg >= CV) return;
    const float4 f0 = filt[cg], f1 = filt[CV + cg], f2 = filt[2 * CV + cg];
    const int teams = blockDim.x / TL;
    for (int64_t f = (int64_t)blockIdx.x * teams + team; f < Nf; f += (int64_t)gridDim.x * teams) {
        int v0 = __ldg(face + 3 * f), v1 = __ldg(face + 3 * f + 1), v2 = __ldg(face + 3 * f + 2);
        float4 x0 = ldg4(in + (int64_t)v0 * CV + cg);
        float4 x1 = ldg4(in + (int64_t)v1 * CV + cg);
        float4 x2 = ldg4(in + (int64_t)v2 * CV + cg);
        float4 o = zero4();
        fma4(o, f0, x0);      // same k-ascending fused-multiply-add chain as the reference
        fma4(o, f1, x1);
        fma4(o, f2, x2);
        __stcs(out + f * CV + cg, o);
    }
}

// ---------------------------------------------------------------------- forward, generic
__global__ void v2f_fwd_generic_kernel(int64_t Nf, int C, int r, const int32_t* __restrict__ face,
                                       const float* __restrict__ in, const float* __restrict__ filt,
                                       float* __restrict__ out) {
    const int Cr = C * r;
    int64_t total = Nf * Cr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t f = i / Cr;
        int co = (int)(i - f * Cr);
        int c = co / r;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 3; ++k)
            acc = fmaf(__ldg(filt + k * Cr + co), __ldg(in + (int64_t)face[3 * f + k] * C + c), acc);
        out[i] = acc;
    }
}

// ------------------------------------------------------------------ backward, vectorised
// A team owns one vertex v: it loads input[v] once, walks the CSR row of v in ascending
// (face, corner) order, and for every incident corner (f,k) reads gradOutput[f]:
//     gradInput[v] += g * filter[k]            (fixed order -> deterministic)
//     gradFilter[k] += g * input[v]            (per-thread registers)
// The per-thread filter-gradient partials are summed over the teams of the block in team
// order and written to partial[blockIdx.x][3][C]; a second kernel adds the blocks in order.
template <int TL>
__global__ void __launch_bounds__(256, 4)
v2f_bwd_vec_kernel(int64_t Nv, int CV, const int32_t* __restrict__ rowptr, const int32_t* __restrict__ entries,
                   const float4* __restrict__ gout, const float4* __restrict__ in, const float4* __restrict__ filt,
                   float4* __restrict__ gin, float4* __restrict__ partial) {
    __shared__ float4 red[3][256];
    const int lane = threadIdx.x % TL;
    const int team = threadIdx.x / TL;
    const int teams = blockDim.x / TL;
    const int cg = blockIdx.y * 32 + lane;
    const bool active = cg < CV;
    float4 gf0 = zero4(), gf1 = zero4(), gf2 = zero4();
    if (active) {
        const float4 f0 = filt[cg], f1 = filt[CV + cg], f2 = filt[2 * CV + cg];
        for (int64_t v = (int64_t)blockIdx.x * teams + team; v < Nv; v += (int64_t)gridDim.x * teams) {
            int beg = __ldg(rowptr + v), end = __ldg(rowptr + v + 1);
            float4 acc = zero4();
            if (end > beg) {
                float4 x = ldg4(in + v * CV + cg);
                auto accumulate = [&](int ent, const float4& g) {
                    const int k = ent & 3;
                    const float4 fk = (k == 0) ? f0 : ((k == 1) ? f1 : f2);
                    fma4(acc, g, fk);
                    const float4 t = mul4(g, x);
                    if (k == 0) add4(gf0, t); else if (k == 1) add4(gf1, t); else add4(gf2, t);
                };
                // four gradOutput rows in flight at a time, added in entry order
                int e = beg;
                for (; e + 3 < end; e += 4) {
                    int ent[4];
                    float4 g[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) ent[u] = __ldg(entries + e + u);
#pragma unroll
                    for (int u = 0; u < 4; ++u) g[u] = ldg4(gout + (int64_t)(ent[u] >> 2) * CV + cg);
#pragma unroll
                    for (int u = 0; u < 4; ++u) accumulate(ent[u], g[u]);
                }
                for (; e + 1 < end; e += 2) {
                    const int ent0 = __ldg(entries + e), ent1 = __ldg(entries + e + 1);
                    const float4 g0 = ldg4(gout + (int64_t)(ent0 >> 2) * CV + cg);
                    const float4 g1 = ldg4(gout + (int64_t)(ent1 >> 2) * CV + cg);
                    accumulate(ent0, g0);
                    accumulate(ent1, g1);
                }
                if (e < end) {
                    const int ent = __ldg(entries + e);
                    accumulate(ent, ldg4(gout + (int64_t)(ent >> 2) * CV + cg));
                }
            }
            gin[v * CV + cg] = acc;
        }
    }
    red[0][threadIdx.x] = gf0; red[1][threadIdx.x] = gf1; red[2][threadIdx.x] = gf2;
    __syncthreads();
    if (team == 0 && active) {
        float4 s0 = zero4(), s1 = zero4(), s2 = zero4();
        for (int t = 0; t < teams; ++t) {
            add4(s0, red[0][t * TL + lane]); add4(s1, red[1][t * TL + lane]); add4(s2, red[2][t * TL + lane]);
        }
        float4* p = partial + (int64_t)blockIdx.x * 3 * CV;
        p[cg] = s0; p[CV + cg] = s1; p[2 * CV + cg] = s2;
    }
}

// --------------------------------------------------------------------- backward, generic
__global__ void v2f_bwd_input_generic_kernel(int64_t Nv, int C, int r, const int32_t* __restrict__ rowptr,
                                             const int32_t* __restrict__ entries, const float* __restrict__ gout,
                                             const float* __restrict__ filt, float* __restrict__ gin) {
    const int Cr = C * r;
    int64_t total = Nv * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t v = i / C;
        int c = (int)(i - v * C);
        int beg = rowptr[v], end = rowptr[v + 1];
        float acc = 0.f;
        for (int e = beg; e < end; ++e) {
            int ent = entries[e];
            int k = ent & 3;
            const float* g = gout + (int64_t)(ent >> 2) * Cr + c * r;
            const float* w = filt + k * Cr + c * r;
            for (int m = 0; m < r; ++m) acc = fmaf(__ldg(g + m), __ldg(w + m), acc);
        }
        gin[i] = acc;
    }
}

// thread = output channel co, block row = a contiguous chunk of faces walked in order
__global__ void v2f_bwd_filter_generic_kernel(int64_t Nf, int C, int r, int64_t faces_per_chunk,
                                              const int32_t* __restrict__ face, const float* __restrict__ in,
                                              const float* __restrict__ gout, float* __restrict__ partial) {
    const int Cr = C * r;
    int co = blockIdx.y * blockDim.x + threadIdx.x;
    if (co >= Cr) return;
    int c = co / r;
    int64_t f0 = (int64_t)blockIdx.x * faces_per_chunk;
    int64_t f1 = f0 + faces_per_chunk < Nf ? f0 + faces_per_chunk : Nf;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;
    for (int64_t f = f0; f < f1; ++f) {
        float g = __ldg(gout + f * Cr + co);
        a0 = fmaf(g, __ldg(in + (int64_t)face[3 * f] * C + c), a0);
        a1 = fmaf(g, __ldg(in + (int64_t)face[3 * f + 1] * C + c), a1);
        a2 = fmaf(g, __ldg(in + (int64_t)face[3 * f + 2] * C + c), a2);
    }
    float* p = partial + (int64_t)blockIdx.x * 3 * Cr;
    p[co] = a0; p[Cr + co] = a1; p[2 * Cr + co] = a2;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool vec_ok(int C, int r) { return r == 1 && C % 4 == 0; }

struct V2FBwdPlan { bool vec; int grid_x; int64_t faces_per_chunk; };
static V2FBwdPlan v2f_bwd_plan(int64_t Nf, int64_t Nv, int C, int r) {
    V2FBwdPlan p;
    p.vec = vec_ok(C, r);
    if (p.vec) {
        TeamGeom g = team_geom(C / 4);
        p.grid_x = persistent_blocks(Nv, g.teams, 8);
        p.faces_per_chunk = 0;
    } else {
        int64_t chunks = ceil_div(Nf, 64);
        int64_t cap = (int64_t)sm_count() * 8;
        if (chunks > cap) chunks = cap;
        if (chunks < 1) chunks = 1;
        p.faces_per_chunk = ceil_div(Nf > 0 ? Nf : 1, chunks);
        p.grid_x = (int)ceil_div(Nf > 0 ? Nf : 1, p.faces_per_chunk);
    }
    return p;
}

}  // namespace pb

using namespace pb;

extern "C" {

int pb200_vertex2facet_forward(int64_t Nf, int64_t Nv, int C, int r, const float* input, const float* filter,
                               const int32_t* face, float* output, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && Nv >= 0 && C > 0 && r > 0, PB200_EINVAL, "vertex2facet_forward: bad sizes");
    if (Nf == 0) return PB200_OK;
    PB_REQUIRE(input && filter && face && output, PB200_EINVAL, "vertex2facet_forward: null pointer");
    if (vec_ok(C, r) && aligned16(input) && aligned16(filter) && aligned16(output)) {
        int CV = C / 4;
        TeamGeom g = team_geom(CV);
        dim3 grid(persistent_blocks(Nf, g.teams, 8), g.chunks);
        PB_DISPATCH_TL(g.TL, PB_LAUNCH("v2f_fwd", v2f_fwd_vec_kernel<TL>, grid, 256, 0, stream, Nf, CV, face,
                                       (const float4*)input, (const float4*)filter, (float4*)output));
    } else {
        int grid = persistent_blocks(Nf * C * r, 256, 16);
        PB_LAUNCH("v2f_fwd_generic", v2f_fwd_generic_kernel, grid, 256, 0, stream, Nf, C, r, face, input, filter, output);
    }
    return PB200_OK;
}

size_t pb200_vertex2facet_backward_workspace_bytes(int64_t Nf, int64_t Nv, int C, int r) {
    if (Nf < 0 || Nv < 0 || C <= 0 || r <= 0) return 0;
    V2FBwdPlan p = v2f_bwd_plan(Nf, Nv, C, r);
    return align_up(sizeof(float) * (size_t)p.grid_x * 3 * C * r, 256);
}

int pb200_vertex2facet_backward(int64_t Nf, int64_t Nv, int C, int r, const float* gradOutput, const float* input,
                                const float* filter, const int32_t* face, const int32_t* rowptr,
                                const int32_t* entries, float* gradInput, float* gradFilter, void* workspace,
                                size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && Nv >= 0 && C > 0 && r > 0, PB200_EINVAL, "vertex2facet_backward: bad sizes");
    PB_REQUIRE(gradFilter && (Nv == 0 || (gradInput && rowptr && input)), PB200_EINVAL,
               "vertex2facet_backward: null pointer");
    const int Cr = C * r;
    if (Nf == 0 || Nv == 0) {
        PB_CUDA(cudaMemsetAsync(gradFilter, 0, sizeof(float) * 3 * Cr, stream));
        if (Nv > 0) PB_CUDA(cudaMemsetAsync(gradInput, 0, sizeof(float) * Nv * C, stream));
        return PB200_OK;
    }
    PB_REQUIRE(gradOutput && filter && face && entries, PB200_EINVAL, "vertex2facet_backward: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_vertex2facet_backward_workspace_bytes(Nf, Nv, C, r),
               PB200_EWORKSPACE, "vertex2facet_backward: workspace too small");
    V2FBwdPlan p = v2f_bwd_plan(Nf, Nv, C, r);
    float* partial = (float*)workspace;
    bool vec = p.vec && aligned16(gradOutput) && aligned16(input) && aligned16(filter) && aligned16(gradInput);
    if (vec) {
        int CV = C / 4;
        TeamGeom g = team_geom(CV);
        dim3 grid(p.grid_x, g.chunks);
        PB_DISPATCH_TL(g.TL, PB_LAUNCH("v2f_bwd", v2f_bwd_vec_kernel<TL>, grid, 256, 0, stream, Nv, CV, rowptr,
                                       entries, (const float4*)gradOutput, (const float4*)input,
                                       (const float4*)filter, (float4*)gradInput, (float4*)partial));
        return reduce_partials(partial, p.grid_x, 3 * Cr, gradFilter, stream);
    }
    // generic path (any C, r): plan for the non-vector layout even if only alignment failed
    V2FBwdPlan q = p;
    if (p.vec) {
        int64_t chunks = ceil_div(Nf, 64);
        int64_t cap = p.grid_x;            // the workspace was sized for p.grid_x partial rows
        if (chunks > cap) chunks = cap;
        q.faces_per_chunk = ceil_div(Nf, chunks);
        q.grid_x = (int)ceil_div(Nf, q.faces_per_chunk);
    }
    int gi = persistent_blocks(Nv * C, 256, 16);
    PB_LAUNCH("v2f_bwd_input_generic", v2f_bwd_input_generic_kernel, gi, 256, 0, stream, Nv, C, r, rowptr, entries,
              gradOutput, filter, gradInput);
    dim3 gridf(q.grid_x, (unsigned)ceil_div(Cr, 128));
    PB_LAUNCH("v2f_bwd_filter_generic", v2f_bwd_filter_generic_kernel, gridf, 128, 0, stream, Nf, C, r,
              q.faces_per_chunk, face, input, gradOutput, partial);
    return reduce_partials(partial, q.grid_x, 3 * Cr, gradFilter, stream);
}

}  // extern "C"

// ------------------------------------------------------------- allocation-free variant
// Some hosts of this library may not allocate device memory at the moment they call it:
// a plugin invoked inside a region the embedding framework has frozen (its allocator is
// locked or its pool already handed out), a real-time or signal-adjacent callback, or a
// process whose memory budget was fixed at start-up.  For them the filter-gradient
// partials of vertex2facet_backward live in a fixed array that is part of the loaded
// library image on every GPU (it costs PB200_STATIC_SCRATCH_BYTES of device memory per
// GPU from load until exit).
//
// In host code `g_v2f_bwd_static_scratch` is only a handle for the runtime; the device
// address must be asked for with cudaGetSymbolAddress, once per device, with that device
// current.
#define PB200_STATIC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char g_v2f_bwd_static_scratch[PB200_STATIC_SCRATCH_BYTES];

namespace pb {
static int static_scratch_for_current_device(void** out) {
    static void* cached[64] = {nullptr};
    static std::mutex mu;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    PB_REQUIRE(dev >= 0 && dev < 64, PB200_EINVAL, "vertex2facet_backward_static: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lk(mu);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_v2f_bwd_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_v2f_bwd_static_scratch)");
        PB_REQUIRE(p != nullptr, PB200_ECUDA, "vertex2facet_backward_static: null scratch address");
        cached[dev] = p;
    }
    *out = cached[dev];
    return PB200_OK;
}
}  // namespace pb

extern "C" {

size_t pb200_vertex2facet_backward_static_max_bytes(void) { return PB200_STATIC_SCRATCH_BYTES; }

int pb200_vertex2facet_backward_static(int64_t Nf, int64_t Nv, int C, int r, const float* gradOutput,
                                       const float* input, const float* filter, const int32_t* face,
                                       const int32_t* rowptr, const int32_t* entries, float* gradInput,
                                       float* gradFilter, void* stream_) {
    PB_REQUIRE(Nf >= 0 && Nv >= 0 && C > 0 && r > 0, PB200_EINVAL, "vertex2facet_backward_static: bad sizes");
    size_t need = pb200_vertex2facet_backward_workspace_bytes(Nf, Nv, C, r);
    PB_REQUIRE(need <= PB200_STATIC_SCRATCH_BYTES, PB200_EWORKSPACE,
               "vertex2facet_backward_static: this shape needs %zu bytes of scratch, the built-in array holds %u; "
               "use pb200_vertex2facet_backward with a caller-provided workspace",
               need, (unsigned)PB200_STATIC_SCRATCH_BYTES);
    // argument checks before the first-call set-up, so that a bad call never triggers it
    PB_REQUIRE(gradFilter && (Nf == 0 || (gradOutput && input && filter && face && rowptr && entries && gradInput)),
               PB200_EINVAL, "vertex2facet_backward_static: null pointer");
    void* scratch = nullptr;
    int rc = static_scratch_for_current_device(&scratch);
    if (rc != PB200_OK) return rc;
    // Every partial the second stage reads is written by the first stage of the same call,
    // so nothing in the array has to start at zero.
    return pb200_vertex2facet_backward(Nf, Nv, C, r, gradOutput, input, filter, face, rowptr, entries, gradInput,
                                       gradFilter, scratch, PB200_STATIC_SCRATCH_BYTES, stream_);
}

}  // extern "C"

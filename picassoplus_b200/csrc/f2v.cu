// facet2vertex: forward as a vertex-centred pull over the CSR (segmented sum in a fixed
// order, no atomics); backward as a face-centred gather that yields the input gradient
// and per-thread filter-gradient partials in one pass.
#include "common.cuh"

namespace pb {

// -------------------------------------------------------------------- forward, vectorised
// r == 1, C % 4 == 0.  Team per output vertex, thread per float4 of channels.  KT > 0: the
// filter column of the thread's channels lives in registers (K == KT); KT == 0: it is
// read from shared memory (any K).
template <int TL, int KT>
__global__ void __launch_bounds__(256)
f2v_fwd_vec_kernel(int64_t NvOut, int CV, int K, const int32_t* __restrict__ rowptr,
                   const int32_t* __restrict__ entries, const int32_t* __restrict__ nfCount,
                   const float* __restrict__ coeff, const float4* __restrict__ in,
                   const float4* __restrict__ filt, float4* __restrict__ out) {
    extern __shared__ float4 sfilt[];          // [K][32] when KT == 0
    const int lane = threadIdx.x % TL;
    const int team = threadIdx.x / TL;
    const int teams = blockDim.x / TL;
    const int cg = blockIdx.y * 32 + lane;
    const bool active = cg < CV;
    float4 rf[KT > 0 ? KT : 1];
    if (KT > 0) {
#pragma unroll
        for (int k = 0; k < KT; ++k) rf[k] = active ? filt[k * CV + cg] : zero4();
    } else {
        for (int i = threadIdx.x; i < K * 32; i += blockDim.x) {
            int k = i >> 5, l = i & 31;
            int g = blockIdx.y * 32 + l;
            sfilt[i] = g < CV ? filt[k * CV + g] : zero4();
        }
        __syncthreads();
    }
    if (!active) return;
    for (int64_t v = (int64_t)blockIdx.x * teams + team; v < NvOut; v += (int64_t)gridDim.x * teams) {
        int beg = __ldg(rowptr + v), end = __ldg(rowptr + v + 1);
        float4 acc = zero4();
        for (int e = beg; e < end; ++e) {
            int64_t f = __ldg(entries + e) >> 2;
            float4 x = ldg4(in + f * CV + cg);
            const float* cf = coeff + f * K;
            float4 w = zero4();
            if (KT > 0) {
#pragma unroll
                for (int k = 0; k < KT; ++k) fma4s(w, __ldg(cf + k), rf[k]);
            } else {
                for (int k = 0; k < K; ++k) fma4s(w, __ldg(cf + k), sfilt[k * 32 + lane]);
            }
            fma4(acc, w, x);
        }
        if (end > beg) {
            float nf = (float)__ldg(nfCount + v);
            acc = make_float4(acc.x / nf, acc.y / nf, acc.z / nf, acc.w / nf);
        }
        __stcs(out + v * CV + cg, acc);
    }
}

// ----------------------------------------------------------------------- forward, generic
__global__ void f2v_fwd_generic_kernel(int64_t NvOut, int C, int r, int K, const int32_t* __restrict__ rowptr,
                                       const int32_t* __restrict__ entries, const int32_t* __restrict__ nfCount,
                                       const float* __restrict__ coeff, const float* __restrict__ in,
                                       const float* __restrict__ filt, float* __restrict__ out) {
    const int Cr = C * r;
    int64_t total = NvOut * Cr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t v = i / Cr;
        int co = (int)(i - v * Cr);
        int c = co / r;
        int beg = rowptr[v], end = rowptr[v + 1];
        float acc = 0.f;
        for (int e = beg; e < end; ++e) {
            int64_t f = entries[e] >> 2;
            float w = 0.f;
            for (int k = 0; k < K; ++k) w = fmaf(__ldg(coeff + f * K + k), __ldg(filt + k * Cr + co), w);
            acc = fmaf(w, __ldg(in + f * C + c), acc);
        }
        out[i] = end > beg ? acc / (float)nfCount[v] : 0.f;
    }
}

// ------------------------------------------------------------------- backward, vectorised
// Team per face f.  gt = sum over the three corners of gradOutput[vo]/nfCount[vo];
// w = sum_k coeff[f,k]*filter[k];  gradInput[f] = gt*w;  gradFilter[k] += coeff[f,k]*x*gt.
// The filter is read from shared memory, the K filter-gradient accumulators are registers.
template <int TL, int KT>
__global__ void __launch_bounds__(256)
f2v_bwd_vec_kernel(int64_t Nf, int CV, const int32_t* __restrict__ face, const int32_t* __restrict__ vtMap,
                   const int32_t* __restrict__ nfCount, const float* __restrict__ coeff,
                   const float4* __restrict__ in, const float4* __restrict__ filt, const float4* __restrict__ gout,
                   float4* __restrict__ gin, float4* __restrict__ partial) {
    extern __shared__ float4 smem[];           // [KT][32] filter, then [256] reduction slots
    float4* sfilt = smem;
    float4* red = smem + KT * 32;
    const int lane = threadIdx.x % TL;
    const int team = threadIdx.x / TL;
    const int teams = blockDim.x / TL;
    const int cg = blockIdx.y * 32 + lane;
    const bool active = cg < CV;
    for (int i = threadIdx.x; i < KT * 32; i += blockDim.x) {
        int k = i >> 5, l = i & 31;
        int g = blockIdx.y * 32 + l;
        sfilt[i] = g < CV ? filt[k * CV + g] : zero4();
    }
    __syncthreads();
    float4 gf[KT];
#pragma unroll
    for (int k = 0; k < KT; ++k) gf[k] = zero4();
    if (active) {
        for (int64_t f = (int64_t)blockIdx.x * teams + team; f < Nf; f += (int64_t)gridDim.x * teams) {
            float4 gt = zero4();
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                int vi = __ldg(face + 3 * f + j);
                int vo = vtMap ? __ldg(vtMap + vi) : vi;
                if (vo >= 0) {
                    float nf = (float)__ldg(nfCount + vo);
                    float4 g = ldg4(gout + (int64_t)vo * CV + cg);
                    gt.x += g.x / nf; gt.y += g.y / nf; gt.z += g.z / nf; gt.w += g.w / nf;
                }
            }
            float4 x = ldg4(in + f * CV + cg);
            float4 t = mul4(x, gt);
            const float* cf = coeff + f * KT;
            float4 w = zero4();
#pragma unroll
            for (int k = 0; k < KT; ++k) {
                float ck = __ldg(cf + k);
                fma4s(w, ck, sfilt[k * 32 + lane]);
                fma4s(gf[k], ck, t);
            }
            __stcs(gin + f * CV + cg, mul4(gt, w));
        }
    }
    // block reduction in team order, one k at a time
#pragma unroll
    for (int k = 0; k < KT; ++k) {
        red[threadIdx.x] = gf[k];
        __syncthreads();
        if (team == 0 && active) {
            float4 s = zero4();
            for (int t = 0; t < teams; ++t) add4(s, red[t * TL + lane]);
            partial[((int64_t)blockIdx.x * KT + k) * CV + cg] = s;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------- backward, generic
__device__ __forceinline__ float f2v_gt(const int32_t* __restrict__ face, const int32_t* __restrict__ vtMap,
                                        const int32_t* __restrict__ nfCount, const float* __restrict__ gout,
                                        int64_t f, int Cr, int co) {
    float gt = 0.f;
    for (int j = 0; j < 3; ++j) {
        int vi = face[3 * f + j];
        int vo = vtMap ? vtMap[vi] : vi;
        if (vo >= 0) gt += __ldg(gout + (int64_t)vo * Cr + co) / (float)nfCount[vo];
    }
    return gt;
}

__global__ void f2v_bwd_input_generic_kernel(int64_t Nf, int C, int r, int K, const int32_t* __restrict__ face,
                                             const int32_t* __restrict__ vtMap, const int32_t* __restrict__ nfCount,
                                             const float* __restrict__ coeff, const float* __restrict__ filt,
                                             const float* __restrict__ gout, float* __restrict__ gin) {
    const int Cr = C * r;
    int64_t total = Nf * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t f = i / C;
        int c = (int)(i - f * C);
        float acc = 0.f;
        for (int m = 0; m < r; ++m) {
            int co = c * r + m;
            float w = 0.f;
            for (int k = 0; k < K; ++k) w = fmaf(__ldg(coeff + f * K + k), __ldg(filt + k * Cr + co), w);
            acc = fmaf(f2v_gt(face, vtMap, nfCount, gout, f, Cr, co), w, acc);
        }
        gin[i] = acc;
    }
}

// thread = output channel co, blockIdx.x = chunk of faces (walked in order), blockIdx.z = k
__global__ void f2v_bwd_filter_generic_kernel(int64_t Nf, int C, int r, int K, int64_t faces_per_chunk,
                                              const int32_t* __restrict__ face, const int32_t* __restrict__ vtMap,
                                              const int32_t* __restrict__ nfCount, const float* __restrict__ coeff,
                                              const float* __restrict__ in, const float* __restrict__ gout,
                                              float* __restrict__ partial) {
    const int Cr = C * r;
    int co = blockIdx.y * blockDim.x + threadIdx.x;
    int k = blockIdx.z;
    if (co >= Cr) return;
    int c = co / r;
    int64_t f0 = (int64_t)blockIdx.x * faces_per_chunk;
    int64_t f1 = f0 + faces_per_chunk < Nf ? f0 + faces_per_chunk : Nf;
    float acc = 0.f;
    for (int64_t f = f0; f < f1; ++f) {
        float gt = f2v_gt(face, vtMap, nfCount, gout, f, Cr, co);
        acc = fmaf(__ldg(coeff + f * K + k) * __ldg(in + f * C + c), gt, acc);
    }
    partial[((int64_t)blockIdx.x * K + k) * Cr + co] = acc;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool vec_ok(int C, int r) { return r == 1 && C % 4 == 0; }
static bool kt_ok(int K) { return K == 4 || K == 9 || K == 16 || K == 25 || K == 36; }

struct F2VBwdPlan { bool vec; int grid_x; int64_t faces_per_chunk; };
static F2VBwdPlan f2v_bwd_plan(int64_t Nf, int C, int r, int K) {
    F2VBwdPlan p;
    p.vec = vec_ok(C, r) && kt_ok(K);
    int64_t n = Nf > 0 ? Nf : 1;
    if (p.vec) {
        TeamGeom g = team_geom(C / 4);
        p.grid_x = persistent_blocks(n, g.teams, 4);
        p.faces_per_chunk = 0;
    } else {
        int64_t chunks = ceil_div(n, 64);
        int64_t cap = (int64_t)sm_count() * 4;
        if (chunks > cap) chunks = cap;
        p.faces_per_chunk = ceil_div(n, chunks);
        p.grid_x = (int)ceil_div(n, p.faces_per_chunk);
    }
    return p;
}

#define PB_DISPATCH_KT(Kv, ...)                                      \
    switch (Kv) {                                                    \
        case 4:  { constexpr int KT = 4;  __VA_ARGS__; } break;      \
        case 9:  { constexpr int KT = 9;  __VA_ARGS__; } break;      \
        case 16: { constexpr int KT = 16; __VA_ARGS__; } break;      \
        case 25: { constexpr int KT = 25; __VA_ARGS__; } break;      \
        default: { constexpr int KT = 36; __VA_ARGS__; } break;      \
    }

}  // namespace pb

using namespace pb;

extern "C" {

int pb200_facet2vertex_forward(int64_t Nf, int64_t NvOut, int C, int r, int K, const float* input,
                               const float* filter, const float* coeff, const int32_t* nfCount,
                               const int32_t* rowptr, const int32_t* entries, float* output, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NvOut >= 0 && C > 0 && r > 0 && K > 0, PB200_EINVAL, "facet2vertex_forward: bad sizes");
    if (NvOut == 0) return PB200_OK;
    PB_REQUIRE(output && rowptr && nfCount, PB200_EINVAL, "facet2vertex_forward: null pointer");
    PB_REQUIRE(Nf == 0 || (input && filter && coeff && entries), PB200_EINVAL, "facet2vertex_forward: null pointer");
    if (vec_ok(C, r) && aligned16(input) && aligned16(filter) && aligned16(output)) {
        int CV = C / 4;
        TeamGeom g = team_geom(CV);
        dim3 grid(persistent_blocks(NvOut, g.teams, 8), g.chunks);
        const float4 *in4 = (const float4*)input, *f4 = (const float4*)filter;
        float4* o4 = (float4*)output;
        if (K == 16) {
            PB_DISPATCH_TL(g.TL, PB_LAUNCH("f2v_fwd", (f2v_fwd_vec_kernel<TL, 16>), grid, 256, 0, stream, NvOut, CV, K,
                                           rowptr, entries, nfCount, coeff, in4, f4, o4));
        } else if (K == 25) {
            PB_DISPATCH_TL(g.TL, PB_LAUNCH("f2v_fwd", (f2v_fwd_vec_kernel<TL, 25>), grid, 256, 0, stream, NvOut, CV, K,
                                           rowptr, entries, nfCount, coeff, in4, f4, o4));
        } else {
            size_t smem = sizeof(float4) * 32 * (size_t)K;
            PB_REQUIRE(smem <= 48 * 1024, PB200_EINVAL, "facet2vertex_forward: K too large (%d)", K);
            PB_DISPATCH_TL(g.TL, PB_LAUNCH("f2v_fwd", (f2v_fwd_vec_kernel<TL, 0>), grid, 256, smem, stream, NvOut, CV,
                                           K, rowptr, entries, nfCount, coeff, in4, f4, o4));
        }
    } else {
        int grid = persistent_blocks(NvOut * C * r, 256, 16);
        PB_LAUNCH("f2v_fwd_generic", f2v_fwd_generic_kernel, grid, 256, 0, stream, NvOut, C, r, K, rowptr, entries,
                  nfCount, coeff, input, filter, output);
    }
    return PB200_OK;
}

size_t pb200_facet2vertex_backward_workspace_bytes(int64_t Nf, int C, int r, int K) {
    if (Nf < 0 || C <= 0 || r <= 0 || K <= 0) return 0;
    F2VBwdPlan p = f2v_bwd_plan(Nf, C, r, K);
    return align_up(sizeof(float) * (size_t)p.grid_x * K * C * r, 256);
}

int pb200_facet2vertex_backward(int64_t Nf, int64_t NvIn, int64_t NvOut, int C, int r, int K,
                                const float* gradOutput, const float* input, const float* filter,
                                const float* coeff, const int32_t* face, const int32_t* nfCount,
                                const int32_t* vtMap, float* gradInput, float* gradFilter, void* workspace,
                                size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NvIn >= 0 && NvOut >= 0 && C > 0 && r > 0 && K > 0, PB200_EINVAL,
               "facet2vertex_backward: bad sizes");
    PB_REQUIRE(gradFilter, PB200_EINVAL, "facet2vertex_backward: null pointer");
    const int Cr = C * r;
    if (Nf == 0) {
        PB_CUDA(cudaMemsetAsync(gradFilter, 0, sizeof(float) * K * Cr, stream));
        return PB200_OK;
    }
    PB_REQUIRE(gradOutput && input && filter && coeff && face && nfCount && gradInput, PB200_EINVAL,
               "facet2vertex_backward: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_facet2vertex_backward_workspace_bytes(Nf, C, r, K),
               PB200_EWORKSPACE, "facet2vertex_backward: workspace too small");
    F2VBwdPlan p = f2v_bwd_plan(Nf, C, r, K);
    float* partial = (float*)workspace;
    bool vec = p.vec && aligned16(gradOutput) && aligned16(input) && aligned16(filter) && aligned16(gradInput);
    if (vec) {
        int CV = C / 4;
        TeamGeom g = team_geom(CV);
        dim3 grid(p.grid_x, g.chunks);
        size_t smem = sizeof(float4) * (32 * (size_t)K + 256);
        PB_DISPATCH_KT(K, PB_DISPATCH_TL(g.TL, PB_LAUNCH("f2v_bwd", (f2v_bwd_vec_kernel<TL, KT>), grid, 256, smem,
                                                         stream, Nf, CV, face, vtMap, nfCount, coeff,
                                                         (const float4*)input, (const float4*)filter,
                                                         (const float4*)gradOutput, (float4*)gradInput,
                                                         (float4*)partial)));
        return reduce_partials(partial, p.grid_x, (int64_t)K * Cr, gradFilter, stream);
    }
    F2VBwdPlan q = p;
    if (p.vec) {      // alignment fell through: reuse the workspace rows that were sized for p
        int64_t chunks = ceil_div(Nf, 64);
        if (chunks > p.grid_x) chunks = p.grid_x;
        q.faces_per_chunk = ceil_div(Nf, chunks);
        q.grid_x = (int)ceil_div(Nf, q.faces_per_chunk);
    }
    int gi = persistent_blocks(Nf * C, 256, 16);
    PB_LAUNCH("f2v_bwd_input_generic", f2v_bwd_input_generic_kernel, gi, 256, 0, stream, Nf, C, r, K, face, vtMap,
              nfCount, coeff, filter, gradOutput, gradInput);
    PB_REQUIRE(K <= 65535, PB200_EINVAL, "facet2vertex_backward: K too large");
    dim3 gridf(q.grid_x, (unsigned)ceil_div(Cr, 128), K);
    PB_LAUNCH("f2v_bwd_filter_generic", f2v_bwd_filter_generic_kernel, gridf, 128, 0, stream, Nf, C, r, K,
              q.faces_per_chunk, face, vtMap, nfCount, coeff, input, gradOutput, partial);
    return reduce_partials(partial, q.grid_x, (int64_t)K * Cr, gradFilter, stream);
}

}  // extern "C"

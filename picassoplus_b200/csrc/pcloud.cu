// Point-cloud depthwise convolution with hard or fuzzy filter-bin assignment (the SPH3D kernel of
// the dual point/mesh blocks): forward, input gradient and filter gradient.  The reference scatters
// every neighbour pair with float atomics; here the forward pass is a pull over the pairs grouped
// by output point, the input gradient a pull over the pairs grouped by input point (both groupings:
// pb200_build_key_csr on the two columns of nnIndex, pair ids ascending), and the filter gradient
// a fixed-order reduction (a thread owns one output channel, walks its block's pairs in order,
// blocks are added in order).  No floating-point atomics: results do not depend on scheduling.
#include "common.cuh"

namespace pb {
namespace pcloud {

// weight of pair p for output channel co: filter[bin[p], co] (hard assignment) or
// sum_t coeff[p,t] * filter[bin[p,t], co] (fuzzy).  A bin index outside [0, F) contributes 0.
__device__ __forceinline__ float pair_weight(int64_t p, int co, int Cr, int F, int T, const int32_t* __restrict__ bin,
                                             const float* __restrict__ coeff, const float* __restrict__ filter) {
    if (!coeff) {
        const int f = bin[p];
        return (f >= 0 && f < F) ? __ldg(filter + (int64_t)f * Cr + co) : 0.f;
    }
    float w = 0.f;
    for (int t = 0; t < T; ++t) {
        const int f = bin[p * T + t];
        if (f >= 0 && f < F) w = fmaf(coeff[p * T + t], __ldg(filter + (int64_t)f * Cr + co), w);
    }
    return w;
}

// output[o, co] = sum over the pairs p of output point o of input[in_p, co / r] * w_p[co] / nnCount[o]
// (reference: depthwise_conv3d_forward / fuzzy_depthwise_conv3d_forward, pcloud_conv3d_gpu.cu:8-27,94-118:
// each term is divided before it is added)
__global__ void conv_fwd_kernel(int64_t Np, int64_t Mp, int F, int C, int r, int T, const float* __restrict__ input,
                                const float* __restrict__ filter, const int32_t* __restrict__ nnCount,
                                const int32_t* __restrict__ nnIndex, const int32_t* __restrict__ bin,
                                const float* __restrict__ coeff, const int32_t* __restrict__ rowptr,
                                const int32_t* __restrict__ members, float* __restrict__ output) {
    const int Cr = C * r;
    const int64_t total = Mp * Cr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = i / Cr;
        const int co = (int)(i - o * Cr), cin = co / r;
        const float nn = (float)nnCount[o];
        float acc = 0.f;
        for (int e = rowptr[o]; e < rowptr[o + 1]; ++e) {
            const int64_t p = members[e];
            const int in = nnIndex[2 * p + 1];
            if (in < 0 || in >= Np) continue;
            acc += __ldg(input + (int64_t)in * C + cin) * pair_weight(p, co, Cr, F, T, bin, coeff, filter) / nn;
        }
        output[i] = acc;
    }
}

// gradInput[n, c] = sum over the pairs p of input point n, over m < r, of
// gradOutput[out_p, c*r+m] * w_p[c*r+m] / nnCount[out_p]
// (reference: depthwise_input_backward / fuzzy_depthwise_input_backward, pcloud_conv3d_gpu.cu:30-48,121-147)
__global__ void conv_bwd_input_kernel(int64_t Np, int64_t Mp, int F, int C, int r, int T, const float* __restrict__ gout,
                                      const float* __restrict__ filter, const int32_t* __restrict__ nnCount,
                                      const int32_t* __restrict__ nnIndex, const int32_t* __restrict__ bin,
                                      const float* __restrict__ coeff, const int32_t* __restrict__ rowptr,
                                      const int32_t* __restrict__ members, float* __restrict__ gin) {
    const int Cr = C * r;
    const int64_t total = Np * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / C;
        const int c = (int)(i - n * C);
        float acc = 0.f;
        for (int e = rowptr[n]; e < rowptr[n + 1]; ++e) {
            const int64_t p = members[e];
            const int o = nnIndex[2 * p];
            if (o < 0 || o >= Mp) continue;
            const float nn = (float)nnCount[o];
            for (int m = 0; m < r; ++m) {
                const int co = c * r + m;
                acc += __ldg(gout + (int64_t)o * Cr + co) * pair_weight(p, co, Cr, F, T, bin, coeff, filter) / nn;
            }
        }
        gin[i] = acc;
    }
}

// partial[block][f, co] = sum over the block's pairs (ascending) of coeff * gradOutput[out_p, co] *
// input[in_p, co / r] / nnCount[out_p] (reference: depthwise_filter_backward /
// fuzzy_depthwise_filter_backward, pcloud_conv3d_gpu.cu:51-88,150-193).  Thread = output channel:
// it alone touches column co of the block's accumulator in shared memory.
__global__ void conv_bwd_filter_kernel(int64_t Np, int64_t Mp, int64_t Nout, int64_t pairs_per_block, int F, int C, int r,
                                       int T, const float* __restrict__ input, const float* __restrict__ gout,
                                       const int32_t* __restrict__ nnCount, const int32_t* __restrict__ nnIndex,
                                       const int32_t* __restrict__ bin, const float* __restrict__ coeff,
                                       float* __restrict__ partial) {
    extern __shared__ float acc[];                   // [F][Cr]
    const int Cr = C * r;
    for (int i = threadIdx.x; i < F * Cr; i += blockDim.x) acc[i] = 0.f;
    __syncthreads();
    const int64_t p0 = (int64_t)blockIdx.x * pairs_per_block;
    int64_t p1 = p0 + pairs_per_block;
    if (p1 > Nout) p1 = Nout;
    for (int co = threadIdx.x; co < Cr; co += blockDim.x) {
        const int cin = co / r;
        for (int64_t p = p0; p < p1; ++p) {
            const int o = nnIndex[2 * p], in = nnIndex[2 * p + 1];
            if (o < 0 || o >= Mp || in < 0 || in >= Np) continue;
            const float d = __ldg(gout + (int64_t)o * Cr + co) * __ldg(input + (int64_t)in * C + cin) / (float)nnCount[o];
            if (!coeff) {
                const int f = bin[p];
                if (f >= 0 && f < F) acc[f * Cr + co] += d;
            } else {
                for (int t = 0; t < T; ++t) {
                    const int f = bin[p * T + t];
                    if (f >= 0 && f < F) acc[f * Cr + co] += coeff[p * T + t] * d;
                }
            }
        }
    }
    __syncthreads();
    float* out = partial + (int64_t)blockIdx.x * F * Cr;
    for (int i = threadIdx.x; i < F * Cr; i += blockDim.x) out[i] = acc[i];
}

// ------------------------------------------------------------------------ vector kernels
// Depth multiplier 1 and C a multiple of 4 (every layer of the reference's networks): a thread owns four
// channels of a point, the filter table lives in shared memory, a term is x * w * (1 / nnCount).
__device__ __forceinline__ float4 pair_weight4(int64_t p, int cg, int CV, int F, int T, const int32_t* __restrict__ bin,
                                               const float* __restrict__ coeff, const float4* __restrict__ sfilt) {
    if (!coeff) {
        const int f = __ldg(bin + p);
        return (f >= 0 && f < F) ? sfilt[f * CV + cg] : zero4();
    }
    float4 w = zero4();
    for (int t = 0; t < T; ++t) {
        const int f = __ldg(bin + p * T + t);
        if (f >= 0 && f < F) fma4s(w, __ldg(coeff + p * T + t), sfilt[f * CV + cg]);
    }
    return w;
}

__global__ void conv_fwd_vec_kernel(int64_t Np, int64_t Mp, int F, int CV, int T, const float4* __restrict__ input,
                                    const float4* __restrict__ filter, const int32_t* __restrict__ nnCount,
                                    const int32_t* __restrict__ nnIndex, const int32_t* __restrict__ bin,
                                    const float* __restrict__ coeff, const int32_t* __restrict__ rowptr,
                                    const int32_t* __restrict__ members, float4* __restrict__ output) {
    extern __shared__ float4 sfilt[];                // [F][CV]
    for (int i = threadIdx.x; i < F * CV; i += blockDim.x) sfilt[i] = filter[i];
    __syncthreads();
    const int64_t total = Mp * CV;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = i / CV;
        const int cg = (int)(i - o * CV);
        const float rn = 1.f / (float)__ldg(nnCount + o);
        float4 acc = zero4();
        for (int e = __ldg(rowptr + o); e < __ldg(rowptr + o + 1); ++e) {
            const int64_t p = __ldg(members + e);
            const int in = __ldg(nnIndex + 2 * p + 1);
            if (in < 0 || in >= Np) continue;
            const float4 w = pair_weight4(p, cg, CV, F, T, bin, coeff, sfilt);
            fma4(acc, scale4(ldg4(input + (int64_t)in * CV + cg), rn), w);
        }
        output[i] = acc;
    }
}

__global__ void conv_bwd_input_vec_kernel(int64_t Np, int64_t Mp, int F, int CV, int T, const float4* __restrict__ gout,
                                          const float4* __restrict__ filter, const int32_t* __restrict__ nnCount,
                                          const int32_t* __restrict__ nnIndex, const int32_t* __restrict__ bin,
                                          const float* __restrict__ coeff, const int32_t* __restrict__ rowptr,
                                          const int32_t* __restrict__ members, float4* __restrict__ gin) {
    extern __shared__ float4 sfilt[];
    for (int i = threadIdx.x; i < F * CV; i += blockDim.x) sfilt[i] = filter[i];
    __syncthreads();
    const int64_t total = Np * CV;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / CV;
        const int cg = (int)(i - n * CV);
        float4 acc = zero4();
        for (int e = __ldg(rowptr + n); e < __ldg(rowptr + n + 1); ++e) {
            const int64_t p = __ldg(members + e);
            const int o = __ldg(nnIndex + 2 * p);
            if (o < 0 || o >= Mp) continue;
            const float rn = 1.f / (float)__ldg(nnCount + o);
            const float4 w = pair_weight4(p, cg, CV, F, T, bin, coeff, sfilt);
            fma4(acc, scale4(ldg4(gout + (int64_t)o * CV + cg), rn), w);
        }
        gin[i] = acc;
    }
}

// Filter gradient: a block takes a contiguous run of pairs; its 256 threads are SUB groups of CV lanes, group g
// walks every SUB-th pair of the run in order and adds into its own copy of the [F][C] accumulator in shared
// memory (a lane alone touches its four columns of its copy); the copies are added in group order, the blocks in
// block order: fixed order throughout.
__global__ void conv_bwd_filter_vec_kernel(int64_t Np, int64_t Mp, int64_t Nout, int pairs_per_block, int F, int CV, int T,
                                           int SUB, const float4* __restrict__ input, const float4* __restrict__ gout,
                                           const int32_t* __restrict__ nnCount, const int32_t* __restrict__ nnIndex,
                                           const int32_t* __restrict__ bin, const float* __restrict__ coeff,
                                           float4* __restrict__ partial) {
    extern __shared__ float4 acc4[];                 // [SUB][F][CV]
    for (int i = threadIdx.x; i < SUB * F * CV; i += blockDim.x) acc4[i] = zero4();
    __syncthreads();
    const int g = threadIdx.x / CV, cg = threadIdx.x - g * CV;
    const int64_t p0 = (int64_t)blockIdx.x * pairs_per_block;
    int64_t p1 = p0 + pairs_per_block;
    if (p1 > Nout) p1 = Nout;
    if (g < SUB) {
        float4* mine = acc4 + (size_t)g * F * CV;
        for (int64_t p = p0 + g; p < p1; p += SUB) {
            const int o = __ldg(nnIndex + 2 * p), in = __ldg(nnIndex + 2 * p + 1);
            if (o < 0 || o >= Mp || in < 0 || in >= Np) continue;
            const float rn = 1.f / (float)__ldg(nnCount + o);
            const float4 d = mul4(scale4(ldg4(gout + (int64_t)o * CV + cg), rn), ldg4(input + (int64_t)in * CV + cg));
            if (!coeff) {
                const int f = __ldg(bin + p);
                if (f >= 0 && f < F) add4(mine[f * CV + cg], d);
            } else {
                for (int t = 0; t < T; ++t) {
                    const int f = __ldg(bin + p * T + t);
                    if (f >= 0 && f < F) fma4s(mine[f * CV + cg], __ldg(coeff + p * T + t), d);
                }
            }
        }
    }
    __syncthreads();
    float4* out = partial + (int64_t)blockIdx.x * F * CV;
    for (int i = threadIdx.x; i < F * CV; i += blockDim.x) {
        float4 s4 = acc4[i];
        for (int q = 1; q < SUB; ++q) add4(s4, acc4[(size_t)q * F * CV + i]);
        out[i] = s4;
    }
}

static bool sizes_ok(int64_t Np, int64_t Mp, int64_t Nout, int F, int C, int r, int T) {
    return Np >= 0 && Mp >= 0 && Nout >= 0 && F > 0 && C > 0 && r > 0 && T > 0 && Np < (1LL << 31) && Mp < (1LL << 31) &&
           Nout < (1LL << 31) && (int64_t)F * C * r * 4 <= 200 * 1024;
}
// ------------------------------------------------------------------------ cooperative kernels
// C of 32, 64 or 128: the CV = C / 4 lanes of a point sit in one warp, so lane j fetches the indices of the j-th
// pair of a run and the run is walked with shuffles, four pairs at a time: the four row gathers and the bin
// fetches of a step are in flight together. TT: 1 = one bin per pair, 3 = three weighted bins, 0 = any T.
// Same order of additions as the vector kernels.
template <int CV>
__device__ __forceinline__ unsigned group_mask(int gbase) {
    return CV == 32 ? 0xffffffffu : (((1u << (CV & 31)) - 1u) << gbase);
}

template <int TT, int CV>
__device__ __forceinline__ float4 pair_weight4t(int64_t p, int cg, int F, int T, const int32_t* __restrict__ bin,
                                                const float* __restrict__ coeff, const float4* __restrict__ sfilt) {
    if constexpr (TT == 0) {
        return pair_weight4(p, cg, CV, F, T, bin, coeff, sfilt);
    } else if constexpr (TT == 1) {
        const int f = __ldg(bin + p);
        const bool ok = (unsigned)f < (unsigned)F;
        const float4 w = sfilt[(ok ? f : 0) * CV + cg];
        return ok ? w : zero4();
    } else {
    int f[3];
    float c[3];
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        f[t] = __ldg(bin + p * 3 + t);
        c[t] = __ldg(coeff + p * 3 + t);
    }
    float4 w = zero4();
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const bool ok = (unsigned)f[t] < (unsigned)F;
        fma4s(w, ok ? c[t] : 0.f, sfilt[(ok ? f[t] : 0) * CV + cg]);
    }
    return w;
    }
}

template <int TT, int CV>
__global__ void __launch_bounds__(256)
conv_fwd_coop_kernel(int64_t Np, int64_t Mp, int F, int T, const float4* __restrict__ input,
                     const float4* __restrict__ filter, const int32_t* __restrict__ nnCount,
                     const int32_t* __restrict__ nnIndex, const int32_t* __restrict__ bin, const float* __restrict__ coeff,
                     const int32_t* __restrict__ rowptr, const int32_t* __restrict__ members, float4* __restrict__ output) {
    extern __shared__ float4 sfilt[];
    for (int i = threadIdx.x; i < F * CV; i += blockDim.x) sfilt[i] = filter[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, cg = lane % CV, gbase = lane - cg;
    const unsigned mask = group_mask<CV>(gbase);
    const int64_t stride = (int64_t)gridDim.x * (blockDim.x / CV);
    for (int64_t o = (int64_t)blockIdx.x * (blockDim.x / CV) + threadIdx.x / CV; o < Mp; o += stride) {
        const int e0 = __ldg(rowptr + o), e1 = __ldg(rowptr + o + 1);
        const float rn = 1.f / (float)__ldg(nnCount + o);
        float4 acc = zero4();
        for (int e = e0; e < e1; e += CV) {
            int p_mine = 0, in_mine = -1;
            if (e + cg < e1) {
                p_mine = __ldg(members + e + cg);
                in_mine = __ldg(nnIndex + 2 * (int64_t)p_mine + 1);
            }
            const int n = e1 - e < CV ? e1 - e : CV;
            for (int j = 0; j < n; j += 4) {
                float4 x[4], w[4];
                int pp[4];
                bool ok[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int src = gbase + ((j + u) & (CV - 1));
                    pp[u] = __shfl_sync(mask, p_mine, src);
                    const int in = __shfl_sync(mask, in_mine, src);
                    ok[u] = j + u < n && in >= 0 && in < Np;
                    x[u] = ok[u] ? ldg4(input + (int64_t)in * CV + cg) : zero4();
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) w[u] = pair_weight4t<TT, CV>(pp[u], cg, F, T, bin, coeff, sfilt);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (ok[u]) fma4(acc, scale4(x[u], rn), w[u]);
            }
        }
        output[o * CV + cg] = acc;
    }
}

// The bins and weights of the pair a lane fetched (TT of 1 or 3), handed to the group's lanes by shuffles.
template <int TT>
struct LaneBins {
    int f[TT == 3 ? 3 : 1];
    float c[TT == 3 ? 3 : 1];
};

template <int TT>
__device__ __forceinline__ void load_bins(LaneBins<TT>& b, bool have, int64_t p, const int32_t* __restrict__ bin,
                                          const float* __restrict__ coeff) {
#pragma unroll
    for (int t = 0; t < (TT == 3 ? 3 : 1); ++t) {
        b.f[t] = have ? __ldg(bin + p * (TT == 3 ? 3 : 1) + t) : -1;
        b.c[t] = TT == 3 ? (have ? __ldg(coeff + p * 3 + t) : 0.f) : 1.f;
    }
}

template <int TT, int CV>
__device__ __forceinline__ float4 shuffled_weight4(const LaneBins<TT>& b, unsigned mask, int src, int cg, int F,
                                                   const float4* __restrict__ sfilt) {
    float4 w = zero4();
#pragma unroll
    for (int t = 0; t < (TT == 3 ? 3 : 1); ++t) {
        const int f = __shfl_sync(mask, b.f[t], src);
        const float c = TT == 3 ? __shfl_sync(mask, b.c[t], src) : 1.f;
        const bool ok = (unsigned)f < (unsigned)F;
        fma4s(w, ok ? c : 0.f, sfilt[(ok ? f : 0) * CV + cg]);
    }
    return w;
}

// one step of the input gradient: up to four pairs whose indices sit in the lanes of the group, slots j .. j + 3
// of [j, end); the four rows of the output gradient and the bin fetches are in flight together
template <int TT, int CV>
__device__ __forceinline__ void bwd_input_step(float4& acc, int j, int end, unsigned mask, int gbase, int cg, int p_mine,
                                               int o_mine, float rn_mine, const LaneBins<TT>& mybins, int64_t Mp, int F, int T,
                                               const float4* __restrict__ gout, const int32_t* __restrict__ bin,
                                               const float* __restrict__ coeff, const float4* __restrict__ sfilt) {
    float4 x[4], w[4];
    int pp[4];
    float rn[4];
    bool ok[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int src = gbase + ((j + u) & (CV - 1));
        pp[u] = __shfl_sync(mask, p_mine, src);
        const int o = __shfl_sync(mask, o_mine, src);
        rn[u] = __shfl_sync(mask, rn_mine, src);
        ok[u] = j + u < end && o >= 0 && o < Mp;
        x[u] = ok[u] ? ldg4(gout + (int64_t)o * CV + cg) : zero4();
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        if constexpr (TT == 0) w[u] = pair_weight4(pp[u], cg, CV, F, T, bin, coeff, sfilt);
        else w[u] = shuffled_weight4<TT, CV>(mybins, mask, gbase + ((j + u) & (CV - 1)), cg, F, sfilt);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
        if (ok[u]) fma4(acc, scale4(x[u], rn[u]), w[u]);
}

// A group takes W = CV / 4 consecutive input points per step: their pairs are one contiguous run of the grouping,
// and when it fits the group's lanes (the usual case: an input point is the neighbour of a few output points) one
// fetch of the indices serves all W points.
template <int TT, int CV>
__global__ void __launch_bounds__(256, 4)
conv_bwd_input_coop_kernel(int64_t Np, int64_t Mp, int F, int T, const float4* __restrict__ gout,
                           const float4* __restrict__ filter, const int32_t* __restrict__ nnCount,
                           const int32_t* __restrict__ nnIndex, const int32_t* __restrict__ bin,
                           const float* __restrict__ coeff, const int32_t* __restrict__ rowptr,
                           const int32_t* __restrict__ members, float4* __restrict__ gin) {
    constexpr int W = CV / 4;
    extern __shared__ float4 sfilt[];
    for (int i = threadIdx.x; i < F * CV; i += blockDim.x) sfilt[i] = filter[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, cg = lane % CV, gbase = lane - cg;
    const unsigned mask = group_mask<CV>(gbase);
    const int64_t stride = (int64_t)gridDim.x * (blockDim.x / CV) * W;
    for (int64_t base = ((int64_t)blockIdx.x * (blockDim.x / CV) + threadIdx.x / CV) * W; base < Np; base += stride) {
        int rp_mine = 0;
        if (cg <= W) rp_mine = __ldg(rowptr + (base + cg < Np ? base + cg : Np));
        const int E0 = __shfl_sync(mask, rp_mine, gbase), EW = __shfl_sync(mask, rp_mine, gbase + W);
        const bool together = EW - E0 <= CV;
        int p_mine = 0, o_mine = -1;
        float rn_mine = 0.f;
        LaneBins<TT> mybins;
        if (together) {
            const bool have = E0 + cg < EW;
            if (have) p_mine = __ldg(members + E0 + cg);
            if (have) o_mine = __ldg(nnIndex + 2 * (int64_t)p_mine);
            if constexpr (TT != 0) load_bins<TT>(mybins, have, p_mine, bin, coeff);
            if (o_mine >= 0 && o_mine < Mp) rn_mine = 1.f / (float)__ldg(nnCount + o_mine);
        }
#pragma unroll 1
        for (int k = 0; k < W; ++k) {
            const int e0 = __shfl_sync(mask, rp_mine, gbase + k), e1 = __shfl_sync(mask, rp_mine, gbase + k + 1);
            float4 acc = zero4();
            if (together) {
                for (int j = e0 - E0; j < e1 - E0; j += 4)
                    bwd_input_step<TT, CV>(acc, j, e1 - E0, mask, gbase, cg, p_mine, o_mine, rn_mine, mybins, Mp, F, T, gout, bin,
                                           coeff, sfilt);
            } else {
                for (int e = e0; e < e1; e += CV) {
                    p_mine = 0, o_mine = -1, rn_mine = 0.f;
                    const bool have = e + cg < e1;
                    if (have) p_mine = __ldg(members + e + cg);
                    if (have) o_mine = __ldg(nnIndex + 2 * (int64_t)p_mine);
                    if constexpr (TT != 0) load_bins<TT>(mybins, have, p_mine, bin, coeff);
                    if (o_mine >= 0 && o_mine < Mp) rn_mine = 1.f / (float)__ldg(nnCount + o_mine);
                    const int n = e1 - e < CV ? e1 - e : CV;
                    for (int j = 0; j < n; j += 4)
                        bwd_input_step<TT, CV>(acc, j, n, mask, gbase, cg, p_mine, o_mine, rn_mine, mybins, Mp, F, T, gout, bin,
                                               coeff, sfilt);
                }
            }
            if (base + k < Np) gin[(base + k) * CV + cg] = acc;
        }
    }
}

// Filter gradient: a block of SUB groups of CV lanes takes a contiguous run of pairs, group g the g-th equal part
// of it, walked in order into the group's own copy of the [F][C] accumulator in shared memory; copies are added in
// group order, blocks in block order.
template <int TT, int CV>
__global__ void __launch_bounds__(256)
conv_bwd_filter_coop_kernel(int64_t Np, int64_t Mp, int64_t Nout, int pairs_per_block, int SUB, int F, int T,
                            const float4* __restrict__ input, const float4* __restrict__ gout,
                            const int32_t* __restrict__ nnCount, const int32_t* __restrict__ nnIndex,
                            const int32_t* __restrict__ bin, const float* __restrict__ coeff, float4* __restrict__ partial) {
    extern __shared__ float4 acc4[];                 // [SUB][F][CV]
    for (int i = threadIdx.x; i < SUB * F * CV; i += blockDim.x) acc4[i] = zero4();
    __syncthreads();
    const int lane = threadIdx.x & 31, cg = lane % CV, gbase = lane - cg, g = threadIdx.x / CV;
    const unsigned mask = group_mask<CV>(gbase);
    const int per_group = (pairs_per_block + SUB - 1) / SUB;
    const int64_t b0 = (int64_t)blockIdx.x * pairs_per_block;
    int64_t b1 = b0 + pairs_per_block;
    if (b1 > Nout) b1 = Nout;
    const int64_t q0 = b0 + (int64_t)g * per_group;
    int64_t q1 = q0 + per_group;
    if (q1 > b1) q1 = b1;
    float4* mine = acc4 + (size_t)g * F * CV;
    for (int64_t q = q0; q < q1; q += CV) {
        int o_mine = -1, in_mine = -1;
        float rn_mine = 0.f;
        LaneBins<TT> mybins;
        const bool have = q + cg < q1;
        if (have) {
            o_mine = __ldg(nnIndex + 2 * (q + cg));
            in_mine = __ldg(nnIndex + 2 * (q + cg) + 1);
        }
        if constexpr (TT != 0) load_bins<TT>(mybins, have, q + cg, bin, coeff);
        if (o_mine >= 0 && o_mine < Mp) rn_mine = 1.f / (float)__ldg(nnCount + o_mine);
        const int n = q1 - q < CV ? (int)(q1 - q) : CV;
        for (int j = 0; j < n; j += 4) {
            float4 gr[4], xr[4];
            float rn[4];
            bool ok[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int src = gbase + ((j + u) & (CV - 1));
                const int o = __shfl_sync(mask, o_mine, src);
                const int in = __shfl_sync(mask, in_mine, src);
                rn[u] = __shfl_sync(mask, rn_mine, src);
                ok[u] = j + u < n && o >= 0 && o < Mp && in >= 0 && in < Np;
                gr[u] = ok[u] ? ldg4(gout + (int64_t)o * CV + cg) : zero4();
                xr[u] = ok[u] ? ldg4(input + (int64_t)in * CV + cg) : zero4();
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 d = mul4(scale4(gr[u], rn[u]), xr[u]);
                if constexpr (TT != 0) {
                    const int src = gbase + ((j + u) & (CV - 1));
#pragma unroll
                    for (int t = 0; t < (TT == 3 ? 3 : 1); ++t) {
                        const int f = __shfl_sync(mask, mybins.f[t], src);
                        const float c = TT == 3 ? __shfl_sync(mask, mybins.c[t], src) : 1.f;
                        if (ok[u] && (unsigned)f < (unsigned)F) fma4s(mine[f * CV + cg], c, d);
                    }
                } else if (ok[u]) {
                    const int64_t p = q + j + u;
                    if (!coeff) {
                        const int fb = __ldg(bin + p);
                        if (fb >= 0 && fb < F) add4(mine[fb * CV + cg], d);
                    } else {
                        for (int t = 0; t < T; ++t) {
                            const int fb = __ldg(bin + p * T + t);
                            if (fb >= 0 && fb < F) fma4s(mine[fb * CV + cg], __ldg(coeff + p * T + t), d);
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    float4* out = partial + (int64_t)blockIdx.x * F * CV;
    for (int i = threadIdx.x; i < F * CV; i += blockDim.x) {
        float4 s4 = acc4[i];
        for (int k = 1; k < SUB; ++k) add4(s4, acc4[(size_t)k * F * CV + i]);
        out[i] = s4;
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
// the vector kernels: depth multiplier 1, channels a multiple of 4 and at most 1024 (one group of lanes per point),
// and a filter table that leaves room in shared memory for at least one accumulator copy
static bool vec_ok(int F, int C, int r) { return r == 1 && C % 4 == 0 && C <= 1024 && (size_t)F * C * 4 <= 48 * 1024; }
constexpr int VEC_PAIRS_PER_BLOCK = 2048;
static int vec_filter_blocks(int64_t Nout) { return (int)ceil_div(Nout > 0 ? Nout : 1, VEC_PAIRS_PER_BLOCK); }
static int vec_sub_groups(int F, int C) {
    int sub = 256 / (C / 4);
    if (sub < 1) sub = 1;
    while (sub > 1 && (size_t)sub * F * C * 4 > 96 * 1024) --sub;
    return sub;
}

// groups of a filter-gradient block: as many accumulator copies as fit 56 KB (four blocks on an SM), whole warps
static int coop_sub_groups(int F, int C) {
    const int CV = C / 4, step = 32 / CV, most = 256 / CV;
    int sub = (int)((56 * 1024) / ((size_t)F * C * 4)) / step * step;
    return sub < step ? step : sub > most ? most : sub;
}
static bool coop_ok(int F, int C) {
    return (C == 32 || C == 64 || C == 128) && (size_t)coop_sub_groups(F, C) * F * C * 4 <= 200 * 1024;
}

template <int TT, int CV>
static int launch_fwd_coop(int64_t Np, int64_t Mp, int F, int T, const float* input, const float* filter, const int32_t* nnCount,
                           const int32_t* nnIndex, const int32_t* bin, const float* coeff, const int32_t* rowptr,
                           const int32_t* members, float* output, cudaStream_t stream) {
    PB_LAUNCH("pcloud_conv_fwd", (conv_fwd_coop_kernel<TT, CV>), persistent_blocks(Mp * CV, 256, 8), 256, sizeof(float4) * F * CV,
              stream, Np, Mp, F, T, (const float4*)input, (const float4*)filter, nnCount, nnIndex, bin, coeff, rowptr, members,
              (float4*)output);
    return PB200_OK;
}

template <int TT, int CV>
static int launch_bwd_coop(int64_t Np, int64_t Mp, int64_t Nout, int nb, int F, int T, const float* input, const float* filter,
                           const float* gout, const int32_t* nnCount, const int32_t* nnIndex, const int32_t* bin,
                           const float* coeff, const int32_t* rowptr, const int32_t* members, float* gin, float* partial,
                           cudaStream_t stream) {
    if (Np > 0)
        PB_LAUNCH("pcloud_conv_bwd_input", (conv_bwd_input_coop_kernel<TT, CV>), persistent_blocks(Np * CV, 256, 8), 256,
                  sizeof(float4) * F * CV, stream, Np, Mp, F, T, (const float4*)gout, (const float4*)filter, nnCount, nnIndex, bin,
                  coeff, rowptr, members, (float4*)gin);
    const int sub = coop_sub_groups(F, 4 * CV);
    const size_t smem = sizeof(float4) * (size_t)sub * F * CV;
    PB_CUDA(cudaFuncSetAttribute(conv_bwd_filter_coop_kernel<TT, CV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PB_LAUNCH("pcloud_conv_bwd_filter", (conv_bwd_filter_coop_kernel<TT, CV>), nb, sub * CV, smem, stream, Np, Mp, Nout,
              VEC_PAIRS_PER_BLOCK, sub, F, T, (const float4*)input, (const float4*)gout, nnCount, nnIndex, bin, coeff,
              (float4*)partial);
    return PB200_OK;
}

// the kernels are built for CV of 8, 16, 32 and for one bin per pair, three weighted bins, or any T
#define PB_COOP_DISPATCH(FN, ...)                                                                                  \
    (tt == 1 ? (CV == 8 ? FN<1, 8>(__VA_ARGS__) : CV == 16 ? FN<1, 16>(__VA_ARGS__) : FN<1, 32>(__VA_ARGS__))      \
     : tt == 3 ? (CV == 8 ? FN<3, 8>(__VA_ARGS__) : CV == 16 ? FN<3, 16>(__VA_ARGS__) : FN<3, 32>(__VA_ARGS__))    \
               : (CV == 8 ? FN<0, 8>(__VA_ARGS__) : CV == 16 ? FN<0, 16>(__VA_ARGS__) : FN<0, 32>(__VA_ARGS__)))

static int filter_blocks(int64_t Nout) {
    int64_t b = ceil_div(Nout > 0 ? Nout : 1, 256);         // at least 256 pairs per block
    const int cap = 4 * sm_count();
    return (int)(b < cap ? b : cap);
}

}  // namespace pcloud
}  // namespace pb

using namespace pb;
using namespace pb::pcloud;

extern "C" {

int pb200_pcloud_conv3d_forward(int64_t Np, int64_t Mp, int64_t Nout, int F, int C, int r, int T, const float* input,
                                const float* filter, const int32_t* nnCount, const int32_t* nnIndex,
                                const int32_t* binIndex, const float* binCoeff, const int32_t* rowptr_out,
                                const int32_t* members_out, float* output, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(Np, Mp, Nout, F, C, r, T), PB200_EINVAL, "pcloud_conv3d_forward: bad sizes");
    if (Mp == 0) return PB200_OK;
    PB_REQUIRE(filter && nnCount && rowptr_out && output && (Nout == 0 || (input && nnIndex && binIndex && members_out)),
               PB200_EINVAL, "pcloud_conv3d_forward: null pointer");
    if (vec_ok(F, C, r) && aligned16(input) && aligned16(filter) && aligned16(output)) {
        const int CV = C / 4;
        if (coop_ok(F, C)) {
            const int tt = !binCoeff ? 1 : T == 3 ? 3 : 0;
            return PB_COOP_DISPATCH(launch_fwd_coop, Np, Mp, F, T, input, filter, nnCount, nnIndex, binIndex, binCoeff, rowptr_out,
                                    members_out, output, stream);
        }
        PB_LAUNCH("pcloud_conv_fwd", conv_fwd_vec_kernel, persistent_blocks(Mp * CV, 256, 8), 256, sizeof(float) * F * C, stream,
                  Np, Mp, F, CV, T, (const float4*)input, (const float4*)filter, nnCount, nnIndex, binIndex, binCoeff, rowptr_out,
                  members_out, (float4*)output);
        return PB200_OK;
    }
    PB_LAUNCH("pcloud_conv_fwd", conv_fwd_kernel, persistent_blocks(Mp * C * r, 256, 16), 256, 0, stream, Np, Mp, F, C, r, T,
              input, filter, nnCount, nnIndex, binIndex, binCoeff, rowptr_out, members_out, output);
    return PB200_OK;
}

size_t pb200_pcloud_conv3d_backward_workspace_bytes(int64_t Nout, int F, int C, int r) {
    if (Nout < 0 || F <= 0 || C <= 0 || r <= 0) return 0;
    const size_t nb = vec_ok(F, C, r) && vec_filter_blocks(Nout) > filter_blocks(Nout) ? vec_filter_blocks(Nout) : filter_blocks(Nout);
    return align_up(nb * F * C * r * sizeof(float), 256);
}

int pb200_pcloud_conv3d_backward(int64_t Np, int64_t Mp, int64_t Nout, int F, int C, int r, int T, const float* gradOutput,
                                 const float* input, const float* filter, const int32_t* nnCount, const int32_t* nnIndex,
                                 const int32_t* binIndex, const float* binCoeff, const int32_t* rowptr_in,
                                 const int32_t* members_in, float* gradInput, float* gradFilter, void* workspace,
                                 size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(sizes_ok(Np, Mp, Nout, F, C, r, T), PB200_EINVAL, "pcloud_conv3d_backward: bad sizes");
    PB_REQUIRE(gradFilter && filter && (Np == 0 || (gradInput && rowptr_in)), PB200_EINVAL,
               "pcloud_conv3d_backward: null pointer");
    PB_REQUIRE(Nout == 0 || (gradOutput && input && nnCount && nnIndex && binIndex && members_in), PB200_EINVAL,
               "pcloud_conv3d_backward: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_pcloud_conv3d_backward_workspace_bytes(Nout, F, C, r), PB200_EWORKSPACE,
               "pcloud_conv3d_backward: workspace too small");
    if (vec_ok(F, C, r) && aligned16(input) && aligned16(filter) && aligned16(gradOutput) && aligned16(gradInput) &&
        aligned16(workspace)) {
        const int CV = C / 4;
        if (coop_ok(F, C)) {
            const int nbc = vec_filter_blocks(Nout);
            const int tt = !binCoeff ? 1 : T == 3 ? 3 : 0;
            const int rc = PB_COOP_DISPATCH(launch_bwd_coop, Np, Mp, Nout, nbc, F, T, input, filter, gradOutput, nnCount, nnIndex,
                                            binIndex, binCoeff, rowptr_in, members_in, gradInput, (float*)workspace, stream);
            if (rc != PB200_OK) return rc;
            return reduce_partials((const float*)workspace, nbc, (int64_t)F * C, gradFilter, stream);
        }
        if (Np > 0)
            PB_LAUNCH("pcloud_conv_bwd_input", conv_bwd_input_vec_kernel, persistent_blocks(Np * CV, 256, 8), 256,
                      sizeof(float) * F * C, stream, Np, Mp, F, CV, T, (const float4*)gradOutput, (const float4*)filter, nnCount,
                      nnIndex, binIndex, binCoeff, rowptr_in, members_in, (float4*)gradInput);
        const int nbv = vec_filter_blocks(Nout), sub = vec_sub_groups(F, C);
        const size_t smemv = sizeof(float) * (size_t)sub * F * C;
        const int threads = sub * CV < 32 ? 32 : ((sub * CV + 31) / 32) * 32;
        PB_CUDA(cudaFuncSetAttribute(conv_bwd_filter_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smemv));
        PB_LAUNCH("pcloud_conv_bwd_filter", conv_bwd_filter_vec_kernel, nbv, threads, smemv, stream, Np, Mp, Nout,
                  VEC_PAIRS_PER_BLOCK, F, CV, T, sub, (const float4*)input, (const float4*)gradOutput, nnCount, nnIndex, binIndex,
                  binCoeff, (float4*)workspace);
        return reduce_partials((const float*)workspace, nbv, (int64_t)F * C, gradFilter, stream);
    }
    if (Np > 0)
        PB_LAUNCH("pcloud_conv_bwd_input", conv_bwd_input_kernel, persistent_blocks(Np * C, 256, 16), 256, 0, stream, Np, Mp,
                  F, C, r, T, gradOutput, filter, nnCount, nnIndex, binIndex, binCoeff, rowptr_in, members_in, gradInput);
    const int nb = filter_blocks(Nout);
    const int Cr = C * r;
    const int threads = Cr >= 256 ? 256 : ((Cr + 31) / 32) * 32;
    const size_t smem = sizeof(float) * (size_t)F * Cr;
    PB_CUDA(cudaFuncSetAttribute(conv_bwd_filter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PB_LAUNCH("pcloud_conv_bwd_filter", conv_bwd_filter_kernel, nb, threads, smem, stream, Np, Mp, Nout,
              ceil_div(Nout > 0 ? Nout : 1, nb), F, C, r, T, input, gradOutput, nnCount, nnIndex, binIndex, binCoeff,
              (float*)workspace);
    return reduce_partials((const float*)workspace, nb, (int64_t)F * Cr, gradFilter, stream);
}

}  // extern "C"

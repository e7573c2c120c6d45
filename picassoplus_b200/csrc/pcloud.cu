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

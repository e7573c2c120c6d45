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

static bool sizes_ok(int64_t Np, int64_t Mp, int64_t Nout, int F, int C, int r, int T) {
    return Np >= 0 && Mp >= 0 && Nout >= 0 && F > 0 && C > 0 && r > 0 && T > 0 && Np < (1LL << 31) && Mp < (1LL << 31) &&
           Nout < (1LL << 31) && (int64_t)F * C * r * 4 <= 200 * 1024;
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
    PB_LAUNCH("pcloud_conv_fwd", conv_fwd_kernel, persistent_blocks(Mp * C * r, 256, 16), 256, 0, stream, Np, Mp, F, C, r, T,
              input, filter, nnCount, nnIndex, binIndex, binCoeff, rowptr_out, members_out, output);
    return PB200_OK;
}

size_t pb200_pcloud_conv3d_backward_workspace_bytes(int64_t Nout, int F, int C, int r) {
    if (Nout < 0 || F <= 0 || C <= 0 || r <= 0) return 0;
    return align_up((size_t)filter_blocks(Nout) * F * C * r * sizeof(float), 256);
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

// facet2facet entry points: argument checks and the choice between the fp32 FFMA path
// (every shape, fp32-faithful) and the tensor-core path.
#include "common.cuh"

namespace pb {
size_t f2f_simt_fwd_ws(int64_t Nf, int Cin, int Cout, int F);
size_t f2f_simt_bwd_ws(int64_t Nf, int Cin, int Cout, int F);
int f2f_simt_forward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* input, const float* filter,
                     const float* bary, const int32_t* cum, float* output, void* ws, cudaStream_t stream);
int f2f_simt_backward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* gout, const float* input,
                      const float* filter, const float* bary, const int32_t* cum, float* gin, float* gfilter,
                      void* ws, cudaStream_t stream, bool want_gin, bool want_gfilter);
namespace tc {
bool fwd_supported(int Cin, int Cout, int F);
size_t fwd_workspace_bytes(int64_t NiK, int Cin, int Cout, int F, int precision);
int forward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* input, const float* filter,
            const float* bary, const int32_t* cum, float* output, int precision, void* ws, cudaStream_t stream);
int check_async_error(const char* where);
namespace gin {
bool supported(int Cin, int Cout, int F);
bool fits(int Cin, int Cout, int F, int precision);
size_t workspace_bytes(int Cin, int Cout, int F, int precision);
int backward_input(int64_t Nf, int Cin, int Cout, int F, const float* gout, const float* filter, const float* bary,
                   const float* bary_p, int Fp, const int32_t* cum, float* gin, int precision, void* ws,
                   cudaStream_t stream, bool transposed);
}  // namespace gin
namespace gfilter {
bool supported(int Cin, int Cout, int F);
bool fits(int64_t Nf, int Cin, int Cout, int F, int precision);
size_t workspace_bytes(int64_t Nf, int Cin, int Cout, int F, int precision);
int backward_filter(int64_t Nf, int Cin, int Cout, int F, const float* gout, const float* input, const float* bary_p,
                    int Fp, const int32_t* cum, float* gfilter, int precision, void* ws, cudaStream_t stream);
}  // namespace gfilter
int padded_F(int F);
size_t padded_bary_bytes(int64_t NiK, int F);
int pad_bary(int64_t NiK, int F, const float* bary, float* dst, cudaStream_t stream);
int padded_channels(int Cin);
size_t padded_input_bytes(int64_t NiK, int Cin);
int pad_input(int64_t NiK, int Cin, const float* input, float* dst, cudaStream_t stream);
}  // namespace tc
}  // namespace pb

using namespace pb;

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool use_tc_fwd(int Cin, int Cout, int F, int precision) {
    return precision != PB200_PREC_FP32_FFMA && tc::fwd_supported(Cin, Cout, F);
}
static bool use_tc_gf(int64_t Nf, int Cin, int Cout, int F, int precision) {
    return precision != PB200_PREC_FP32_FFMA && tc::gfilter::supported(Cin, Cout, F) &&
           tc::gfilter::fits(Nf, Cin, Cout, F, precision);
}
static bool use_tc_gin(int Cin, int Cout, int F, int precision) {
    return precision != PB200_PREC_FP32_FFMA && tc::gin::supported(Cin, Cout, F) && tc::gin::fits(Cin, Cout, F, precision);
}

static bool f2f_sizes_ok(int64_t Nf, int64_t NiK, int Cin, int Cout, int F) {
    return Nf >= 0 && NiK >= 0 && Cin > 0 && Cout > 0 && F > 0 && F <= 50 && NiK < (1LL << 31) && Nf < (1LL << 31);
}

extern "C" {

size_t pb200_facet2facet_forward_workspace_bytes(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, int precision) {
    if (!f2f_sizes_ok(Nf, NiK, Cin, Cout, F)) return 0;
    if (use_tc_fwd(Cin, Cout, F, precision)) return tc::fwd_workspace_bytes(NiK, Cin, Cout, F, precision);
    return f2f_simt_fwd_ws(Nf, Cin, Cout, F);
}

int pb200_facet2facet_forward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* input,
                              const float* filter, const float* bary, const int32_t* numInterior, float* output,
                              int precision, void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(f2f_sizes_ok(Nf, NiK, Cin, Cout, F), PB200_EINVAL,
               "facet2facet_forward: bad sizes (F must be in 1..50)");
    PB_REQUIRE(precision >= PB200_PREC_FP32 && precision <= PB200_PREC_FP32_TF32X3, PB200_EINVAL,
               "facet2facet_forward: unknown precision %d", precision);
    if (Nf == 0) return PB200_OK;
    PB_REQUIRE(filter && numInterior && output && (NiK == 0 || (input && bary)), PB200_EINVAL,
               "facet2facet_forward: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_facet2facet_forward_workspace_bytes(Nf, NiK, Cin, Cout, F, precision),
               PB200_EWORKSPACE, "facet2facet_forward: workspace too small");
    if (use_tc_fwd(Cin, Cout, F, precision)) {
        PB_REQUIRE(NiK == 0 || aligned16(input), PB200_EINVAL, "facet2facet_forward: input must be 16-byte aligned");
        PB_REQUIRE(aligned16(workspace), PB200_EINVAL, "facet2facet_forward: workspace must be 16-byte aligned");
        return tc::forward(Nf, NiK, Cin, Cout, F, input, filter, bary, numInterior, output, precision, workspace,
                           stream);
    }
    return f2f_simt_forward(Nf, NiK, Cin, Cout, F, input, filter, bary, numInterior, output, workspace, stream);
}

// One sample per face: output[f,co] = sum_d weights[f,d] * (sum_ci input[f,ci] * filter[co,ci,d]).  The inner
// sum is a plain GEMM over the input rows (no face operand of F * Cin products to build, split and store) and
// the outer one an epilogue over the accumulator: the input-gradient kernel with the channel roles exchanged.
static bool one_sample_on_gin(int Cin, int Cout, int F, int precision) { return use_tc_gin(Cout, Cin, F, precision); }

size_t pb200_facet2facet_one_sample_forward_workspace_bytes(int64_t Nf, int Cin, int Cout, int F, int precision) {
    if (!f2f_sizes_ok(Nf, Nf, Cin, Cout, F)) return 0;
    if (one_sample_on_gin(Cin, Cout, F, precision))
        return tc::gin::workspace_bytes(Cout, Cin, F, precision) + tc::padded_bary_bytes(Nf, F);
    return align_up(sizeof(int32_t) * (size_t)(Nf > 0 ? Nf : 1), 256) +
           pb200_facet2facet_forward_workspace_bytes(Nf, Nf, Cin, Cout, F, precision);
}

__global__ void count_up_kernel(int64_t n, int32_t* out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = (int32_t)(i + 1);
}

int pb200_facet2facet_one_sample_forward(int64_t Nf, int Cin, int Cout, int F, const float* input, const float* filter,
                                         const float* weights, const float* weightsPadded, float* output, int precision,
                                         void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(f2f_sizes_ok(Nf, Nf, Cin, Cout, F), PB200_EINVAL, "facet2facet_one_sample_forward: bad sizes (F must be in 1..50)");
    PB_REQUIRE(precision >= PB200_PREC_FP32 && precision <= PB200_PREC_FP32_TF32X3, PB200_EINVAL,
               "facet2facet_one_sample_forward: unknown precision %d", precision);
    if (Nf == 0) return PB200_OK;
    PB_REQUIRE(input && filter && weights && output, PB200_EINVAL, "facet2facet_one_sample_forward: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_facet2facet_one_sample_forward_workspace_bytes(Nf, Cin, Cout, F, precision),
               PB200_EWORKSPACE, "facet2facet_one_sample_forward: workspace too small");
    char* w = (char*)workspace;
    if (one_sample_on_gin(Cin, Cout, F, precision)) {
        PB_REQUIRE(aligned16(input) && aligned16(weights) && aligned16(workspace), PB200_EINVAL,
                   "facet2facet_one_sample_forward: input, weights and workspace must be 16-byte aligned");
        const float* wp = weights;
        const int Fp = tc::padded_F(F);
        if (F % 4 != 0 && weightsPadded) {
            PB_REQUIRE(aligned16(weightsPadded), PB200_EINVAL,
                       "facet2facet_one_sample_forward: weightsPadded must be 16-byte aligned");
            wp = weightsPadded;
        } else if (F % 4 != 0) {
            float* dst = (float*)(w + tc::gin::workspace_bytes(Cout, Cin, F, precision));
            int rc = tc::pad_bary(Nf, F, weights, dst, stream);
            if (rc) return rc;
            wp = dst;
        }
        return tc::gin::backward_input(Nf, Cout, Cin, F, input, filter, weights, wp, Fp, nullptr, output, precision, w,
                                       stream, true);
    }
    int32_t* one_each = (int32_t*)w;
    w += align_up(sizeof(int32_t) * (size_t)Nf, 256);
    PB_LAUNCH("count_up", count_up_kernel, persistent_blocks(Nf, 256, 8), 256, 0, stream, Nf, one_each);
    return pb200_facet2facet_forward(Nf, Nf, Cin, Cout, F, input, filter, weights, one_each, output, precision, w,
                                     workspace_bytes - (size_t)(w - (char*)workspace), stream_);
}

size_t pb200_facet2facet_backward_workspace_bytes(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, int precision) {
    if (!f2f_sizes_ok(Nf, NiK, Cin, Cout, F)) return 0;
    const bool tg = use_tc_gin(Cin, Cout, F, precision), tf = use_tc_gf(Nf, Cin, Cout, F, precision);
    size_t n = (tg && tf) ? 0 : f2f_simt_bwd_ws(Nf, Cin, Cout, F);
    if (tg) n += tc::gin::workspace_bytes(Cin, Cout, F, precision);
    if (tf) n += tc::gfilter::workspace_bytes(Nf, Cin, Cout, F, precision);
    if (tg || tf) n += tc::padded_bary_bytes(NiK, F);
    if (tf) n += tc::padded_input_bytes(NiK, Cin);
    return n;
}

}  // extern "C"

// baryPadded: optional copy of bary with rows padded to padded_F(F) floats (pad columns zero), as pb200_pad_rows
// makes it; given, the tensor-core kernels read it instead of padding bary into the workspace on every call
static int f2f_backward_impl(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* gradOutput,
                             const float* input, const float* filter, const float* bary, const float* baryPadded,
                             const int32_t* numInterior, float* gradInput, float* gradFilter, int precision,
                             void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(f2f_sizes_ok(Nf, NiK, Cin, Cout, F), PB200_EINVAL,
               "facet2facet_backward: bad sizes (F must be in 1..50)");
    PB_REQUIRE(precision >= PB200_PREC_FP32 && precision <= PB200_PREC_FP32_TF32X3, PB200_EINVAL,
               "facet2facet_backward: unknown precision %d", precision);
    PB_REQUIRE(gradFilter, PB200_EINVAL, "facet2facet_backward: null pointer");
    if (Nf == 0) {
        PB_CUDA(cudaMemsetAsync(gradFilter, 0, sizeof(float) * (size_t)Cout * Cin * F, stream));
        return PB200_OK;
    }
    PB_REQUIRE(gradOutput && filter && numInterior && (NiK == 0 || (input && bary && gradInput)), PB200_EINVAL,
               "facet2facet_backward: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_facet2facet_backward_workspace_bytes(Nf, NiK, Cin, Cout, F, precision),
               PB200_EWORKSPACE, "facet2facet_backward: workspace too small");
    const bool tg = use_tc_gin(Cin, Cout, F, precision), tf = use_tc_gf(Nf, Cin, Cout, F, precision);
    if (tg || tf)
        PB_REQUIRE(aligned16(gradOutput) && aligned16(workspace) && (NiK == 0 || (aligned16(input) && aligned16(bary))),
                   PB200_EINVAL, "facet2facet_backward: gradOutput, input, bary and workspace must be 16-byte aligned");
    char* w = (char*)workspace;
    void* simt_ws = w;
    if (!(tg && tf)) w += f2f_simt_bwd_ws(Nf, Cin, Cout, F);
    // both tensor-core kernels read bary rows with 16-byte loads: rows padded to 4 floats
    const float* bary_p = bary;
    const int Fp = tc::padded_F(F);
    if ((tg || tf) && F % 4 != 0 && NiK > 0) {
        if (baryPadded) {
            PB_REQUIRE(aligned16(baryPadded), PB200_EINVAL, "facet2facet_backward: baryPadded must be 16-byte aligned");
            bary_p = baryPadded;
        } else {
            char* wp = w + (tg ? tc::gin::workspace_bytes(Cin, Cout, F, precision) : 0) +
                       (tf ? tc::gfilter::workspace_bytes(Nf, Cin, Cout, F, precision) : 0);
            int rc = tc::pad_bary(NiK, F, bary, (float*)wp, stream);
            if (rc) return rc;
            bary_p = (const float*)wp;
        }
    }
    if (tg) {
        if (NiK > 0) {
            int rc = tc::gin::backward_input(Nf, Cin, Cout, F, gradOutput, filter, bary, bary_p, Fp, numInterior,
                                             gradInput, precision, w, stream, false);
            if (rc) return rc;
        }
        w += tc::gin::workspace_bytes(Cin, Cout, F, precision);
    }
    if (tf) {
        // the filter-gradient kernel reads 16 input channels per CTA with 16-byte copies: channel counts that
        // are not a multiple of 16 go through a zero-padded copy at the end of the workspace
        const float* input_p = input;
        if (Cin % 16 != 0 && NiK > 0) {
            char* wx = (char*)workspace + pb200_facet2facet_backward_workspace_bytes(Nf, NiK, Cin, Cout, F, precision) -
                       tc::padded_input_bytes(NiK, Cin);
            int rc = tc::pad_input(NiK, Cin, input, (float*)wx, stream);
            if (rc) return rc;
            input_p = (const float*)wx;
        }
        int rc = tc::gfilter::backward_filter(Nf, Cin, Cout, F, gradOutput, input_p, bary_p, Fp, numInterior, gradFilter,
                                              precision, w, stream);
        if (rc) return rc;
    }
    if (tg && tf) return PB200_OK;
    return f2f_simt_backward(Nf, NiK, Cin, Cout, F, gradOutput, input, filter, bary, numInterior, gradInput,
                             gradFilter, simt_ws, stream, !tg, !tf);
}

extern "C" {

int pb200_facet2facet_backward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* gradOutput,
                               const float* input, const float* filter, const float* bary,
                               const int32_t* numInterior, float* gradInput, float* gradFilter, int precision,
                               void* workspace, size_t workspace_bytes, void* stream) {
    return f2f_backward_impl(Nf, NiK, Cin, Cout, F, gradOutput, input, filter, bary, nullptr, numInterior, gradInput,
                             gradFilter, precision, workspace, workspace_bytes, stream);
}

int pb200_facet2facet_backward_padded(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* gradOutput,
                                      const float* input, const float* filter, const float* bary, const float* baryPadded,
                                      const int32_t* numInterior, float* gradInput, float* gradFilter, int precision,
                                      void* workspace, size_t workspace_bytes, void* stream) {
    return f2f_backward_impl(Nf, NiK, Cin, Cout, F, gradOutput, input, filter, bary, baryPadded, numInterior, gradInput,
                             gradFilter, precision, workspace, workspace_bytes, stream);
}

int pb200_padded_row_floats(int F) { return F > 0 ? tc::padded_F(F) : 0; }

int pb200_pad_rows(int64_t N, int F, const float* rows, float* out, void* stream) {
    PB_REQUIRE(N >= 0 && F > 0, PB200_EINVAL, "pad_rows: bad sizes");
    if (N == 0) return PB200_OK;
    PB_REQUIRE(rows && out, PB200_EINVAL, "pad_rows: null pointer");
    PB_REQUIRE(aligned16(out), PB200_EINVAL, "pad_rows: out must be 16-byte aligned");
    return tc::pad_bary(N, F, rows, out, (cudaStream_t)stream);
}

}  // extern "C"

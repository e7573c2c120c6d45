// facet2facet, fp32-faithful path for every shape: the per-face basis-weighted means
// A[f,(d,ci)] are built for a chunk of faces in workspace, and the dense (F*Cin) x Cout
// contraction and its two gradients run as fp32 FFMA tile GEMMs over that chunk.
// Deterministic: every sum has one fixed order.
#include "common.cuh"

namespace pb {

// Wt[(d*Cin+ci)*Cout + co] = filter[(co*Cin+ci)*F + d]
__global__ void f2f_transpose_filter_kernel(int F, int Cin, int Cout, const float* __restrict__ filter,
                                            float* __restrict__ Wt) {
    int64_t total = (int64_t)F * Cin * Cout;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int co = (int)(i % Cout);
        int64_t q = i / Cout;
        int ci = (int)(q % Cin);
        int d = (int)(q / Cin);
        Wt[i] = __ldg(filter + ((int64_t)co * Cin + ci) * F + d);
    }
}

// gradFilter[(co*Cin+ci)*F + d] = gWt[(d*Cin+ci)*Cout + co]
__global__ void f2f_untranspose_grad_kernel(int F, int Cin, int Cout, const float* __restrict__ gWt,
                                            float* __restrict__ gfilter) {
    int64_t total = (int64_t)F * Cin * Cout;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int d = (int)(i % F);
        int64_t t = i / F;
        int ci = (int)(t % Cin);
        int co = (int)(t / Cin);
        gfilter[i] = __ldg(gWt + ((int64_t)d * Cin + ci) * Cout + co);
    }
}

// A[(f-f0)*Q + d*Cin + ci] = (1/T_f) sum_{k in f} bary[k,d]*in[k,ci]   (0 when T_f == 0)
__global__ void f2f_build_A_kernel(int64_t f0, int64_t nfaces, int F, int Cin, const int32_t* __restrict__ cum,
                                   const float* __restrict__ bary, const float* __restrict__ in,
                                   float* __restrict__ A) {
    const int Q = F * Cin;
    int64_t total = nfaces * Q;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t fl = i / Q;
        int q = (int)(i - fl * Q);
        int d = q / Cin, ci = q - d * Cin;
        int64_t f = f0 + fl;
        int k0 = f > 0 ? cum[f - 1] : 0, k1 = cum[f];
        float acc = 0.f;
        for (int k = k0; k < k1; ++k)
            acc = fmaf(__ldg(bary + (int64_t)k * F + d), __ldg(in + (int64_t)k * Cin + ci), acc);
        A[i] = k1 > k0 ? acc / (float)(k1 - k0) : 0.f;
    }
}

// C[m*ldc + n] (+)= sum_k A[m*sam + k*sak] * B[k*sbk + n*sbn]; 64x64x16 tiles, 4x4 per thread.
constexpr int GM = 64, GN = 64, GK = 16;

__global__ void __launch_bounds__(256)
sgemm_tile_kernel(int M, int N, int K, const float* __restrict__ A, int64_t sam, int64_t sak,
                  const float* __restrict__ B, int64_t sbk, int64_t sbn, float* __restrict__ C, int64_t ldc,
                  int accumulate) {
    __shared__ float As[GK][GM + 4];
    __shared__ float Bs[GK][GN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.x * GM, n0 = blockIdx.y * GN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const bool a_kfast = (sak == 1);
    const bool b_kfast = (sbk == 1 && sbn != 1);
    for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            int e = tid + it * 256;
            int m, k;
            if (a_kfast) { k = e & (GK - 1); m = e >> 4; } else { m = e & (GM - 1); k = e >> 6; }
            int gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < M && gk < K) ? __ldg(A + gm * sam + gk * sak) : 0.f;
            int n, kb;
            if (b_kfast) { kb = e & (GK - 1); n = e >> 4; } else { n = e & (GN - 1); kb = e >> 6; }
            int gn = n0 + n, gkb = k0 + kb;
            Bs[kb][n] = (gn < N && gkb < K) ? __ldg(B + gkb * sbk + gn * sbn) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float* c = C + gm * ldc + gn;
            *c = accumulate ? (*c + acc[i][j]) : acc[i][j];
        }
    }
}

static int sgemm(cudaStream_t stream, const char* name, int64_t M, int64_t N, int64_t K, const float* A, int64_t sam,
                 int64_t sak, const float* B, int64_t sbk, int64_t sbn, float* C, int64_t ldc, int accumulate) {
    if (M <= 0 || N <= 0) return PB200_OK;
    dim3 grid((unsigned)ceil_div(M, GM), (unsigned)ceil_div(N, GN));
    PB_LAUNCH(name, sgemm_tile_kernel, grid, 256, 0, stream, (int)M, (int)N, (int)K, A, sam, sak, B, sbk, sbn, C, ldc,
              accumulate);
    return PB200_OK;
}

// faces per workspace chunk: about 96 MB of A rows, at least 64 faces
int64_t f2f_chunk_faces(int64_t Nf, int Q) {
    int64_t fc = ((int64_t)96 << 20) / ((int64_t)Q * 4);
    fc = fc / 64 * 64;
    if (fc < 64) fc = 64;
    if (fc > Nf) fc = Nf > 0 ? Nf : 1;
    return fc;
}

size_t f2f_simt_fwd_ws(int64_t Nf, int Cin, int Cout, int F) {
    int Q = F * Cin;
    return align_up(sizeof(float) * (size_t)Q * Cout, 256) +
           align_up(sizeof(float) * (size_t)f2f_chunk_faces(Nf, Q) * Q, 256);
}

size_t f2f_simt_bwd_ws(int64_t Nf, int Cin, int Cout, int F) {
    int Q = F * Cin;
    return 2 * align_up(sizeof(float) * (size_t)Q * Cout, 256) +
           2 * align_up(sizeof(float) * (size_t)f2f_chunk_faces(Nf, Q) * Q, 256);
}

int f2f_simt_forward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* input, const float* filter,
                     const float* bary, const int32_t* cum, float* output, void* ws, cudaStream_t stream) {
    const int Q = F * Cin;
    char* w = (char*)ws;
    float* Wt = (float*)w; w += align_up(sizeof(float) * (size_t)Q * Cout, 256);
    float* A = (float*)w;
    int64_t FC = f2f_chunk_faces(Nf, Q);
    PB_LAUNCH("f2f_transpose_filter", f2f_transpose_filter_kernel, persistent_blocks((int64_t)Q * Cout, 256, 8), 256, 0,
              stream, F, Cin, Cout, filter, Wt);
    for (int64_t f0 = 0; f0 < Nf; f0 += FC) {
        int64_t nf = Nf - f0 < FC ? Nf - f0 : FC;
        PB_LAUNCH("f2f_build_A", f2f_build_A_kernel, persistent_blocks(nf * Q, 256, 16), 256, 0, stream, f0, nf, F, Cin,
                  cum, bary, input, A);
        int rc = sgemm(stream, "f2f_fwd_sgemm", nf, Cout, Q, A, Q, 1, Wt, Cout, 1, output + f0 * Cout, Cout, 0);
        if (rc) return rc;
    }
    return PB200_OK;
}

// gradInput[k,ci] = (1/T_f) sum_d bary[k,d]*gA[(f-f0)*Q + d*Cin + ci] for the samples of the
// chunk; the chunk's sample range is read from `cum` on the device (no host round trip).
__global__ void f2f_gin_all_kernel(int64_t f0, int64_t nfaces, int64_t Nf, int F, int Cin,
                                   const int32_t* __restrict__ cum, const float* __restrict__ bary,
                                   const float* __restrict__ gA, float* __restrict__ gin) {
    int64_t k_begin = f0 > 0 ? cum[f0 - 1] : 0;
    int64_t k_end = cum[f0 + nfaces - 1];
    const int Q = F * Cin;
    int64_t total = (k_end - k_begin) * Cin;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t k = k_begin + i / Cin;
        int ci = (int)(i % Cin);
        int64_t lo = f0, hi = f0 + nfaces;
        while (lo < hi) {
            int64_t mid = (lo + hi) >> 1;
            if (cum[mid] > k) hi = mid; else lo = mid + 1;
        }
        int64_t f = lo;
        int ks = f > 0 ? cum[f - 1] : 0;
        float T = (float)(cum[f] - ks);
        const float* g = gA + (f - f0) * Q + ci;
        const float* b = bary + k * F;
        float acc = 0.f;
        for (int d = 0; d < F; ++d) acc = fmaf(__ldg(b + d), __ldg(g + (int64_t)d * Cin), acc);
        gin[k * Cin + ci] = acc / T;
    }
}

// want_gin / want_gfilter = false skip that half (the caller computes it elsewhere)
int f2f_simt_backward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* gout, const float* input,
                      const float* filter, const float* bary, const int32_t* cum, float* gin, float* gfilter,
                      void* ws, cudaStream_t stream, bool want_gin, bool want_gfilter) {
    const int Q = F * Cin;
    char* w = (char*)ws;
    float* Wt = (float*)w;  w += align_up(sizeof(float) * (size_t)Q * Cout, 256);
    float* gWt = (float*)w; w += align_up(sizeof(float) * (size_t)Q * Cout, 256);
    int64_t FC = f2f_chunk_faces(Nf, Q);
    float* A = (float*)w;   w += align_up(sizeof(float) * (size_t)FC * Q, 256);
    float* gA = (float*)w;
    PB_LAUNCH("f2f_transpose_filter", f2f_transpose_filter_kernel, persistent_blocks((int64_t)Q * Cout, 256, 8), 256, 0,
              stream, F, Cin, Cout, filter, Wt);
    PB_CUDA(cudaMemsetAsync(gWt, 0, sizeof(float) * (size_t)Q * Cout, stream));
    for (int64_t f0 = 0; f0 < Nf; f0 += FC) {
        int64_t nf = Nf - f0 < FC ? Nf - f0 : FC;
        int rc = PB200_OK;
        if (want_gfilter) {
            PB_LAUNCH("f2f_build_A", f2f_build_A_kernel, persistent_blocks(nf * Q, 256, 16), 256, 0, stream, f0, nf, F,
                      Cin, cum, bary, input, A);
            // gWt[Q x Cout] += A^T[Q x nf] @ gout[nf x Cout]
            rc = sgemm(stream, "f2f_gfilter_sgemm", Q, Cout, nf, A, 1, Q, gout + f0 * Cout, Cout, 1, gWt, Cout, 1);
            if (rc) return rc;
        }
        if (!want_gin) continue;
        // gA[nf x Q] = gout[nf x Cout] @ Wt^T[Cout x Q]
        rc = sgemm(stream, "f2f_gA_sgemm", nf, Q, Cout, gout + f0 * Cout, Cout, 1, Wt, 1, Cout, gA, Q, 0);
        if (rc) return rc;
        if (NiK > 0)
            PB_LAUNCH("f2f_gin_from_gA", f2f_gin_all_kernel, persistent_blocks(nf * 3 * Cin, 256, 16), 256, 0, stream,
                      f0, nf, Nf, F, Cin, cum, bary, (const float*)gA, gin);
    }
    if (want_gfilter)
        PB_LAUNCH("f2f_untranspose_grad", f2f_untranspose_grad_kernel, persistent_blocks((int64_t)Q * Cout, 256, 8), 256,
                  0, stream, F, Cin, Cout, (const float*)gWt, gfilter);
    return PB200_OK;
}

}  // namespace pb

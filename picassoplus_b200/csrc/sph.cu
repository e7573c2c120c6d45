// Spherical-harmonic basis of (N,3) cartesian points: projection to the unit sphere,
// azimuth / polar angles, and the (L+1)^2 real components in the reference's column
// order (per degree l: cos(m*phi) terms m = l..1, the m = 0 term, sin(m*phi) terms
// m = l..1), L <= 5.  One thread per point; the K outputs are staged through shared
// memory so the global store is coalesced.
#include "common.cuh"
#include "sph_core.cuh"

namespace pb {

constexpr int SPH_BLOCK = 128;

__global__ void __launch_bounds__(SPH_BLOCK)
sph_harm_kernel(int64_t N, int L, const float* __restrict__ xyz, SphConst cst, float* __restrict__ out) {
    extern __shared__ float stage[];            // [SPH_BLOCK][K+1]
    const int K = (L + 1) * (L + 1);
    const int KP = K + 1;
    const float* c = cst.c;
    int64_t base = (int64_t)blockIdx.x * SPH_BLOCK;
    int64_t i = base + threadIdx.x;
    if (i < N) {
        sph_eval(xyz[3 * i], xyz[3 * i + 1], xyz[3 * i + 2], L, c, stage + threadIdx.x * KP);
    }
    __syncthreads();
    int64_t npts = N - base < SPH_BLOCK ? N - base : SPH_BLOCK;
    float* dst = out + base * K;
    for (int64_t j = threadIdx.x; j < npts * K; j += SPH_BLOCK) {
        int p = (int)(j / K), k = (int)(j - (int64_t)p * K);
        dst[j] = stage[p * KP + k];
    }
}

// out[f] = mean over the samples k of face f of the components of xyz[k] (0 for a face without samples): the two
// steps sph_harm + per-face mean of the rows in one pass, without the (samples, K) array in between.  A thread walks
// its face's samples in ascending order and adds each evaluation to its row in shared memory, so the result has the
// bits of the two-step path.
__global__ void __launch_bounds__(SPH_BLOCK)
face_mean_sph_harm_kernel(int64_t Nf, int64_t NiK, int L, const float* __restrict__ xyz, const int32_t* __restrict__ cum,
                          SphConst cst, float* __restrict__ out) {
    extern __shared__ float stage[];            // [SPH_BLOCK][K+1] sums, then [SPH_BLOCK][K+1] one evaluation
    const int K = (L + 1) * (L + 1);
    const int KP = K + 1;
    const float* c = cst.c;
    float* acc = stage + threadIdx.x * KP;
    float* one = stage + (SPH_BLOCK + threadIdx.x) * KP;
    const int64_t base = (int64_t)blockIdx.x * SPH_BLOCK;
    const int64_t f = base + threadIdx.x;
    if (f < Nf) {
        int64_t k0 = f > 0 ? cum[f - 1] : 0, k1 = cum[f];
        if (k0 < 0) k0 = 0;
        if (k1 > NiK) k1 = NiK;
        for (int k = 0; k < K; ++k) acc[k] = 0.f;
        for (int64_t i = k0; i < k1; ++i) {
            sph_eval(xyz[3 * i], xyz[3 * i + 1], xyz[3 * i + 2], L, c, one);
            for (int k = 0; k < K; ++k) acc[k] += one[k];
        }
        const float inv = k1 > k0 ? 1.f / (float)(k1 - k0) : 0.f;
        for (int k = 0; k < K; ++k) acc[k] *= inv;
    }
    __syncthreads();
    const int64_t nrows = Nf - base < SPH_BLOCK ? Nf - base : SPH_BLOCK;
    float* dst = out + base * K;
    for (int64_t j = threadIdx.x; j < nrows * K; j += SPH_BLOCK) {
        int r = (int)(j / K), k = (int)(j - (int64_t)r * K);
        dst[j] = stage[r * KP + k];
    }
}

}  // namespace pb

using namespace pb;

extern "C" int pb200_face_mean_sph_harm(int64_t Nf, int64_t NiK, int L, const float* xyz, const int32_t* numInterior,
                                        float* out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NiK >= 0, PB200_EINVAL, "face_mean_sph_harm: bad size");
    PB_REQUIRE(L >= 0 && L <= 5, PB200_EINVAL, "face_mean_sph_harm: degree L=%d not supported (0..5)", L);
    if (Nf == 0) return PB200_OK;
    PB_REQUIRE(numInterior && out && (NiK == 0 || xyz), PB200_EINVAL, "face_mean_sph_harm: null pointer");
    static const SphConst cst = make_sph_const();
    int K = (L + 1) * (L + 1);
    size_t smem = sizeof(float) * 2 * SPH_BLOCK * (K + 1);
    PB_LAUNCH("face_mean_sph_harm", face_mean_sph_harm_kernel, (unsigned)ceil_div(Nf, SPH_BLOCK), SPH_BLOCK, smem, stream, Nf,
              NiK, L, xyz, numInterior, cst, out);
    return PB200_OK;
}

extern "C" int pb200_sph_harm_coeff(int64_t N, int L, const float* xyz, float* out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(N >= 0, PB200_EINVAL, "sph_harm_coeff: bad size");
    PB_REQUIRE(L >= 0 && L <= 5, PB200_EINVAL, "sph_harm_coeff: degree L=%d not supported (0..5)", L);
    if (N == 0) return PB200_OK;
    PB_REQUIRE(xyz && out, PB200_EINVAL, "sph_harm_coeff: null pointer");
    static const SphConst cst = make_sph_const();
    int K = (L + 1) * (L + 1);
    size_t smem = sizeof(float) * SPH_BLOCK * (K + 1);
    PB_LAUNCH("sph_harm", sph_harm_kernel, (unsigned)ceil_div(N, SPH_BLOCK), SPH_BLOCK, smem, stream, N, L, xyz, cst, out);
    return PB200_OK;
}

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

}  // namespace pb

using namespace pb;

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

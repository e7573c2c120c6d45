// facet2vertex: forward as a vertex-centred pull over the CSR (segmented sum in a fixed
// order, no atomics); backward as a face-centred gather that yields the input gradient
// and per-thread filter-gradient partials in one pass.
#include "common.cuh"

namespace pb {

// -------------------------------------------------------------------- forward, vectorised
// r == 1, C % 4 == 0, K <= 64.  Two kernels:
//   f2v_fwd_face    item = (face, float4 channel group): wx[f] = (sum_k coeff[f,k]*filter[k]) * input[f],
//                   once per face (a vertex-centred pull would evaluate the K-term sum three
//                   times per face), filter and the tile's coeff rows in shared memory;
//   f2v_fwd_gather  team per output vertex: sum of the wx rows of its CSR entries in ascending
//                   order, times 1/nfCount.  No atomics: deterministic.
constexpr int F2VF_TF = 64;

__global__ void __launch_bounds__(256)
f2v_fwd_face_kernel(int64_t Nf, int CV, int K, const float* __restrict__ coeff, const float4* __restrict__ in,
                    const float4* __restrict__ filt, float4* __restrict__ wx) {
    extern __shared__ float4 smem[];
    const int KP = (K + 3) / 4 * 4 + 4;
    float4* sfilt = smem;                                          // [K][32]
    float* scoef = reinterpret_cast<float*>(smem + K * 32);       // [TF][KP]
    const int cg0 = blockIdx.y * 32;
    const int CVc = CV - cg0 < 32 ? CV - cg0 : 32;
    for (int i = threadIdx.x; i < K * 32; i += blockDim.x) {
        int k = i >> 5, l = i & 31;
        sfilt[i] = l < CVc ? filt[k * CV + cg0 + l] : zero4();
    }
    const int64_t ntiles = (Nf + F2VF_TF - 1) / F2VF_TF;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int64_t f0 = tile * F2VF_TF;
        const int nf_tile = Nf - f0 < F2VF_TF ? (int)(Nf - f0) : F2VF_TF;
        __syncthreads();
        for (int i = threadIdx.x; i < nf_tile * K; i += blockDim.x) {
            int fl = i / K;
            scoef[fl * KP + (i - fl * K)] = __ldg(coeff + f0 * K + i);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nf_tile * CVc; i += blockDim.x) {
            const int fl = i / CVc, c = i - fl * CVc;
            const int64_t f = f0 + fl;
            const float4 x = ldg4(in + f * CV + cg0 + c);
            const float* cf = scoef + fl * KP;
            float4 w = zero4();
            int k = 0;
            for (; k + 4 <= K; k += 4) {
                const float4 c4 = *reinterpret_cast<const float4*>(cf + k);
                fma4s(w, c4.x, sfilt[k * 32 + c]);
                fma4s(w, c4.y, sfilt[(k + 1) * 32 + c]);
                fma4s(w, c4.z, sfilt[(k + 2) * 32 + c]);
                fma4s(w, c4.w, sfilt[(k + 3) * 32 + c]);
            }
            for (; k < K; ++k) fma4s(w, cf[k], sfilt[k * 32 + c]);
            wx[f * CV + cg0 + c] = mul4(w, x);
        }
    }
}

// The same for whole 128-channel chunks (lane = float4 channel group) and K <= 32, register-
// blocked so that the shared-memory pipe is not the limit: warp w owns faces w, w+8, ..., w+56
// of the tile, and a filter row read from shared memory (512 distinct bytes per warp) is used
// for all eight; the coefficient loads are one broadcast address per warp.  The coefficient
// rows of the next tile arrive by 4-byte asynchronous copies while this tile is computed.
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(256)
f2v_fwd_face_blocked_kernel(int64_t Nf, int CV, int K, const float* __restrict__ coeff, const float4* __restrict__ in,
                            const float4* __restrict__ filt, float4* __restrict__ wx) {
    extern __shared__ float4 smem[];
    constexpr int FB = F2VF_TF / 8;                            // faces per warp
    const int KP = (K + 3) / 4 * 4, KG = KP / 4;               // coeff row pitch, pad columns zero
    float4* sfilt = smem;                                      // [KP][32], rows K..KP-1 zero
    float4* scoef0 = smem + KP * 32;                           // [2][TF][KG], double-buffered
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cg = blockIdx.y * 32 + lane;
    for (int i = threadIdx.x; i < KP * 32; i += blockDim.x) {
        const int k = i >> 5;
        sfilt[i] = k < K ? filt[k * CV + blockIdx.y * 32 + (i & 31)] : zero4();
    }
    for (int i = threadIdx.x; i < 2 * F2VF_TF * KG; i += blockDim.x) scoef0[i] = zero4();
    __syncthreads();
    const int64_t ntiles = (Nf + F2VF_TF - 1) / F2VF_TF;
    auto fetch_coef = [&](int64_t tile, int buf) {             // the pad columns stay zero
        if (tile < ntiles) {
            const int64_t f0 = tile * F2VF_TF;
            const int nf_tile = Nf - f0 < F2VF_TF ? (int)(Nf - f0) : F2VF_TF;
            float* sc = reinterpret_cast<float*>(scoef0 + buf * F2VF_TF * KG);
            for (int i = threadIdx.x; i < nf_tile * K; i += blockDim.x) {
                const int fl = i / K;
                cp_async4(sc + fl * KP + (i - fl * K), coeff + f0 * K + i);
            }
        }
        cp_async_commit();
    };
    fetch_coef(blockIdx.x, 0);
    int buf = 0;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, buf ^= 1) {
        const int64_t f0 = tile * F2VF_TF;
        const int nf_tile = Nf - f0 < F2VF_TF ? (int)(Nf - f0) : F2VF_TF;
        fetch_coef(tile + gridDim.x, buf ^ 1);                 // its readers finished behind the barrier below
        cp_async_wait<1>();                                    // this tile's rows have landed (own copies) ...
        __syncthreads();                                       // ... and everybody else's
        const float4* scoef = scoef0 + buf * F2VF_TF * KG;
        float4 x[FB], w[FB];
#pragma unroll
        for (int i = 0; i < FB; ++i) {
            const int fl = warp + 8 * i;
            w[i] = zero4();
            x[i] = fl < nf_tile ? ldg4(in + (f0 + fl) * CV + cg) : zero4();
        }
        for (int g = 0; g < KG; ++g) {
            const float4 f0v = sfilt[(4 * g) * 32 + lane], f1v = sfilt[(4 * g + 1) * 32 + lane];
            const float4 f2v = sfilt[(4 * g + 2) * 32 + lane], f3v = sfilt[(4 * g + 3) * 32 + lane];
#pragma unroll
            for (int i = 0; i < FB; ++i) {
                const float4 cf = scoef[(warp + 8 * i) * KG + g];        // rows past the tile are stale or zero: unused
                fma4s(w[i], cf.x, f0v); fma4s(w[i], cf.y, f1v); fma4s(w[i], cf.z, f2v); fma4s(w[i], cf.w, f3v);
            }
        }
#pragma unroll
        for (int i = 0; i < FB; ++i) {
            const int fl = warp + 8 * i;
            if (fl < nf_tile) wx[(f0 + fl) * CV + cg] = mul4(w[i], x[i]);
        }
        __syncthreads();                                       // this tile's buffer may be refilled now
    }
    cp_async_wait<0>();
}

template <int TL>
__global__ void __launch_bounds__(256)
f2v_fwd_gather_kernel(int64_t NvOut, int CV, const int32_t* __restrict__ rowptr, const int32_t* __restrict__ entries,
                      const int32_t* __restrict__ nfCount, const float4* __restrict__ wx, float4* __restrict__ out) {
    const int lane = threadIdx.x % TL;
    const int team = threadIdx.x / TL;
    const int teams = blockDim.x / TL;
    const int cg = blockIdx.y * 32 + lane;
    const bool active = cg < CV;
    // inactive lanes stay in the loop: the team shares its CSR entries through shuffles
    const unsigned tmask = TL == 32 ? 0xffffffffu : (((1u << TL) - 1u) << ((threadIdx.x & 31) / TL * TL));
    for (int64_t v = (int64_t)blockIdx.x * teams + team; v < NvOut; v += (int64_t)gridDim.x * teams) {
        const int beg = __ldg(rowptr + v), end = __ldg(rowptr + v + 1);
        float4 acc = zero4();
        for (int base = beg; base < end; base += TL) {
            const int mine = base + lane < end ? __ldg(entries + base + lane) : 0;
            const int cnt = end - base < TL ? end - base : TL;
            for (int i = 0; i < cnt; ++i) {
                const int64_t f = __shfl_sync(tmask, mine, i, TL) >> 2;
                if (active) add4(acc, ldg4(wx + f * CV + cg));
            }
        }
        if (active) {
            if (end > beg) acc = scale4(acc, 1.f / (float)__ldg(nfCount + v));
            __stcs(out + v * CV + cg, acc);
        }
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
// r == 1, C % 4 == 0, any K <= 64.  A block walks tiles of 32 faces; per tile
//   phase 1  item = (face, float4 channel group): gt = sum over the three corners of
//            gradOutput[vo] * (1/nfCount[vo]);  w = sum_k coeff[f,k]*filter[k];
//            gradInput[f] = gt*w;  t[f] = input[f]*gt is parked in shared memory;
//   phase 2  item = (k, channel group), up to NACC per thread, kept in registers for the whole
//            kernel: gradFilter[k] += coeff[f,k] * t[f] over the tile's faces in face order.
// Phase 1 needs few registers (full occupancy hides the gather latency), phase 2 has no
// global traffic.  Per-block accumulators go to partial[block][K][C]; a second kernel adds
// the blocks in order, so the result is deterministic.
constexpr int F2VB_TF = 32;

template <int NACC>
__global__ void __launch_bounds__(256)
f2v_bwd_tile_kernel(int64_t Nf, int CV, int K, const int32_t* __restrict__ face, const int32_t* __restrict__ vtMap,
                    const int32_t* __restrict__ nfCount, const float* __restrict__ coeff,
                    const float4* __restrict__ in, const float4* __restrict__ filt, const float4* __restrict__ gout,
                    float4* __restrict__ gin, float4* __restrict__ partial) {
    extern __shared__ float4 smem[];
    const int KP = (K + 3) / 4 * 4 + 4;                       // coeff row pitch (floats): 16-byte rows, spread banks
    float4* sfilt = smem;                                      // [K][32]
    float4* st = smem + K * 32;                                // [TF][32]   t = input * gt
    float* scoef = reinterpret_cast<float*>(st + F2VB_TF * 32);    // [TF][KP]
    const int cg0 = blockIdx.y * 32;
    const int CVc = CV - cg0 < 32 ? CV - cg0 : 32;             // channel groups of this chunk
    for (int i = threadIdx.x; i < K * 32; i += blockDim.x) {
        int k = i >> 5, l = i & 31;
        sfilt[i] = l < CVc ? filt[k * CV + cg0 + l] : zero4();
    }
    // this thread's accumulator items (k, c): j = tid + 256 n
    float4 acc[NACC];
    int ak[NACC], ac[NACC];
#pragma unroll
    for (int n = 0; n < NACC; ++n) {
        int j = threadIdx.x + 256 * n;
        ak[n] = j / CVc; ac[n] = j - ak[n] * CVc;
        if (ak[n] >= K) { ak[n] = -1; ac[n] = 0; }
        acc[n] = zero4();
    }
    const int64_t ntiles = (Nf + F2VB_TF - 1) / F2VB_TF;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int64_t f0 = tile * F2VB_TF;
        const int nf_tile = Nf - f0 < F2VB_TF ? (int)(Nf - f0) : F2VB_TF;
        __syncthreads();                                       // previous tile fully consumed
        for (int i = threadIdx.x; i < nf_tile * K; i += blockDim.x) {
            int fl = i / K;
            scoef[fl * KP + (i - fl * K)] = __ldg(coeff + f0 * K + i);
        }
        __syncthreads();
        // ---- phase 1
        for (int i = threadIdx.x; i < nf_tile * CVc; i += blockDim.x) {
            const int fl = i / CVc, c = i - fl * CVc;
            const int64_t f = f0 + fl;
            const int cg = cg0 + c;
            float4 gt = zero4();
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                int vi = __ldg(face + 3 * f + j);
                int vo = vtMap ? __ldg(vtMap + vi) : vi;
                if (vo >= 0) {
                    float rn = __frcp_rn((float)__ldg(nfCount + vo));
                    fma4s(gt, rn, ldg4(gout + (int64_t)vo * CV + cg));
                }
            }
            const float4 x = ldg4(in + f * CV + cg);
            const float* cf = scoef + fl * KP;
            float4 w = zero4();
            int k = 0;
            for (; k + 4 <= K; k += 4) {
                const float4 c4 = *reinterpret_cast<const float4*>(cf + k);
                fma4s(w, c4.x, sfilt[k * 32 + c]);
                fma4s(w, c4.y, sfilt[(k + 1) * 32 + c]);
                fma4s(w, c4.z, sfilt[(k + 2) * 32 + c]);
                fma4s(w, c4.w, sfilt[(k + 3) * 32 + c]);
            }
            for (; k < K; ++k) fma4s(w, cf[k], sfilt[k * 32 + c]);
            __stcs(gin + f * CV + cg, mul4(gt, w));
            st[fl * 32 + c] = mul4(x, gt);
        }
        __syncthreads();
        // ---- phase 2
#pragma unroll
        for (int n = 0; n < NACC; ++n) {
            if (ak[n] >= 0) {
                const float* cf = scoef + ak[n];
                const float4* tp = st + ac[n];
                float4 a = acc[n];
                for (int fl = 0; fl < nf_tile; ++fl) fma4s(a, cf[fl * KP], tp[fl * 32]);
                acc[n] = a;
            }
        }
    }
#pragma unroll
    for (int n = 0; n < NACC; ++n)
        if (ak[n] >= 0) partial[((int64_t)blockIdx.x * K + ak[n]) * CV + cg0 + ac[n]] = acc[n];
}

// The same two phases, register-blocked for whole 128-channel chunks (lane = float4 channel
// group) and K <= 32, so that the shared-memory pipe is not the limit: every 16-byte shared
// load of a warp is either 512 distinct bytes or one broadcast address.
//   phase 1  warp w owns faces w, w+8, w+16, w+24 of the tile: a filter row read from shared
//            memory is used for all four faces;
//   phase 2  warp g owns the coefficients 4g..4g+3: a row of t read from shared memory feeds
//            four accumulators.
// The index chain of the gather (face -> vtMap -> nfCount) is resolved by 96 threads one hop
// per tile for the block's next three tiles, so that phase 1 finds output vertex and 1/nfCount
// of every corner in shared memory and issues its twelve gradOutput row loads at once.
__global__ void __launch_bounds__(256, 2)
f2v_bwd_blocked_kernel(int64_t Nf, int CV, int K, const int32_t* __restrict__ face, const int32_t* __restrict__ vtMap,
                       const int32_t* __restrict__ nfCount, const float* __restrict__ coeff,
                       const float4* __restrict__ in, const float4* __restrict__ filt, const float4* __restrict__ gout,
                       float4* __restrict__ gin, float4* __restrict__ partial) {
    extern __shared__ float4 smem[];
    const int KP = (K + 3) / 4 * 4;                            // coeff row pitch (floats), pad columns zero
    const int KG = KP / 4;                                     // groups of 4 coefficients (<= 8)
    float4* sfilt = smem;                                      // [KP][32], rows K..KP-1 zero
    float4* st = smem + KP * 32;                               // [TF][32]   t = input * gt
    float4* scoef0 = st + F2VB_TF * 32;                        // [2][TF][KG], double-buffered (asynchronous copies)
    int* svo = reinterpret_cast<int*>(scoef0 + 2 * F2VB_TF * KG);   // [2][96] output vertex of (face, corner), -1 = none
    float* srn = reinterpret_cast<float*>(svo + 2 * 96);       // [2][96] 1 / nfCount of that vertex
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cg = blockIdx.y * 32 + lane;                     // this lane's channel group
    for (int i = threadIdx.x; i < KP * 32; i += blockDim.x) {
        const int k = i >> 5;
        sfilt[i] = k < K ? filt[k * CV + blockIdx.y * 32 + (i & 31)] : zero4();
    }
    for (int i = threadIdx.x; i < 2 * F2VB_TF * KG; i += blockDim.x) scoef0[i] = zero4();
    float4 acc[4] = {zero4(), zero4(), zero4(), zero4()};     // coefficients 4*warp .. 4*warp+3
    const int64_t ntiles = (Nf + F2VB_TF - 1) / F2VB_TF;
    // index pipeline of thread e < 96 (entry e = 3*face + corner of a tile): vertex id of the
    // tile three steps ahead, output vertex two steps ahead, 1/nfCount one step ahead
    const bool ix = threadIdx.x < 96;
    auto hop_face = [&](int64_t tile) -> int {
        const int64_t e = tile * (F2VB_TF * 3) + threadIdx.x;
        return (ix && tile < ntiles && e < Nf * 3) ? __ldg(face + e) : -1;
    };
    auto hop_vo = [&](int vi) -> int { return vi < 0 ? -1 : (vtMap ? __ldg(vtMap + vi) : vi); };
    auto hop_rn = [&](int vo) -> float { return vo < 0 ? 0.f : __frcp_rn((float)__ldg(nfCount + vo)); };
    const int64_t tstep = gridDim.x;
    int vo1 = hop_vo(hop_face(blockIdx.x));                                   // first tile: resolved up front
    float rn1 = hop_rn(vo1);
    if (ix) { svo[threadIdx.x] = vo1; srn[threadIdx.x] = rn1; }
    vo1 = hop_vo(hop_face(blockIdx.x + tstep));                               // second tile
    int vi2 = hop_face(blockIdx.x + 2 * tstep);                               // third tile
    auto fetch_coef = [&](int64_t tile, int b) {               // the pad columns stay zero
        if (tile < ntiles) {
            const int64_t f0 = tile * F2VB_TF;
            const int nf_tile = Nf - f0 < F2VB_TF ? (int)(Nf - f0) : F2VB_TF;
            float* sc = reinterpret_cast<float*>(scoef0 + b * F2VB_TF * KG);
            for (int i = threadIdx.x; i < nf_tile * K; i += blockDim.x) {
                const int fl = i / K;
                cp_async4(sc + fl * KP + (i - fl * K), coeff + f0 * K + i);
            }
        }
        cp_async_commit();
    };
    __syncthreads();                                           // the zero fill above is complete
    fetch_coef(blockIdx.x, 0);
    int buf = 0;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += tstep, buf ^= 1) {
        const int64_t f0 = tile * F2VB_TF;
        const int nf_tile = Nf - f0 < F2VB_TF ? (int)(Nf - f0) : F2VB_TF;
        // one hop for each of the next three tiles (results are used in the next iteration)
        const float rn_next = hop_rn(vo1);
        const int vo_next = hop_vo(vi2);
        const int vi_next = hop_face(tile + 3 * tstep);
        __syncthreads();                                       // previous tile fully consumed
        fetch_coef(tile + tstep, buf ^ 1);                     // the next tile's coefficient rows, asynchronously
        cp_async_wait<1>();                                    // this tile's rows have landed (own copies) ...
        __syncthreads();                                       // ... and everybody else's
        const float4* scoef = scoef0 + buf * F2VB_TF * KG;
        // ---- phase 1: faces warp, warp+8, warp+16, warp+24
        // all sixteen row loads of the warp's four faces are issued first; the filter sums below need
        // only the coefficients and run while the rows are on their way
        float4 gt[4], x[4], w[4], gr[4][3];
        float rn[4][3];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int fl = warp + 8 * i;
            x[i] = zero4(); w[i] = zero4();
#pragma unroll
            for (int j = 0; j < 3; ++j) { gr[i][j] = zero4(); rn[i][j] = 0.f; }
            if (fl < nf_tile) {
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int vo = svo[buf * 96 + fl * 3 + j];
                    rn[i][j] = srn[buf * 96 + fl * 3 + j];
                    if (vo >= 0) gr[i][j] = ldg4(gout + (int64_t)vo * CV + cg);
                }
                x[i] = ldg4(in + (f0 + fl) * CV + cg);
            }
        }
        for (int g = 0; g < KG; ++g) {
            float4 cf[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) cf[i] = scoef[(warp + 8 * i) * KG + g];   // rows past the tile are stale or zero: unused
            const float4 f0v = sfilt[(4 * g) * 32 + lane], f1v = sfilt[(4 * g + 1) * 32 + lane];
            const float4 f2v = sfilt[(4 * g + 2) * 32 + lane], f3v = sfilt[(4 * g + 3) * 32 + lane];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                fma4s(w[i], cf[i].x, f0v); fma4s(w[i], cf[i].y, f1v); fma4s(w[i], cf[i].z, f2v); fma4s(w[i], cf[i].w, f3v);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            gt[i] = zero4();
#pragma unroll
            for (int j = 0; j < 3; ++j) fma4s(gt[i], rn[i][j], gr[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int fl = warp + 8 * i;
            if (fl < nf_tile) {
                __stcs(gin + (f0 + fl) * CV + cg, mul4(gt[i], w[i]));
                st[fl * 32 + lane] = mul4(x[i], gt[i]);
            }
        }
        __syncthreads();
        // the next tile's corners go to the other index buffer (its readers are behind the barrier above)
        if (ix) { svo[(buf ^ 1) * 96 + threadIdx.x] = vo1; srn[(buf ^ 1) * 96 + threadIdx.x] = rn_next; }
        vo1 = vo_next; vi2 = vi_next;
        // ---- phase 2: coefficients 4*warp .. 4*warp+3, faces in order
        if (warp < KG) {
#pragma unroll 4
            for (int fl = 0; fl < nf_tile; ++fl) {
                const float4 c = scoef[fl * KG + warp];
                const float4 t = st[fl * 32 + lane];
                fma4s(acc[0], c.x, t); fma4s(acc[1], c.y, t); fma4s(acc[2], c.z, t); fma4s(acc[3], c.w, t);
            }
        }
    }
    cp_async_wait<0>();
    if (warp < KG) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = 4 * warp + j;
            if (k < K) partial[((int64_t)blockIdx.x * K + k) * CV + cg] = acc[j];
        }
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
static bool kt_ok(int K) { return K >= 1 && K <= 64; }

struct F2VBwdPlan { bool vec; int grid_x; int64_t faces_per_chunk; };
static F2VBwdPlan f2v_bwd_plan(int64_t Nf, int C, int r, int K) {
    F2VBwdPlan p;
    p.vec = vec_ok(C, r) && kt_ok(K);
    int64_t n = Nf > 0 ? Nf : 1;
    if (p.vec) {
        p.grid_x = persistent_blocks(n, F2VB_TF, 4);
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

// The per-face stage of the vectorised forward pass on its own: wx[f, :] = (coeff[f] @ filter) * input[f]
// (r = 1, C % 4 == 0); used by pb200_facet2vertex_forward and by the fused facet2vertex + pointwise entry.
bool f2v_face_products_supported(int C, int K) { return vec_ok(C, 1) && kt_ok(K); }

int f2v_face_products(int64_t Nf, int C, int K, const float* input, const float* filter, const float* coeff, float* wx_,
                      cudaStream_t stream) {
    const int CV = C / 4;
    float4* wx = (float4*)wx_;
    if (Nf <= 0) return PB200_OK;
    if (CV % 32 == 0 && K <= 32) {
        const int KPb = (K + 3) / 4 * 4;
        const size_t smemb = sizeof(float4) * ((size_t)KPb * 32 + 2 * F2VF_TF * (KPb / 4));
        dim3 gridf(persistent_blocks(Nf, F2VF_TF, 4), (unsigned)(CV / 32));
        PB_LAUNCH("f2v_fwd_face", f2v_fwd_face_blocked_kernel, gridf, 256, smemb, stream, Nf, CV, K, coeff,
                  (const float4*)input, (const float4*)filter, wx);
    } else {
        const int KP = (K + 3) / 4 * 4 + 4;
        size_t smem = sizeof(float4) * 32 * (size_t)K + sizeof(float) * F2VF_TF * KP;
        dim3 gridf(persistent_blocks(Nf, F2VF_TF, 6), (unsigned)ceil_div(CV, 32));
        if (smem > 48 * 1024)
            PB_CUDA(cudaFuncSetAttribute(f2v_fwd_face_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        PB_LAUNCH("f2v_fwd_face", f2v_fwd_face_kernel, gridf, 256, smem, stream, Nf, CV, K, coeff,
                  (const float4*)input, (const float4*)filter, wx);
    }
    return PB200_OK;
}

}  // namespace pb

using namespace pb;

extern "C" {

size_t pb200_facet2vertex_forward_workspace_bytes(int64_t Nf, int C, int r, int K) {
    if (Nf < 0 || C <= 0 || r <= 0 || K <= 0) return 0;
    if (vec_ok(C, r) && kt_ok(K)) return align_up(sizeof(float) * (size_t)(Nf > 0 ? Nf : 1) * C, 256);
    return 0;
}

int pb200_facet2vertex_forward(int64_t Nf, int64_t NvOut, int C, int r, int K, const float* input,
                               const float* filter, const float* coeff, const int32_t* nfCount,
                               const int32_t* rowptr, const int32_t* entries, float* output,
                               void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NvOut >= 0 && C > 0 && r > 0 && K > 0, PB200_EINVAL, "facet2vertex_forward: bad sizes");
    if (NvOut == 0) return PB200_OK;
    PB_REQUIRE(output && rowptr && nfCount, PB200_EINVAL, "facet2vertex_forward: null pointer");
    PB_REQUIRE(Nf == 0 || (input && filter && coeff && entries), PB200_EINVAL, "facet2vertex_forward: null pointer");
    const bool vec = vec_ok(C, r) && kt_ok(K) && aligned16(input) && aligned16(filter) && aligned16(output) &&
                     workspace && aligned16(workspace) &&
                     workspace_bytes >= pb200_facet2vertex_forward_workspace_bytes(Nf, C, r, K);
    if (vec_ok(C, r) && kt_ok(K) && aligned16(input) && aligned16(filter) && aligned16(output))
        PB_REQUIRE(vec, PB200_EWORKSPACE, "facet2vertex_forward: workspace missing, misaligned or too small");
    if (vec) {
        int CV = C / 4;
        float4* wx = (float4*)workspace;
        int rc = f2v_face_products(Nf, C, K, input, filter, coeff, (float*)wx, stream);
        if (rc) return rc;
        TeamGeom g = team_geom(CV);
        dim3 grid(persistent_blocks(NvOut, g.teams, 8), g.chunks);
        PB_DISPATCH_TL(g.TL, PB_LAUNCH("f2v_fwd_gather", f2v_fwd_gather_kernel<TL>, grid, 256, 0, stream, NvOut, CV,
                                       rowptr, entries, nfCount, (const float4*)wx, (float4*)output));
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
        dim3 grid(p.grid_x, (unsigned)ceil_div(CV, 32));
        const int KP = (K + 3) / 4 * 4 + 4;
        size_t smem = sizeof(float4) * (32 * (size_t)K + F2VB_TF * 32) + sizeof(float) * F2VB_TF * KP;
        if (CV % 32 == 0 && K <= 32) {
            const int KPb = (K + 3) / 4 * 4;
            const size_t smemb = sizeof(float4) * ((size_t)KPb * 32 + F2VB_TF * 32 + 2 * F2VB_TF * (KPb / 4)) + 2 * 96 * 8;
            PB_LAUNCH("f2v_bwd", f2v_bwd_blocked_kernel, grid, 256, smemb, stream, Nf, CV, K, face, vtMap, nfCount, coeff,
                      (const float4*)input, (const float4*)filter, (const float4*)gradOutput, (float4*)gradInput,
                      (float4*)partial);
            return reduce_partials(partial, p.grid_x, (int64_t)K * Cr, gradFilter, stream);
        }
        const int cvc = CV < 32 ? CV : 32;
        const int nacc = (int)ceil_div((int64_t)K * cvc, 256);
#define PB_F2VB_LAUNCH(N)                                                                                        \
        PB_LAUNCH("f2v_bwd", f2v_bwd_tile_kernel<N>, grid, 256, smem, stream, Nf, CV, K, face, vtMap, nfCount,   \
                  coeff, (const float4*)input, (const float4*)filter, (const float4*)gradOutput,                \
                  (float4*)gradInput, (float4*)partial)
        if (smem > 48 * 1024) {
            PB_CUDA(cudaFuncSetAttribute(f2v_bwd_tile_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            PB_F2VB_LAUNCH(8);
        } else if (nacc <= 1) { PB_F2VB_LAUNCH(1); }
        else if (nacc <= 2) { PB_F2VB_LAUNCH(2); }
        else if (nacc <= 4) { PB_F2VB_LAUNCH(4); }
        else { PB_F2VB_LAUNCH(8); }
#undef PB_F2VB_LAUNCH
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

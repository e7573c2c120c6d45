// facet2facet filter gradient on tcgen05 + TMEM, one fused kernel:
//
//   gradFilter[co, ci, d] = sum_f g[f,co] * A[f,d,ci],   A[f,d,ci] = (1/T_f) sum_k bary[k,d]*in[k,ci]
//
// The reduction runs over FACES, so faces are the K dimension of the tensor-core product
// D[co, (d,kk)] += g^T[co, f] * A^T[(d,kk), f].  A CTA owns one group of 16 input channels
// (its F*16 <= 512 accumulator columns live in TMEM for the whole kernel) and one contiguous
// chunk of faces; per stage of 16 faces
//   * 8 producer warps build both operands in shared memory as K-major (face-contiguous)
//     64-byte swizzled rows: the transposed gradOutput block (128 rows) and the A^T block
//     (F*16 rows) -- thread = (face, 8 channels), a warp walks its share of the F bases;
//   * one thread issues tcgen05.mma (M = 128 output channels, N = F*16 in chunks of <= 256,
//     K = 8 faces per instruction) and commits the stage back.
// At the end the accumulator is drained once into partial[chunk] (final gradFilter layout);
// a second kernel adds the chunks in order, so the result is deterministic.
// Modes: 1 split (tf32 operands) or 2 splits (tf32 hi+lo, three MMAs per k-step).
#include "common.cuh"
#include "tc_ptx.cuh"

namespace pb {
namespace tc {

int* async_error_word();
int check_async_error(const char* where);

namespace gfilter {

using namespace ptx;

constexpr int UM = 128;                       // output channels (UMMA M), Cout zero-padded
constexpr int CG = 16;                        // input channels per CTA
constexpr int KF = 16;                        // faces per stage (64-byte K-major rows)
constexpr int PWARPS = 8;
constexpr int NTHREADS = (PWARPS + 1) * 32;   // + MMA warp
constexpr int G_TILE_BYTES = UM * 64;
constexpr int TREG = 4;

struct Params {
    int64_t Nf;
    int Cin, Cout, F;
    int ncg;                  // channel groups = Cin / 16
    int nchunks;              // face chunks
    int64_t stages_per_chunk; // 16-face stages per chunk
    int nstages;              // ring depth
    const float* gout;
    const float* in;
    const float* bary;
    const int32_t* cum;
    float* partial;           // [nchunks][Cout*Cin*F]
    int* async_err;
};

template <int NSPLIT>
__global__ void __launch_bounds__(NTHREADS, 1) f2f_bwd_gfilter_tc_kernel(Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.nstages, F = p.F, Cin = p.Cin, Cout = p.Cout;
    const int NR = F * CG;                                   // accumulator columns / A^T rows
    const size_t at_bytes = (size_t)NR * 64;
    const size_t stage_bytes = (size_t)NSPLIT * (G_TILE_BYTES + at_bytes);   // [g hi][g lo?][A^T hi][A^T lo?]
    uint8_t* stages = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)S * stage_bytes);
    uint64_t* full = bars;                // [S] 8 producer warps
    uint64_t* empty = bars + S;           // [S] MMA done with the stage
    uint64_t* acc_done = bars + 2 * S;    // all MMAs of the CTA complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], PWARPS); mbar_init(&empty[s], 1); }
        mbar_init(acc_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == PWARPS) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int cgp = blockIdx.x % p.ncg;                      // channel group of this CTA
    const int chunk = blockIdx.x / p.ncg;                    // face chunk
    const int64_t st0 = (int64_t)chunk * p.stages_per_chunk;
    const int64_t total_stages = (p.Nf + KF - 1) / KF;
    int64_t st1 = st0 + p.stages_per_chunk;
    if (st1 > total_stages) st1 = total_stages;
    const int64_t nst = st1 > st0 ? st1 - st0 : 0;

    if (warp < PWARPS) {
        // ==================================== producers ====================================
        const int fl = lane >> 1, half = lane & 1;            // face of the stage, 8-channel half
        const uint32_t fchunk = (uint32_t)(fl >> 2), fsub = (uint32_t)(fl & 3) * 4u;
        int si = 0;
        uint32_t sph = 0;
        bool alive = true;
        for (int64_t st = 0; st < nst && alive; ++st) {
            const int64_t f = (st0 + st) * KF + fl;
            const bool valid = f < p.Nf;
            int k0 = 0, k1 = 0;
            if (valid) { k0 = f > 0 ? __ldg(p.cum + f - 1) : 0; k1 = __ldg(p.cum + f); }
            const int T = k1 - k0;
            const float invT = T > 0 ? 1.f / (float)T : 0.f;
            // this thread's 8 input channels of up to TREG samples, pre-scaled by 1/T
            float x[TREG][8];
#pragma unroll
            for (int t = 0; t < TREG; ++t) {
                if (t < T) {
                    const float4* src = reinterpret_cast<const float4*>(p.in + (int64_t)(k0 + t) * Cin + cgp * CG + half * 8);
                    float4 u = ldg4(src), w = ldg4(src + 1);
                    x[t][0] = u.x * invT; x[t][1] = u.y * invT; x[t][2] = u.z * invT; x[t][3] = u.w * invT;
                    x[t][4] = w.x * invT; x[t][5] = w.y * invT; x[t][6] = w.z * invT; x[t][7] = w.w * invT;
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[t][j] = 0.f;
                }
            }
            // transposed gradOutput block: warp w copies output channels [16w, 16w+16)
            float4 gv[2];
            {
                const int co0 = warp * 16 + half * 8;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    int co = co0 + i * 4;
                    gv[i] = (valid && co < Cout) ? ldg4(reinterpret_cast<const float4*>(p.gout + f * Cout + co)) : zero4();
                }
            }
            // wait for the stage to be free
            if (!mbar_try_wait(&empty[si], sph ^ 1u)) {
                int ok = 1;
                if (lane == 0) ok = mbar_wait(&empty[si], sph ^ 1u, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
            }
            uint8_t* sbase = stages + (size_t)si * stage_bytes;
            uint8_t* g_hi = sbase;
            uint8_t* at_hi = sbase + (size_t)NSPLIT * G_TILE_BYTES;
            // element (row, face fl) of a K-major 64B-swizzled block
            auto elem = [&](uint8_t* base, int row) -> float* {
                return reinterpret_cast<float*>(base + (size_t)row * 64 + ((fchunk ^ (((uint32_t)row >> 1) & 3u)) << 4) + fsub);
            };
            auto put = [&](uint8_t* hi_base, size_t lo_off, int row, float v) {
                if (NSPLIT == 1) {
                    *elem(hi_base, row) = to_tf32_rna(v);
                } else {
                    float hv = tf32_hi(v);
                    *elem(hi_base, row) = hv;
                    *elem(hi_base + lo_off, row) = v - hv;
                }
            };
            {
                const int co0 = warp * 16 + half * 8;
                const float g8[8] = {gv[0].x, gv[0].y, gv[0].z, gv[0].w, gv[1].x, gv[1].y, gv[1].z, gv[1].w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // the two halves of a warp must hit rows of different parity (distinct banks):
                    // half 1 walks its 8 rows rotated by one
                    const int jr = (j + 1) & 7;
                    put(g_hi, G_TILE_BYTES, co0 + (half ? jr : j), half ? g8[jr] : g8[j]);
                }
            }
            for (int d = warp; d < F; d += PWARPS) {
                float a[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] = 0.f;
#pragma unroll
                for (int t = 0; t < TREG; ++t) {
                    if (t < T) {
                        const float b = __ldg(p.bary + (int64_t)(k0 + t) * F + d);
#pragma unroll
                        for (int j = 0; j < 8; ++j) a[j] = fmaf(b, x[t][j], a[j]);
                    }
                }
                for (int t = TREG; t < T; ++t) {               // faces with many samples
                    const float b = __ldg(p.bary + (int64_t)(k0 + t) * F + d) * invT;
                    const float4* src = reinterpret_cast<const float4*>(p.in + (int64_t)(k0 + t) * Cin + cgp * CG + half * 8);
                    float4 u = ldg4(src), w = ldg4(src + 1);
                    a[0] = fmaf(b, u.x, a[0]); a[1] = fmaf(b, u.y, a[1]); a[2] = fmaf(b, u.z, a[2]); a[3] = fmaf(b, u.w, a[3]);
                    a[4] = fmaf(b, w.x, a[4]); a[5] = fmaf(b, w.y, a[5]); a[6] = fmaf(b, w.z, a[6]); a[7] = fmaf(b, w.w, a[7]);
                }
                const int row0 = d * CG + half * 8;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int jr = (j + 1) & 7;
                    put(at_hi, at_bytes, row0 + (half ? jr : j), half ? a[jr] : a[j]);
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[si]);
            if (++si == S) { si = 0; sph ^= 1u; }
        }
        // ==================================== drain ====================================
        if (alive) {
            int ok = 1;
            if (lane == 0) ok = mbar_wait(acc_done, 0u, abort_flag) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok) {
                tc_fence_after();
                const int q = warp & 3, hcol = warp >> 2;       // TMEM lane quadrant, half of the 32-column groups
                const int co = q * 32 + lane;
                float* out = p.partial + (int64_t)chunk * Cout * Cin * F;
                const int ngroups = (NR + 31) / 32;
                for (int gi = hcol; gi < ngroups; gi += 2) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(gi * 32), r);
                    tmem_ld_wait();
                    if (co < Cout) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            int col = gi * 32 + j;
                            if (col < NR) {
                                int d = col / CG, kk = col - d * CG;
                                out[((int64_t)co * Cin + cgp * CG + kk) * F + d] = nst > 0 ? __uint_as_float(r[j]) : 0.f;
                            }
                        }
                    }
                }
                tc_fence_before();
            }
        }
    } else {
        // ==================================== MMA issuer ====================================
        if (lane == 0) {
            const int n1 = NR < 256 ? NR : 256, n2 = NR - n1;
            const uint32_t idesc1 = instr_desc(FMT_TF32, UM, (uint32_t)n1);
            const uint32_t idesc2 = instr_desc(FMT_TF32, UM, (uint32_t)(n2 > 0 ? n2 : 16));
            int si = 0;
            uint32_t sph = 0;
            bool alive = true;
            for (int64_t st = 0; st < nst; ++st) {
                if (!mbar_wait(&full[si], sph, abort_flag)) { alive = false; break; }
                tc_fence_after();
                const uint32_t sb = smem_u32(stages + (size_t)si * stage_bytes);
                const uint32_t g_hi = sb, at_hi = sb + NSPLIT * G_TILE_BYTES;
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) {
                    const uint64_t adv = (uint64_t)(k2 * 2);
                    const uint32_t first = (st != 0 || k2 != 0) ? 1u : 0u;
                    for (int c = 0; c < (n2 > 0 ? 2 : 1); ++c) {
                        const uint32_t d_tmem = tmem_base + (uint32_t)(c * 256);
                        const uint32_t idesc = c == 0 ? idesc1 : idesc2;
                        const uint32_t at_c = at_hi + (uint32_t)(c * 256 * 64);
                        const uint64_t dg_hi = smem_desc_kmajor(g_hi, 64, SWZ_64B) + adv;
                        const uint64_t da_hi = smem_desc_kmajor(at_c, 64, SWZ_64B) + adv;
                        if (NSPLIT == 1) {
                            mma_tf32(d_tmem, dg_hi, da_hi, idesc, first);
                        } else {
                            const uint64_t dg_lo = smem_desc_kmajor(g_hi + G_TILE_BYTES, 64, SWZ_64B) + adv;
                            const uint64_t da_lo = smem_desc_kmajor(at_c + (uint32_t)at_bytes, 64, SWZ_64B) + adv;
                            mma_tf32(d_tmem, dg_lo, da_hi, idesc, first);
                            mma_tf32(d_tmem, dg_hi, da_lo, idesc, 1u);
                            mma_tf32(d_tmem, dg_hi, da_hi, idesc, 1u);
                        }
                    }
                }
                tc_commit(&empty[si]);
                if (++si == S) { si = 0; sph ^= 1u; }
            }
            if (alive) tc_commit(acc_done);
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == PWARPS) tmem_dealloc(tmem_base, 512);
    if (tid == 0 && *abort_flag && p.async_err) {
        *p.async_err = 3;
        __threadfence_system();
    }
}

// ---------------------------------------------------------------------------- host side
struct Plan { int nsplit, ncg, nchunks, nstages; int64_t stages_per_chunk; size_t smem, partial_bytes; };

bool supported(int Cin, int Cout, int F) {
    return Cin % CG == 0 && Cout % 4 == 0 && Cout >= 4 && Cout <= UM && F >= 1 && F * CG <= 512;
}

Plan plan(int64_t Nf, int Cin, int Cout, int F, int precision) {
    Plan pl;
    pl.nsplit = precision == PB200_PREC_FP32 ? 2 : 1;
    pl.ncg = Cin / CG;
    int64_t total_stages = ceil_div(Nf > 0 ? Nf : 1, KF);
    int nch = sm_count() / pl.ncg;
    if (nch < 1) nch = 1;
    if (nch > total_stages) nch = (int)total_stages;
    pl.stages_per_chunk = ceil_div(total_stages, nch);
    pl.nchunks = (int)ceil_div(total_stages, pl.stages_per_chunk);
    size_t stage = (size_t)pl.nsplit * (G_TILE_BYTES + (size_t)F * CG * 64);
    int S = 4;
    while (S > 2 && (size_t)S * stage + 1024 + 256 > 224 * 1024) --S;
    pl.nstages = S;
    pl.smem = (size_t)S * stage + 1024 + 256;
    pl.partial_bytes = (size_t)pl.nchunks * Cout * Cin * F * sizeof(float);
    return pl;
}

bool fits(int64_t Nf, int Cin, int Cout, int F, int precision) {
    return plan(Nf, Cin, Cout, F, precision).smem <= 227 * 1024;
}

size_t workspace_bytes(int64_t Nf, int Cin, int Cout, int F, int precision) {
    return align_up(plan(Nf, Cin, Cout, F, precision).partial_bytes, 256);
}

int backward_filter(int64_t Nf, int Cin, int Cout, int F, const float* gout, const float* input, const float* bary,
                    const int32_t* cum, float* gfilter, int precision, void* ws, cudaStream_t stream) {
    int rc = check_async_error("facet2facet_backward");
    if (rc) return rc;
    Plan pl = plan(Nf, Cin, Cout, F, precision);
    Params p;
    p.Nf = Nf; p.Cin = Cin; p.Cout = Cout; p.F = F;
    p.ncg = pl.ncg; p.nchunks = pl.nchunks; p.stages_per_chunk = pl.stages_per_chunk; p.nstages = pl.nstages;
    p.gout = gout; p.in = input; p.bary = bary; p.cum = cum; p.partial = (float*)ws;
    p.async_err = async_error_word();
    int grid = pl.ncg * pl.nchunks;
    if (pl.nsplit == 2) {
        PB_CUDA(cudaFuncSetAttribute(f2f_bwd_gfilter_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
        PB_LAUNCH("f2f_bwd_gfilter_tc", f2f_bwd_gfilter_tc_kernel<2>, grid, NTHREADS, pl.smem, stream, p);
    } else {
        PB_CUDA(cudaFuncSetAttribute(f2f_bwd_gfilter_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
        PB_LAUNCH("f2f_bwd_gfilter_tc", f2f_bwd_gfilter_tc_kernel<1>, grid, NTHREADS, pl.smem, stream, p);
    }
    return reduce_partials((const float*)ws, pl.nchunks, (int64_t)Cout * Cin * F, gfilter, stream);
}

}  // namespace gfilter
}  // namespace tc
}  // namespace pb

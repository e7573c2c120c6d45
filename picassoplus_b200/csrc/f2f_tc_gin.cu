// facet2facet input gradient on tcgen05 + TMEM, one fused kernel:
//
//   gA[f, (ci,d)] = sum_co g[f,co] * W[co,ci,d]            (tensor cores, K = co)
//   gradInput[k, ci] = (1/T_f) sum_d bary[k,d] * gA[f(k), (ci,d)]   (epilogue, straight from TMEM)
//
// gA (F*Cin floats per face, 12.8 KB at 128 channels x 25 bases) never leaves the SM.
// Per CTA (persistent) and per tile of 128 faces (UMMA M = TMEM lanes = faces):
//   * two loader warps copy the tile's gradOutput rows into shared memory as the K-major M-side
//     operand (64-byte swizzled rows; bf16 hi+lo, bf16 or tf32), into one of two tile buffers, so
//     the copy of tile t+1 runs while tile t is multiplied and drained;
//   * one thread streams pre-swizzled filter blocks W'[(ci,d) rows][K block] (N-side operand,
//     N = up to 256 rows = NQ channels x F bases per slice) with 1-D bulk copies;
//   * one thread issues tcgen05.mma into one of two 256-column accumulators;
//   * 8 epilogue warps (thread = face) drain the other accumulator.  The two warps of a TMEM
//     quadrant split the samples of a face (samples 0,1 / 2,3), whose bary rows stay in
//     registers for the whole tile; for every channel pair a thread reads the F columns of both
//     channels (the next pair's columns are requested while the current sums run), contracts
//     them with its two bary rows in packed f32x2 FMAs and writes 16-byte pieces of gradInput.
// Modes: one operand (tf32 or bf16) or hi+lo operands (bf16 or tf32; three MMAs per k-step).
// All waits are bounded; on a time-out the block unwinds and raises the async error word.
#include "common.cuh"
#include "tc_ptx.cuh"
#include "tc_runtime.cuh"

namespace pb {
namespace tc {

namespace gin {

using namespace ptx;

constexpr int TILE_M = 128;
constexpr int NCOLS = 256;
constexpr int KS = 16;
constexpr int EWARPS = 8;
constexpr int GWARPS = 2;                        // gradOutput tile loaders
constexpr int NTHREADS = (EWARPS + 2 + GWARPS) * 32;
constexpr int G_KTILE_BYTES = TILE_M * 64;      // one 16-channel block of the gradOutput tile
constexpr int W_STAGE_BYTES = NCOLS * 64;       // one 16-channel block of a filter slice

// ---- TMEM loads of 1/4/8/16/32 consecutive columns (lane = row)
__device__ __forceinline__ void tmem_ld1(uint32_t taddr, float* v) {
    uint32_t r0;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r0) : "r"(taddr) : "memory");
    v[0] = __uint_as_float(r0);
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float* v) {
    uint32_t r[4];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                   "=r"(r[15])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld32f(uint32_t taddr, float* v) {
    uint32_t r[32];
    tmem_ld32(taddr, r);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// F consecutive columns -> v[0..F)
template <int F>
__device__ __forceinline__ void tmem_ld_row(uint32_t taddr, float* v) {
    int o = 0;
    if (F & 32) { tmem_ld32f(taddr + o, v + o); o += 32; }
    if (F & 16) { tmem_ld16(taddr + o, v + o); o += 16; }
    if (F & 8)  { tmem_ld8(taddr + o, v + o); o += 8; }
    if (F & 4)  { tmem_ld4(taddr + o, v + o); o += 4; }
    if (F & 2)  { tmem_ld1(taddr + o, v + o); tmem_ld1(taddr + o + 1, v + o + 1); o += 2; }
    if (F & 1)  { tmem_ld1(taddr + o, v + o); }
}

// ---- filter image: Wimg[slice][kst][split][row 0..255][16 floats, 64B-swizzled];
//      row = cil*F + d, element (row, kk) = filter[co = kst*16 + kk][ci = slice*NQ + cil][d]
//      (co counts from the chunk's first output channel co0)
//      The filter element (co, ci, d) is read at filter[co * s_co + ci * s_ci + d]: (Cin * F, F) for the operator's
//      (Cout, Cin, F) filter, (F, Cin_of_the_filter * F) when the two channel roles are exchanged.
__global__ void f2f_tc_gin_prep_filter_kernel(int F, int Cin, int co0, int Cout, int nq, int nslices, int kst, int nsplit,
                                              int64_t s_co, int64_t s_ci,
                                              const float* __restrict__ filter, uint8_t* __restrict__ wimg) {
    int64_t total = (int64_t)nslices * kst * NCOLS * 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(i & 3);
        int row = (int)((i >> 2) % NCOLS);
        int64_t blk = i / (4 * NCOLS);
        int ks = (int)(blk % kst);
        int slice = (int)(blk / kst);
        int cil = row / F, d = row - cil * F;
        int ci = slice * nq + cil;
        float hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int co = ks * KS + c * 4 + j;
            float v = (cil < nq && ci < Cin && co < Cout) ? __ldg(filter + (int64_t)(co0 + co) * s_co + (int64_t)ci * s_ci + d) : 0.f;
            if (nsplit == 1) { hi[j] = to_tf32_rna(v); lo[j] = 0.f; }
            else { hi[j] = tf32_hi(v); lo[j] = v - hi[j]; }
        }
        uint8_t* base = wimg + blk * (int64_t)nsplit * W_STAGE_BYTES;
        uint32_t off = swz64_offset((uint32_t)row, (uint32_t)c);
        *reinterpret_cast<float4*>(base + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        if (nsplit == 2)
            *reinterpret_cast<float4*>(base + W_STAGE_BYTES + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// ---- bf16 filter image: Wimg[slice][kst][split][row 0..255][32 bf16, 64B-swizzled];
//      row = cil*F + d, element (row, kk) = filter[co = kst*32 + kk][ci = slice*NQ + cil][d]
__global__ void f2f_tc_gin_prep_filter_bf16_kernel(int F, int Cin, int co0, int Cout, int nq, int nslices, int kst,
                                                   int nsplit, int64_t s_co, int64_t s_ci,
                                                   const float* __restrict__ filter, uint8_t* __restrict__ wimg) {
    int64_t total = (int64_t)nslices * kst * NCOLS * 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(i & 3);
        int row = (int)((i >> 2) % NCOLS);
        int64_t blk = i / (4 * NCOLS);
        int ks = (int)(blk % kst);
        int slice = (int)(blk / kst);
        int cil = row / F, d = row - cil * F;
        int ci = slice * nq + cil;
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                int co = ks * 32 + c * 8 + 2 * j + e;
                v[e] = (cil < nq && ci < Cin && co < Cout) ? __ldg(filter + (int64_t)(co0 + co) * s_co + (int64_t)ci * s_ci + d) : 0.f;
            }
            if (nsplit == 1) { hi[j] = pack_bf16x2(v[0], v[1]); lo[j] = 0u; }
            else split_bf16x2(v[0], v[1], hi[j], lo[j]);
        }
        uint8_t* base = wimg + blk * (int64_t)nsplit * W_STAGE_BYTES;
        uint32_t off = swz64_offset((uint32_t)row, (uint32_t)c);
        *reinterpret_cast<uint4*>(base + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        if (nsplit == 2) *reinterpret_cast<uint4*>(base + W_STAGE_BYTES + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// running sample count after face f; a null array stands for one sample per face
__device__ __forceinline__ int cum_at(const int32_t* cum, int64_t f) { return cum ? __ldg(cum + f) : (int)(f + 1); }

struct Params {
    int64_t Nf;
    int Cin, Cout;
    int nq, nslices, kst, nmma;      // channels per slice, slices, 16-channel K blocks, UMMA N
    int nstages;                     // filter ring depth
    int gbufs;                       // gradOutput tile buffers (2 = the copy runs a tile ahead)
    int bary_rows, bpitch;           // staged bary rows per tile (0 = read from global), row pitch in floats
    const float* gout;               // first output channel of this launch's chunk
    int g_stride;                    // floats per gradOutput row (all output channels of the operator)
    int accumulate;                  // 0: gradInput = result; 1: gradInput += result (later output-channel chunks)
    const float* bary;
    const float* bary_p;             // bary with rows padded to Fp floats (pad columns zero)
    int Fp;
    const int32_t* cum;
    const uint8_t* wimg;
    float* gin;
    int* async_err;
    int wait_budget;                 // bounded waits give up after this many units of 1024 clocks
};

// BF: operands as bf16 (a 64-byte operand row holds 32 output channels, MMAs of kind::f16 at
// twice the tf32 rate) instead of tf32 (16 output channels per row)
template <int NSPLIT, int F, bool BF>
__global__ void __launch_bounds__(NTHREADS, 1) f2f_bwd_gin_tc_kernel(Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.nstages, KST = p.kst;
    const int Cin = p.Cin, Cout = p.Cout;
    const size_t gtile_bytes = (size_t)NSPLIT * KST * G_KTILE_BYTES;       // [split][kst][8 KB]
    const size_t wstage_bytes = (size_t)NSPLIT * W_STAGE_BYTES;           // [split][16 KB]
    uint8_t* gtile = smem;
    uint8_t* wst = smem + (size_t)p.gbufs * gtile_bytes;        // one or two gradOutput tile buffers
    float* bary_s = reinterpret_cast<float*>(wst + (size_t)S * wstage_bytes);
    uint8_t* tail = reinterpret_cast<uint8_t*>(bary_s + (size_t)p.bary_rows * p.bpitch);
    uint64_t* bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(tail) + 15) & ~(uintptr_t)15);
    uint64_t* w_full = bars;                  // [S]
    uint64_t* w_empty = bars + S;             // [S]
    uint64_t* acc_full = bars + 2 * S;        // [2]
    uint64_t* acc_empty = bars + 2 * S + 2;   // [2]
    uint64_t* g_full = bars + 2 * S + 4;      // [2] gradOutput tile buffer written
    uint64_t* g_empty = bars + 2 * S + 6;     // [2] all MMAs of the tile done reading the buffer
    uint64_t* b_ready = bars + 2 * S + 8;     // bary rows of the tile staged
    uint64_t* b_free = bars + 2 * S + 9;      // all warps done with the staged rows
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 10);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&w_full[s], 1); mbar_init(&w_empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], EWARPS); }
        for (int b = 0; b < 2; ++b) { mbar_init(&g_full[b], GWARPS); mbar_init(&g_empty[b], 1); }
        mbar_init(b_ready, EWARPS);
        mbar_init(b_free, EWARPS);
        abort_flag[0] = 0;
        abort_flag[1] = p.wait_budget;
        fence_barrier_init();
    }
    if (warp == EWARPS) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int64_t ntiles = (p.Nf + TILE_M - 1) / TILE_M;

    if (warp < EWARPS) {
        // ===================== gradOutput tile loader + epilogue (thread = face) =====================
        const int q = warp & 3, half = warp >> 2;
        const int r = q * 32 + lane;                            // face row of the tile = TMEM lane
        const int npairs = (p.nq + 1) >> 1;
        const int pair_lo = half == 0 ? 0 : (npairs + 1) >> 1;
        const int pair_hi = half == 0 ? (npairs + 1) >> 1 : npairs;
        uint32_t tcount = 0, sc = 0;
        bool alive = true;
        auto warp_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
            int ok = 1;
            if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
            return __shfl_sync(0xffffffffu, ok, 0) != 0;
        };
        // sample range of the thread's face, fetched one tile ahead
        int k0n = 0, k1n = 0;
        {
            const int64_t f = (int64_t)blockIdx.x * TILE_M + r;
            if (f < p.Nf) { k0n = f > 0 ? cum_at(p.cum, f - 1) : 0; k1n = cum_at(p.cum, f); }
        }
        for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++tcount) {
            const int64_t f0 = tile * TILE_M;
            const int64_t f = f0 + r;
            const bool valid = f < p.Nf;
            const int k0 = k0n, k1 = k1n;
            {
                const int64_t fn = f + (int64_t)gridDim.x * TILE_M;
                k0n = 0; k1n = 0;
                if (fn < p.Nf) { k0n = cum_at(p.cum, fn - 1); k1n = cum_at(p.cum, fn); }
            }
            const int T = k1 - k0;
            const float invT = T > 0 ? 1.f / (float)T : 0.f;
            // ---- 2. stage the bary rows of the tile's samples (as many as fit)
            int kt0 = 0, kt1 = 0;
            {
                int64_t fl = f0 + TILE_M < p.Nf ? f0 + TILE_M : p.Nf;
                kt0 = f0 > 0 ? cum_at(p.cum, f0 - 1) : 0;
                kt1 = cum_at(p.cum, fl - 1);
            }
            int nrows = kt1 - kt0;
            if (nrows > p.bary_rows) nrows = p.bary_rows;
            if (p.bary_rows > 0) {
                if (!warp_wait(b_free, (tcount & 1u) ^ 1u)) { alive = false; break; }
                const float* src = p.bary + (int64_t)kt0 * F;
                for (int i = tid; i < nrows * F; i += EWARPS * 32) {
                    int sr = i / F;
                    bary_s[sr * p.bpitch + (i - sr * F)] = __ldg(src + i);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(b_ready);
                if (!warp_wait(b_ready, tcount & 1u)) { alive = false; break; }
            }
            const int kloc = k0 - kt0;
            const bool staged = valid && (kloc + T <= nrows);
            // bary rows of the face's first four samples, packed (even d, odd d), zero beyond T / F
            constexpr int FH = (F + 1) / 2;
            const bool lean = !__any_sync(0xffffffffu, valid && T > 4);
            // lean path: the two warps of a TMEM quadrant share the samples of a face: warp `half` takes
            // samples 2*half and 2*half + 1 for every channel of the slice
            const int ts = 2 * half;
            float2 breg[2][FH];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                // 16-byte loads from the padded rows (pad columns are zero)
                const bool on = lean && ts + t < T;
                const float4* src = reinterpret_cast<const float4*>(p.bary_p + (int64_t)(k0 + (on ? ts + t : 0)) * p.Fp);
#pragma unroll
                for (int q4 = 0; q4 < (F + 3) / 4; ++q4) {
                    const float4 v = on ? ldg4(src + q4) : zero4();
                    breg[t][2 * q4] = make_float2(v.x, v.y);
                    if (2 * q4 + 1 < FH) breg[t][2 * q4 + 1] = make_float2(v.z, v.w);
                }
            }
            float* const row0 = p.gin + (int64_t)(k0 + ts) * Cin;     // gradInput rows of the thread's two samples
            const bool on0 = ts < T, on1 = ts + 1 < T;
            // 16-byte stores: rows and channel quadruples aligned, every slice made of whole pairs
            const bool vec4 = (Cin % 4 == 0) && (p.nq % 2 == 0) && ((reinterpret_cast<uintptr_t>(p.gin) & 15) == 0);
            float2 h0 = make_float2(0.f, 0.f), h1 = h0;
            // ---- 3. per slice: drain the accumulator, contract with bary, store gradInput
            for (int slice = 0; slice < p.nslices && alive; ++slice, ++sc) {
                const uint32_t a = sc & 1u;
                if (!warp_wait(&acc_full[a], (sc >> 1) & 1u)) { alive = false; break; }
                tc_fence_after();
                const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + a * NCOLS;
                // The bary rows of the thread's two samples were loaded into registers once per tile
                // (packed as (even d, odd d) pairs).  The sum over the F bases runs with fma.f32x2 on
                // those pairs, two samples and two channels at a time, no shared-memory traffic at all.
                if (lean) {
                    const int ci0 = slice * p.nq;
                    // accumulator columns of the first channel pair; later pairs are requested as soon as
                    // the registers of the previous one are free, so the loads overlap the sums and stores
                    float2 va[FH], vb[FH];
#pragma unroll
                    for (int d = 0; d < FH; ++d) { va[d] = make_float2(0.f, 0.f); vb[d] = make_float2(0.f, 0.f); }
                    tmem_ld_row<F>(tbase, reinterpret_cast<float*>(va));
                    if (1 < p.nq) tmem_ld_row<F>(tbase + (uint32_t)F, reinterpret_cast<float*>(vb));
                    for (int cil = 0; cil < p.nq; cil += 2) {
                        const int ci = ci0 + cil;
                        const bool has_b = (cil + 1 < p.nq) && (ci + 1 < Cin);
                        const int nx = cil + 2;
                        tmem_ld_wait();
                        if (F & 1) { va[FH - 1].y = 0.f; vb[FH - 1].y = 0.f; }
                        // two partial sums per sample and channel: four independent chains per block
                        float2 sa[2], sb[2], sa2[2], sb2[2];
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            sa[t] = make_float2(0.f, 0.f); sb[t] = make_float2(0.f, 0.f);
                            sa2[t] = make_float2(0.f, 0.f); sb2[t] = make_float2(0.f, 0.f);
                        }
#pragma unroll
                        for (int d = 0; d < FH; ++d) {
#pragma unroll
                            for (int t = 0; t < 2; ++t) {
                                if (d & 1) sa2[t] = __ffma2_rn(breg[t][d], va[d], sa2[t]);
                                else sa[t] = __ffma2_rn(breg[t][d], va[d], sa[t]);
                            }
                        }
                        if (nx < p.nq) tmem_ld_row<F>(tbase + (uint32_t)(nx * F), reinterpret_cast<float*>(va));
#pragma unroll
                        for (int d = 0; d < FH; ++d) {
#pragma unroll
                            for (int t = 0; t < 2; ++t) {
                                if (d & 1) sb2[t] = __ffma2_rn(breg[t][d], vb[d], sb2[t]);
                                else sb[t] = __ffma2_rn(breg[t][d], vb[d], sb[t]);
                            }
                        }
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            sa[t].x += sa2[t].x; sa[t].y += sa2[t].y;
                            sb[t].x += sb2[t].x; sb[t].y += sb2[t].y;
                        }
                        if (nx + 1 < p.nq) tmem_ld_row<F>(tbase + (uint32_t)((nx + 1) * F), reinterpret_cast<float*>(vb));
                        else {
#pragma unroll
                            for (int d = 0; d < FH; ++d) vb[d] = make_float2(0.f, 0.f);
                        }
                        if (ci < Cin) {
                            const float2 g0 = make_float2((sa[0].x + sa[0].y) * invT, (sb[0].x + sb[0].y) * invT);
                            const float2 g1 = make_float2((sa[1].x + sa[1].y) * invT, (sb[1].x + sb[1].y) * invT);
                            float* d0 = row0 + ci;
                            float* d1 = d0 + Cin;
                            if (vec4) {
                                // channels ci..ci+1 wait for ci+2..ci+3: one 16-byte store per sample and
                                // four channels (a scattered store costs the same pass whatever its width)
                                if ((ci & 2) == 0) { h0 = g0; h1 = g1; }
                                else {
                                    float4 v0 = make_float4(h0.x, h0.y, g0.x, g0.y), v1 = make_float4(h1.x, h1.y, g1.x, g1.y);
                                    if (p.accumulate) {
                                        if (on0) add4(v0, *reinterpret_cast<const float4*>(d0 - 2));
                                        if (on1) add4(v1, *reinterpret_cast<const float4*>(d1 - 2));
                                    }
                                    if (on0) *reinterpret_cast<float4*>(d0 - 2) = v0;
                                    if (on1) *reinterpret_cast<float4*>(d1 - 2) = v1;
                                }
                            } else {
                                const float a0 = p.accumulate && on0 ? d0[0] : 0.f, a1 = p.accumulate && on1 ? d1[0] : 0.f;
                                const float b0 = p.accumulate && on0 && has_b ? d0[1] : 0.f;
                                const float b1 = p.accumulate && on1 && has_b ? d1[1] : 0.f;
                                if (on0) { d0[0] = g0.x + a0; if (has_b) d0[1] = g0.y + b0; }
                                if (on1) { d1[0] = g1.x + a1; if (has_b) d1[1] = g1.y + b1; }
                            }
                        }
                    }
                } else {
                for (int pr = pair_lo; pr < pair_hi; ++pr) {
                    const int cil = 2 * pr;
                    const int ci = slice * p.nq + cil;
                    const bool has_b = (cil + 1 < p.nq) && (ci + 1 < Cin);
                    float va[F], vb[F];
                    tmem_ld_row<F>(tbase + (uint32_t)(cil * F), va);
                    if (cil + 1 < p.nq) tmem_ld_row<F>(tbase + (uint32_t)((cil + 1) * F), vb);
                    else {
#pragma unroll
                        for (int d = 0; d < F; ++d) vb[d] = 0.f;
                    }
                    tmem_ld_wait();
                    if (ci < Cin) {
                        for (int t = 0; t < T; ++t) {
                            float ga = 0.f, gb = 0.f;
                            if (staged) {
                                const float* bp = bary_s + (kloc + t) * p.bpitch;
#pragma unroll
                                for (int d4 = 0; d4 + 4 <= F; d4 += 4) {
                                    float4 b = *reinterpret_cast<const float4*>(bp + d4);
                                    ga = fmaf(b.x, va[d4], ga); gb = fmaf(b.x, vb[d4], gb);
                                    ga = fmaf(b.y, va[d4 + 1], ga); gb = fmaf(b.y, vb[d4 + 1], gb);
                                    ga = fmaf(b.z, va[d4 + 2], ga); gb = fmaf(b.z, vb[d4 + 2], gb);
                                    ga = fmaf(b.w, va[d4 + 3], ga); gb = fmaf(b.w, vb[d4 + 3], gb);
                                }
#pragma unroll
                                for (int d = F & ~3; d < F; ++d) {
                                    float b = bp[d];
                                    ga = fmaf(b, va[d], ga); gb = fmaf(b, vb[d], gb);
                                }
                            } else {
                                const float* bp = p.bary + (int64_t)(k0 + t) * F;
#pragma unroll
                                for (int d = 0; d < F; ++d) {
                                    float b = __ldg(bp + d);
                                    ga = fmaf(b, va[d], ga); gb = fmaf(b, vb[d], gb);
                                }
                            }
                            const int64_t idx = (int64_t)(k0 + t) * Cin + ci;
                            float* dst = p.gin + idx;
                            const float olda = p.accumulate ? dst[0] : 0.f, oldb = (p.accumulate && has_b) ? dst[1] : 0.f;
                            dst[0] = ga * invT + olda;
                            if (has_b) dst[1] = gb * invT + oldb;
                        }
                    }
                }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[a]);
            }
            if (!alive) break;
            if (p.bary_rows > 0) { __syncwarp(); if (lane == 0) mbar_arrive(b_free); }
        }
    } else if (warp >= EWARPS + 2) {
        // ===================== gradOutput tile loaders =====================
        // The tile's rows become the K-major M-side operand (64-byte swizzled rows).  A task is one
        // 16-byte operand chunk of one row (8 channels as bf16, 4 as tf32); consecutive lanes take
        // consecutive chunks of a row, so a warp reads whole rows.  The copy of tile t+1 starts as
        // soon as the last MMAs of tile t have read the operand, while the epilogue warps still
        // drain the last accumulators of tile t.
        const int gt = tid - (EWARPS + 2) * 32;                 // 0 .. GWARPS*32-1
        const int cpr = KST * 4;                                // chunks per row
        const int ntasks = TILE_M * cpr;
        constexpr int U = BF ? 6 : 12;                          // tasks in flight per thread
        uint32_t tcount = 0;
        bool alive = true;
        for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++tcount) {
            const int64_t f0 = tile * TILE_M;
            // with two buffers the copy runs a whole tile ahead of the MMAs
            const uint32_t gb = p.gbufs == 2 ? (tcount & 1u) : 0u;
            const uint32_t gph = p.gbufs == 2 ? ((tcount >> 1) & 1u) : (tcount & 1u);
            uint8_t* const gdst = gtile + (size_t)gb * gtile_bytes;
            {
                int ok = 1;
                if (lane == 0) ok = mbar_wait(&g_empty[gb], gph ^ 1u, abort_flag) ? 1 : 0;
                if (!__shfl_sync(0xffffffffu, ok, 0)) { alive = false; break; }
            }
            for (int base = 0; base < ntasks; base += U * GWARPS * 32) {
                float4 u[U], w[U];
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const int idx = base + j * GWARPS * 32 + gt;
                    const int rr = idx / cpr, c = idx - rr * cpr;
                    const int64_t fr = f0 + rr;
                    const float4* src = reinterpret_cast<const float4*>(p.gout + fr * p.g_stride);
                    u[j] = zero4(); w[j] = zero4();
                    if (BF) {
                        if (idx < ntasks && fr < p.Nf && c * 8 < Cout) u[j] = ldg4(src + 2 * c);
                        if (idx < ntasks && fr < p.Nf && c * 8 + 4 < Cout) w[j] = ldg4(src + 2 * c + 1);
                    } else {
                        if (idx < ntasks && fr < p.Nf && c * 4 < Cout) u[j] = ldg4(src + c);
                    }
                }
#pragma unroll
                for (int j = 0; j < U; ++j) {
                    const int idx = base + j * GWARPS * 32 + gt;
                    if (idx >= ntasks) continue;
                    const int rr = idx / cpr, c = idx - rr * cpr;
                    uint8_t* dst = gdst + (size_t)(c >> 2) * G_KTILE_BYTES + swz64_offset((uint32_t)rr, (uint32_t)(c & 3));
                    if (BF) {
                        uint32_t hi[4], lo[4];
                        if (NSPLIT == 1) {
                            hi[0] = pack_bf16x2(u[j].x, u[j].y); hi[1] = pack_bf16x2(u[j].z, u[j].w);
                            hi[2] = pack_bf16x2(w[j].x, w[j].y); hi[3] = pack_bf16x2(w[j].z, w[j].w);
                        } else {
                            split_bf16x2(u[j].x, u[j].y, hi[0], lo[0]); split_bf16x2(u[j].z, u[j].w, hi[1], lo[1]);
                            split_bf16x2(w[j].x, w[j].y, hi[2], lo[2]); split_bf16x2(w[j].z, w[j].w, hi[3], lo[3]);
                            *reinterpret_cast<uint4*>(dst + (size_t)KST * G_KTILE_BYTES) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        }
                        *reinterpret_cast<uint4*>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    } else if (NSPLIT == 1) {
                        *reinterpret_cast<float4*>(dst) =
                            make_float4(to_tf32_rna(u[j].x), to_tf32_rna(u[j].y), to_tf32_rna(u[j].z), to_tf32_rna(u[j].w));
                    } else {
                        const float4 hv = make_float4(tf32_hi(u[j].x), tf32_hi(u[j].y), tf32_hi(u[j].z), tf32_hi(u[j].w));
                        *reinterpret_cast<float4*>(dst) = hv;
                        *reinterpret_cast<float4*>(dst + (size_t)KST * G_KTILE_BYTES) =
                            make_float4(u[j].x - hv.x, u[j].y - hv.y, u[j].z - hv.z, u[j].w - hv.w);
                    }
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&g_full[gb]);
        }
    } else if (warp == EWARPS) {
        // ===================== filter loader (TMA engine) =====================
        if (lane == 0) {
            const uint32_t bytes = (uint32_t)wstage_bytes;
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
                for (int blk = 0; blk < p.nslices * KST; ++blk) {
                    if (!mbar_wait(&w_empty[s], ph ^ 1u, abort_flag)) { alive = false; break; }
                    mbar_arrive_expect_tx(&w_full[s], bytes);
                    bulk_g2s(wst + (size_t)s * wstage_bytes, p.wimg + (size_t)blk * bytes, bytes, &w_full[s]);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
            if (!alive) {
                long long t0 = clock64();
                while (clock64() - t0 < 2000000) { }
            }
        }
    } else {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            const uint32_t idesc = instr_desc(BF ? FMT_BF16 : FMT_TF32, TILE_M, (uint32_t)p.nmma);
            const uint64_t dg_base = smem_desc_kmajor(smem_u32(gtile), 64, SWZ_64B);
            const uint64_t dw_base = smem_desc_kmajor(smem_u32(wst), 64, SWZ_64B);
            int s = 0;
            uint32_t ph = 0, tcount = 0, sc = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++tcount) {
                const uint32_t gb = p.gbufs == 2 ? (tcount & 1u) : 0u;
                const uint32_t gph = p.gbufs == 2 ? ((tcount >> 1) & 1u) : (tcount & 1u);
                const uint64_t dg_tile = dg_base + (uint64_t)((gb * (uint32_t)gtile_bytes) >> 4);
                if (!mbar_wait(&g_full[gb], gph, abort_flag)) { alive = false; break; }
                for (int slice = 0; slice < p.nslices && alive; ++slice, ++sc) {
                    const uint32_t a = sc & 1u;
                    if (!mbar_wait(&acc_empty[a], ((sc >> 1) & 1u) ^ 1u, abort_flag)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + a * NCOLS;
                    for (int ks = 0; ks < KST; ++ks) {
                        if (!mbar_wait(&w_full[s], ph, abort_flag)) { alive = false; break; }
                        tc_fence_after();
                        // descriptors differ only in the 16-byte-unit start address: add offsets to a base
                        const uint64_t dg_hi = dg_tile + (uint64_t)(((uint32_t)ks * G_KTILE_BYTES) >> 4);
                        const uint64_t dw_hi = dw_base + (uint64_t)(((uint32_t)s * (uint32_t)wstage_bytes) >> 4);
#pragma unroll
                        for (int k2 = 0; k2 < 2; ++k2) {
                            const uint64_t adv = (uint64_t)(k2 * 2);
                            const uint32_t first = (ks | k2) != 0;
                            auto mma = [&](uint64_t a_, uint64_t b_, uint32_t acc) {
                                if (BF) mma_f16(d_tmem, a_, b_, idesc, acc); else mma_tf32(d_tmem, a_, b_, idesc, acc);
                            };
                            if (NSPLIT == 1) {
                                mma(dg_hi + adv, dw_hi + adv, first);
                            } else {
                                const uint64_t dg_lo = dg_hi + (uint64_t)(((uint32_t)KST * G_KTILE_BYTES) >> 4);
                                const uint64_t dw_lo = dw_hi + (uint64_t)(W_STAGE_BYTES >> 4);
                                mma(dg_lo + adv, dw_hi + adv, first);
                                mma(dg_hi + adv, dw_lo + adv, 1u);
                                mma(dg_hi + adv, dw_hi + adv, 1u);
                            }
                        }
                        tc_commit(&w_empty[s]);
                        if (++s == S) { s = 0; ph ^= 1u; }
                    }
                    if (alive) tc_commit(&acc_full[a]);
                }
                if (alive) tc_commit(&g_empty[gb]);
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == EWARPS) tmem_dealloc(tmem_base, 512);
    if (tid == 0 && *abort_flag && p.async_err) {
        *p.async_err = 2;
        __threadfence_system();
    }
}

// ---------------------------------------------------------------------------- host side
struct Plan { int nsplit, bf, nq, nslices, kst, nmma, nstages, gbufs, bary_rows, bpitch; size_t smem, wimg_bytes; };

static bool f_templated(int F) { return F == 4 || F == 9 || F == 16 || F == 25 || F == 36; }

// output channels beyond 256 are walked in chunks of 256; chunks after the first add to gradInput
constexpr int MAX_COUT = 256;
bool supported(int Cin, int Cout, int F) {
    return f_templated(F) && Cout % 4 == 0 && Cout >= 4 && Cin >= 1;
}

Plan plan(int Cin, int CoutAll, int F, int precision) {
    Plan pl;
    const int Cout = CoutAll < MAX_COUT ? CoutAll : MAX_COUT;          // the widest chunk sizes the buffers
    const OperandMode om = operand_mode(precision);
    pl.nsplit = om.nsplit;
    pl.bf = om.bf;
    pl.nq = NCOLS / F;
    if (pl.nq > Cin) pl.nq = Cin;
    pl.nslices = (Cin + pl.nq - 1) / pl.nq;
    pl.kst = pl.bf ? (Cout + 31) / 32 : (Cout + KS - 1) / KS;    // K blocks of one 64-byte operand row
    pl.nmma = (pl.nq * F + 15) / 16 * 16;
    pl.bpitch = ((F + 3) / 4 * 4) | 4;
    const size_t budget = 226 * 1024;
    size_t gt = (size_t)pl.nsplit * pl.kst * G_KTILE_BYTES;
    size_t ws = (size_t)pl.nsplit * W_STAGE_BYTES;
    // a second tile buffer takes the gradOutput copy off the critical path of every tile; it is
    // used when at least three filter stages still fit beside it
    pl.gbufs = (2 * gt + 1024 + 256 + 3 * ws <= budget) ? 2 : 1;
    size_t fixed = pl.gbufs * gt + 1024 + 256;
    int stages = 6;
    while (stages > 2 && fixed + stages * ws > budget) --stages;
    pl.nstages = stages;
    // bary rows live in registers (faces with up to four samples) or are read from global
    // memory (faces with more): nothing is staged in shared memory
    int rows = 0;
    pl.bary_rows = rows;
    pl.smem = fixed + stages * ws + (size_t)rows * pl.bpitch * 4;
    pl.wimg_bytes = (size_t)pl.nslices * pl.kst * ws;
    return pl;
}

bool fits(int Cin, int Cout, int F, int precision) {
    Plan pl = plan(Cin, Cout, F, precision);
    return pl.smem <= 227 * 1024 && pl.nstages >= 2;
}

size_t workspace_bytes(int Cin, int Cout, int F, int precision) {
    return align_up(plan(Cin, Cout, F, precision).wimg_bytes, 256);
}

template <int NSPLIT, int F, bool BF>
static int launch(const char* label, const Params& p, int grid, size_t smem, cudaStream_t stream) {
    PB_CUDA(cudaFuncSetAttribute(f2f_bwd_gin_tc_kernel<NSPLIT, F, BF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    PB_LAUNCH(label, (f2f_bwd_gin_tc_kernel<NSPLIT, F, BF>), grid, NTHREADS, smem, stream, p);
    return PB200_OK;
}

template <int NSPLIT, bool BF>
static int launch_f(const char* label, int F, const Params& p, int grid, size_t smem, cudaStream_t stream) {
    switch (F) {
        case 4: return launch<NSPLIT, 4, BF>(label, p, grid, smem, stream);
        case 9: return launch<NSPLIT, 9, BF>(label, p, grid, smem, stream);
        case 16: return launch<NSPLIT, 16, BF>(label, p, grid, smem, stream);
        case 25: return launch<NSPLIT, 25, BF>(label, p, grid, smem, stream);
        default: return launch<NSPLIT, 36, BF>(label, p, grid, smem, stream);
    }
}

// transposed = false: the operator's input gradient (filter (Cout, Cin, F)).
// transposed = true: the same contraction with the channel roles exchanged, for the forward pass of faces that have
// one sample each (cum null): "gout" is the operator's input (Nf, Cout_here), "Cin" counts the operator's output
// channels, the filter is the operator's (Cin_here, Cout_here, F) array, and gin receives the output.
int backward_input(int64_t Nf, int Cin, int Cout, int F, const float* gout, const float* filter, const float* bary,
                   const float* bary_p, int Fp, const int32_t* cum, float* gin, int precision, void* ws,
                   cudaStream_t stream, bool transposed) {
    const char* label = transposed ? "f2f_fwd_one_sample_tc" : "f2f_bwd_gin_tc";
    const int64_t s_co = transposed ? (int64_t)F : (int64_t)Cin * F, s_ci = transposed ? (int64_t)Cout * F : (int64_t)F;
    int rc = check_async_error(transposed ? "facet2facet_forward" : "facet2facet_backward");
    if (rc) return rc;
    Plan pl = plan(Cin, Cout, F, precision);
    uint8_t* wimg = (uint8_t*)ws;
    const int64_t ntiles = ceil_div(Nf, TILE_M);
    const int grid = (int)(ntiles < sm_count() ? ntiles : sm_count());
    for (int co0 = 0; co0 < Cout; co0 += MAX_COUT) {
        const int cchunk = Cout - co0 < MAX_COUT ? Cout - co0 : MAX_COUT;
        const int kst = pl.bf ? (cchunk + 31) / 32 : (cchunk + KS - 1) / KS;
        const int64_t items = (int64_t)pl.nslices * kst * NCOLS * 4;
        if (pl.bf) {
            PB_LAUNCH("f2f_tc_gin_prep_filter", f2f_tc_gin_prep_filter_bf16_kernel, persistent_blocks(items, 256, 8), 256, 0,
                      stream, F, Cin, co0, cchunk, pl.nq, pl.nslices, kst, pl.nsplit, s_co, s_ci, filter, wimg);
        } else {
            PB_LAUNCH("f2f_tc_gin_prep_filter", f2f_tc_gin_prep_filter_kernel, persistent_blocks(items, 256, 8), 256, 0,
                      stream, F, Cin, co0, cchunk, pl.nq, pl.nslices, kst, pl.nsplit, s_co, s_ci, filter, wimg);
        }
        Params p;
        p.Nf = Nf; p.Cin = Cin; p.Cout = cchunk;
        p.nq = pl.nq; p.nslices = pl.nslices; p.kst = kst; p.nmma = pl.nmma;
        p.nstages = pl.nstages; p.gbufs = pl.gbufs; p.bary_rows = pl.bary_rows; p.bpitch = pl.bpitch;
        p.gout = gout + co0; p.g_stride = Cout; p.accumulate = co0 > 0 ? 1 : 0;
        p.bary = bary; p.bary_p = bary_p; p.Fp = Fp; p.cum = cum; p.wimg = wimg; p.gin = gin;
        p.async_err = async_error_word();
        p.wait_budget = wait_budget_kclocks();
        if (pl.bf) rc = pl.nsplit == 2 ? launch_f<2, true>(label, F, p, grid, pl.smem, stream) : launch_f<1, true>(label, F, p, grid, pl.smem, stream);
        else rc = pl.nsplit == 2 ? launch_f<2, false>(label, F, p, grid, pl.smem, stream) : launch_f<1, false>(label, F, p, grid, pl.smem, stream);
        if (rc) return rc;
    }
    return PB200_OK;
}

}  // namespace gin
}  // namespace tc
}  // namespace pb

// facet2facet filter gradient on tcgen05 + TMEM, one fused kernel:
//
//   gradFilter[co, ci, d] = sum_f g[f,co] * A[f,d,ci],   A[f,d,ci] = (1/T_f) sum_k bary[k,d]*in[k,ci]
//
// The reduction runs over FACES, so faces are the K dimension of the tensor-core product
// D[co, (d,kk)] += g^T[co, f] * A^T[(d,kk), f].  A CTA owns one group of 16 input channels
// (its F*16 <= 512 accumulator columns live in TMEM for the whole kernel) and one contiguous
// chunk of faces; per stage of 16 faces
//   * 8 producer warps first copy the stage's raw rows (gradOutput rows, bary rows, the
//     CTA's 16 input channels of every sample, sample ranges) from global memory with
//     coalesced loads into a double-buffered raw area (two stages ahead of the math), then
//     build both operands in shared memory MN-major (128-byte swizzle, 32-byte base): a face
//     is a K-row whose 128-byte pieces hold 32 consecutive output channels (gradOutput block)
//     or 32 consecutive (basis, channel) columns (A block), so that neither operand is
//     transposed and every thread stores 16-byte vectors -- thread = (face, 8 channels), a
//     warp walks its share of the F bases;
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
constexpr int KF = 16;                        // faces per stage (four groups of 4 K-rows, two per instruction)
constexpr int PWARPS = 8;
constexpr int NTHREADS = (PWARPS + 1) * 32;   // + MMA warp
constexpr int ATOM_BYTES = 512;               // 4 K-rows x 128 bytes (32 M/N elements)
constexpr int G_SBO = (UM / 32) * ATOM_BYTES; // gradOutput block: [4-face group][32-channel block][atom]
constexpr int G_TILE_BYTES = (KF / 4) * G_SBO;
constexpr int TREG = 4;
// raw staging area of one stage (double-buffered)
constexpr int RAW_SAMPLES = 64;               // samples of a stage that are staged (16 faces x 4)
constexpr int RAW_G_PITCH = UM + 4;           // floats per gradOutput row (pitch = 4 mod 32: conflict-free 16-byte reads)
__host__ __device__ constexpr int at_blocks(int F) { return (F * CG + 31) / 32; }   // 32-column blocks of the A operand
constexpr int RAW_X_PITCH = 20;               // floats per sample row (16 channels + pad)
constexpr int RAW_G_BYTES = KF * RAW_G_PITCH * 4;
constexpr int RAW_X_BYTES = (RAW_SAMPLES + TREG) * RAW_X_PITCH * 4;   // + pad rows read (and masked) by short faces
constexpr int RAW_B_BYTES = (RAW_SAMPLES + TREG) * 32 * 4;   // F <= 32
constexpr int RAW_B_ITERS = RAW_SAMPLES * 32 / 256;       // 8 floats per thread at most
constexpr int RAW_X_OFF = RAW_G_BYTES;
constexpr int RAW_B_OFF = RAW_X_OFF + RAW_X_BYTES;
constexpr int RAW_C_OFF = RAW_B_OFF + RAW_B_BYTES;
constexpr int RAW_BYTES = (RAW_C_OFF + 128 + 127) / 128 * 128;

// one operand element: tf32-rounded (1 split) or hi + lo (2 splits, lo block `lo_off` bytes further)
template <int NSPLIT>
__device__ __forceinline__ void put4(uint32_t a, uint32_t lo_off, const float4& v) {
    if (NSPLIT == 1) {
        sts_f4(a, make_float4(to_tf32_rna(v.x), to_tf32_rna(v.y), to_tf32_rna(v.z), to_tf32_rna(v.w)));
    } else {
        const float4 h = make_float4(tf32_hi(v.x), tf32_hi(v.y), tf32_hi(v.z), tf32_hi(v.w));
        sts_f4(a, h);
        sts_f4(a + lo_off, make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w));
    }
}

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
    const uint32_t at_sbo = (uint32_t)at_blocks(F) * ATOM_BYTES;             // A block: [4-face group][32-column block][atom]
    const size_t at_bytes = (KF / 4) * (size_t)at_sbo;
    const size_t stage_bytes = (size_t)NSPLIT * (G_TILE_BYTES + at_bytes);   // [g hi][g lo?][A hi][A lo?]
    uint8_t* stages = smem;
    uint8_t* raw = smem + (size_t)S * stage_bytes;            // [2][RAW_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + 2 * RAW_BYTES);
    uint64_t* full = bars;                // [S] 8 producer warps
    uint64_t* empty = bars + S;           // [S] MMA done with the stage
    uint64_t* acc_done = bars + 2 * S;    // all MMAs of the CTA complete
    uint64_t* raw_ready = bars + 2 * S + 1;   // raw rows of a stage staged by all 8 warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], PWARPS); mbar_init(&empty[s], 1); }
        mbar_init(acc_done, 1);
        mbar_init(raw_ready, PWARPS);
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
        const int half = lane >> 4, fl = lane & 15;           // 8-channel half, face of the stage
        constexpr int DMAX = 4;                               // bases per warp: ceil(32 / PWARPS)
        // This thread's 8 consecutive columns 16*g + 8*half (g = warp for the gradOutput block,
        // g = basis d = warp + 8 i for the A block) of K-row fl are 32-byte chunk j of 32-column
        // block g>>1; chunk j of K-row k is stored at chunk j ^ (k & 3).  A quarter warp (faces
        // 0..7 or 8..15, same j) covers two 4-face groups whose lanes would meet in the same
        // 16-byte bank group: the lanes with fl & 4 keep their two 4-channel halves swapped in
        // registers (`sw`), so the first store of a pair lands in the other half of the chunk.
        const uint32_t j32 = 2u * (uint32_t)(warp & 1) + (uint32_t)half;
        const uint32_t sw = (fl & 4) ? 16u : 0u;
        const uint32_t toff = (uint32_t)(warp >> 1) * ATOM_BYTES + (uint32_t)(fl & 3) * 128u + ((j32 ^ (uint32_t)(fl & 3)) << 5) + sw;
        const uint32_t g_off = (uint32_t)(fl >> 2) * G_SBO + toff;
        const uint32_t a_off = (uint32_t)(NSPLIT * G_TILE_BYTES) + (uint32_t)(fl >> 2) * at_sbo + toff;
        const int ptid = tid;
        const uint32_t raw32 = smem_u32(raw), stages32 = smem_u32(stages);
        // the pad rows behind the staged windows are read (their products are masked) but never
        // written by raw_store: clear both buffers once so they hold finite values
        for (int i = tid; i < 2 * RAW_BYTES / 4; i += PWARPS * 32) reinterpret_cast<float*>(raw)[i] = 0.f;
        asm volatile("bar.sync 1, %0;" ::"n"(PWARPS * 32) : "memory");                                 // 0..255 over the producer warps
        // ---- raw staging: what stage `st` needs, copied with coalesced loads
        struct RawRegs { float4 g[2]; float4 x; float b[RAW_B_ITERS]; int cumv; int ks0, ns; };
        // sample range [ks0, ks1) of stage `st`: loaded one stage before the loads that depend on
        // it are issued, so that no warp ever waits on this (dependent) load
        auto ks_pair = [&](int64_t st) -> int2 {
            if (st >= nst) return make_int2(0, 0);
            const int64_t f0 = (st0 + st) * KF;
            const int64_t fe = f0 + KF < p.Nf ? f0 + KF : p.Nf;
            return make_int2(f0 > 0 ? __ldg(p.cum + f0 - 1) : 0, __ldg(p.cum + fe - 1));
        };
        auto raw_issue = [&](int64_t st, int2 ks) -> RawRegs {
            RawRegs R;
            R.g[0] = R.g[1] = zero4(); R.x = zero4(); R.cumv = 0; R.ks0 = 0; R.ns = 0;
#pragma unroll
            for (int i = 0; i < RAW_B_ITERS; ++i) R.b[i] = 0.f;
            if (st >= nst) return R;
            const int64_t f0 = (st0 + st) * KF;
            const int64_t fe = f0 + KF < p.Nf ? f0 + KF : p.Nf;         // one past the stage's last face
            const int ks0 = ks.x, ks1 = ks.y;
            int ns = ks1 - ks0;
            if (ns > RAW_SAMPLES) ns = RAW_SAMPLES;
            R.ks0 = ks0; R.ns = ns;
            // gradOutput rows: 16 faces x Cout floats, contiguous in global memory
            const int c4n = Cout >> 2;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int idx = ptid + i * 256;
                const int fr = idx / 32, c4 = idx - fr * 32;             // up to 128 channels = 32 float4 per row
                if (f0 + fr < fe && c4 < c4n)
                    R.g[i] = ldg4(reinterpret_cast<const float4*>(p.gout + (f0 + fr) * Cout) + c4);
            }
            // this CTA's 16 input channels of every sample: thread = (sample, 16-byte quarter)
            {
                const int sr = ptid >> 2, qd = ptid & 3;
                if (sr < ns) R.x = ldg4(reinterpret_cast<const float4*>(p.in + (int64_t)(ks0 + sr) * Cin + cgp * CG) + qd);
            }
            // bary rows of the stage's samples: one contiguous block of ns*F floats
            {
                const float* src = p.bary + (int64_t)ks0 * F;
                const int nb = ns * F;
#pragma unroll
                for (int i = 0; i < RAW_B_ITERS; ++i) {
                    const int idx = ptid + i * 256;
                    if (idx < nb) R.b[i] = __ldg(src + idx);
                }
            }
            if (ptid <= KF) {                                            // cum[f0-1 .. f0+15]
                const int64_t fi = f0 - 1 + ptid;
                R.cumv = fi < 0 ? 0 : (fi < p.Nf ? __ldg(p.cum + fi) : __ldg(p.cum + p.Nf - 1));
            }
            return R;
        };
        auto raw_store = [&](const RawRegs& R, int buf) {
            uint8_t* rb = raw + (size_t)buf * RAW_BYTES;
            float* g_raw = reinterpret_cast<float*>(rb);
            float* x_raw = reinterpret_cast<float*>(rb + RAW_X_OFF);
            float* b_raw = reinterpret_cast<float*>(rb + RAW_B_OFF);
            int* c_raw = reinterpret_cast<int*>(rb + RAW_C_OFF);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int idx = ptid + i * 256;
                const int fr = idx / 32, c4 = idx - fr * 32;
                *reinterpret_cast<float4*>(g_raw + fr * RAW_G_PITCH + c4 * 4) = R.g[i];
            }
            {
                const int sr = ptid >> 2, qd = ptid & 3;
                *reinterpret_cast<float4*>(x_raw + sr * RAW_X_PITCH + qd * 4) = R.x;
            }
#pragma unroll
            for (int i = 0; i < RAW_B_ITERS; ++i) b_raw[ptid + i * 256] = R.b[i];
            if (ptid <= KF) c_raw[ptid] = R.cumv;
            if (ptid == KF + 1) c_raw[KF + 1] = R.ks0;
            if (ptid == KF + 2) c_raw[KF + 2] = R.ns;
        };
        auto raw_publish = [&]() {
            __syncwarp();
            if (lane == 0) mbar_arrive(raw_ready);
        };

        int si = 0;
        uint32_t sph = 0;
        bool alive = true;
        // Global loads run two stages ahead of the stage being computed (their registers are
        // parked for one stage), the sample-range loads three stages ahead.
        {
            RawRegs R0 = raw_issue(0, ks_pair(0));
            raw_store(R0, 0);
            raw_publish();
        }
        RawRegs Rn = raw_issue(1, ks_pair(1));
        int2 ksn = ks_pair(2);
        for (int64_t st = 0; st < nst && alive; ++st) {
            const RawRegs Rn2 = raw_issue(st + 2, ksn);
            ksn = ks_pair(st + 3);
            {
                int ok = 1;
                if (lane == 0) ok = mbar_wait(raw_ready, (uint32_t)(st & 1), abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
            }
            const uint32_t rb32 = raw32 + (uint32_t)(st & 1) * RAW_BYTES;
            const int64_t f = (st0 + st) * KF + fl;
            const bool valid = f < p.Nf;
            const int k0 = valid ? lds_i32(rb32 + RAW_C_OFF + fl * 4) : 0;
            const int T = valid ? lds_i32(rb32 + RAW_C_OFF + (fl + 1) * 4) - k0 : 0;
            const int ks0 = lds_i32(rb32 + RAW_C_OFF + (KF + 1) * 4), ns = lds_i32(rb32 + RAW_C_OFF + (KF + 2) * 4);
            const int kloc = valid ? k0 - ks0 : 0;             // lanes past the last face read row 0 (masked)
            const float invT = T > 0 ? 1.f / (float)T : 0.f;
            // lean path: every face of the stage has at most TREG samples, all of them staged
            const bool slow = __any_sync(0xffffffffu, (T > TREG) || (kloc + T > ns));
            // wait for the operand stage to be free
            if (!mbar_try_wait(&empty[si], sph ^ 1u)) {
                int ok = 1;
                if (lane == 0) ok = mbar_wait(&empty[si], sph ^ 1u, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
            }
            // shared-window addresses of this thread's first 16-byte store in the gradOutput block
            // and in the A block (basis d = warp + 8 i sits 4 column blocks = 2 KB further on per i);
            // the second store is the other half of the same 32-byte chunk
            const uint32_t sb32 = stages32 + (uint32_t)si * (uint32_t)stage_bytes;
            const uint32_t ga32 = sb32 + g_off, aa32 = sb32 + a_off;
            if (!slow) {
                float x[TREG][8];
                {
                    const uint32_t xa = rb32 + RAW_X_OFF + (uint32_t)kloc * (RAW_X_PITCH * 4) + (uint32_t)half * 32u;
                    const uint32_t xu = xa + sw, xw = xa + (16u - sw);
#pragma unroll
                    for (int t = 0; t < TREG; ++t) {
                        const float4 u = lds_f4(xu + t * (RAW_X_PITCH * 4)), w = lds_f4(xw + t * (RAW_X_PITCH * 4));
                        x[t][0] = u.x; x[t][1] = u.y; x[t][2] = u.z; x[t][3] = u.w;
                        x[t][4] = w.x; x[t][5] = w.y; x[t][6] = w.z; x[t][7] = w.w;
                    }
                }
                {
                    const uint32_t ga = rb32 + (uint32_t)fl * (RAW_G_PITCH * 4) + (uint32_t)(warp * 16 + half * 8) * 4u;
                    const float4 u = lds_f4(ga + sw), w = lds_f4(ga + (16u - sw));
                    put4<NSPLIT>(ga32, G_TILE_BYTES, u);
                    put4<NSPLIT>(ga32 ^ 16u, G_TILE_BYTES, w);
                }
                const uint32_t ba = rb32 + RAW_B_OFF + (uint32_t)(kloc * F) * 4u;
#pragma unroll
                for (int i = 0; i < DMAX; ++i) {
                    const int d = warp + i * PWARPS;
                    if (d < F) {
                        float a[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) a[j] = 0.f;
#pragma unroll
                        for (int t = 0; t < TREG; ++t) {
                            float b = lds_f32(ba + (uint32_t)(t * F + d) * 4u);
                            b = t < T ? b * invT : 0.f;
#pragma unroll
                            for (int j = 0; j < 8; ++j) a[j] = fmaf(b, x[t][j], a[j]);
                        }
                        const uint32_t da32 = aa32 + (uint32_t)i * (4u * ATOM_BYTES);
                        put4<NSPLIT>(da32, (uint32_t)at_bytes, make_float4(a[0], a[1], a[2], a[3]));
                        put4<NSPLIT>(da32 ^ 16u, (uint32_t)at_bytes, make_float4(a[4], a[5], a[6], a[7]));
                    }
                }
            } else {
                // generic path, straight from global memory
                float g8[8];
                const int co0 = warp * 16 + half * 8;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int co = co0 + (j ^ (int)(sw >> 2));                 // halves swapped where sw is set
                    g8[j] = (valid && co < Cout) ? __ldg(p.gout + f * Cout + co) : 0.f;
                }
                put4<NSPLIT>(ga32, G_TILE_BYTES, make_float4(g8[0], g8[1], g8[2], g8[3]));
                put4<NSPLIT>(ga32 ^ 16u, G_TILE_BYTES, make_float4(g8[4], g8[5], g8[6], g8[7]));
                for (int d = warp; d < F; d += PWARPS) {
                    float a[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) a[j] = 0.f;
                    for (int t = 0; t < T; ++t) {
                        const float b = __ldg(p.bary + (int64_t)(k0 + t) * F + d) * invT;
                        const float* xr = p.in + (int64_t)(k0 + t) * Cin + cgp * CG + half * 8;
#pragma unroll
                        for (int j = 0; j < 8; ++j) a[j] = fmaf(b, __ldg(xr + (j ^ (int)(sw >> 2))), a[j]);
                    }
                    const uint32_t da32 = aa32 + (uint32_t)((d - warp) >> 3) * (4u * ATOM_BYTES);
                    put4<NSPLIT>(da32, (uint32_t)at_bytes, make_float4(a[0], a[1], a[2], a[3]));
                    put4<NSPLIT>(da32 ^ 16u, (uint32_t)at_bytes, make_float4(a[4], a[5], a[6], a[7]));
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[si]);
            if (++si == S) { si = 0; sph ^= 1u; }
            // every warp has passed raw_ready(st), so nobody reads the other raw buffer any more
            raw_store(Rn, (int)((st + 1) & 1));
            raw_publish();
            Rn = Rn2;
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
            const uint32_t idesc1 = instr_desc_mnmajor(FMT_TF32, UM, (uint32_t)n1);
            const uint32_t idesc2 = instr_desc_mnmajor(FMT_TF32, UM, (uint32_t)(n2 > 0 ? n2 : 16));
            const uint64_t dbase_g = smem_desc_mnmajor_b32(smem_u32(stages), ATOM_BYTES, G_SBO);
            const uint64_t dbase_a = smem_desc_mnmajor_b32(smem_u32(stages) + NSPLIT * G_TILE_BYTES, ATOM_BYTES, at_sbo);
            int si = 0;
            uint32_t sph = 0;
            bool alive = true;
            for (int64_t st = 0; st < nst; ++st) {
                if (!mbar_wait(&full[si], sph, abort_flag)) { alive = false; break; }
                tc_fence_after();
                const uint64_t soff = (uint64_t)(((uint32_t)si * (uint32_t)stage_bytes) >> 4);
                const uint64_t dg_hi0 = dbase_g + soff, da_hi0 = dbase_a + soff;
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) {                        // one instruction = 8 faces = two 4-face groups
                    const uint32_t first = (st != 0 || k2 != 0) ? 1u : 0u;
                    for (int c = 0; c < (n2 > 0 ? 2 : 1); ++c) {
                        const uint32_t d_tmem = tmem_base + (uint32_t)(c * 256);
                        const uint32_t idesc = c == 0 ? idesc1 : idesc2;
                        const uint64_t dg_hi = dg_hi0 + (uint64_t)((k2 * 2 * G_SBO) >> 4);
                        const uint64_t da_hi = da_hi0 + (uint64_t)(((uint32_t)k2 * 2u * at_sbo + (uint32_t)c * (8u * ATOM_BYTES)) >> 4);
                        if (NSPLIT == 1) {
                            mma_tf32(d_tmem, dg_hi, da_hi, idesc, first);
                        } else {
                            const uint64_t dg_lo = dg_hi + (uint64_t)(G_TILE_BYTES >> 4);
                            const uint64_t da_lo = da_hi + (uint64_t)(at_bytes >> 4);
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
    return Cin % CG == 0 && Cout % 4 == 0 && Cout >= 4 && Cout <= UM && F >= 1 && F <= 32;   // F*16 <= 512 columns
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
    size_t stage = (size_t)pl.nsplit * (G_TILE_BYTES + (KF / 4) * (size_t)at_blocks(F) * ATOM_BYTES);
    int S = 4;
    const size_t extra = 2 * (size_t)RAW_BYTES + 1024 + 256;
    while (S > 2 && (size_t)S * stage + extra > 224 * 1024) --S;
    pl.nstages = S;
    pl.smem = (size_t)S * stage + extra;
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

// facet2facet filter gradient on tcgen05 + TMEM, one fused kernel:
//
//   gradFilter[co, ci, d] = sum_f g[f,co] * A[f,d,ci],   A[f,d,ci] = (1/T_f) sum_k bary[k,d]*in[k,ci]
//
// The reduction runs over FACES, so faces are the K dimension of the tensor-core product
// D[co, (d,kk)] += g^T[co, f] * A^T[(d,kk), f].  A CTA owns one group of 16 input channels
// (its F*16 <= 512 accumulator columns live in TMEM for the whole kernel) and one contiguous
// chunk of faces.  Per stage of 16 faces three roles cooperate through mbarriers:
//   * two loader warps fill a ring of raw buffers: one writes a record per face (first
//     sample, sample count, 1/T) and fetches the stage's bary rows with one bulk copy (from a
//     copy of bary whose rows are padded to a multiple of 4 floats), the other fetches the
//     CTA's 16 input channels of every sample with 16-byte asynchronous copies into per-face
//     slots; the sample ranges they need are loaded three stages ahead;
//   * both operands live in shared memory MN-major (128-byte swizzle): a face is a K-row whose
//     128-byte pieces hold consecutive output channels (gradOutput block) or consecutive
//     (basis, channel) columns (A block), so neither operand is transposed and every store is
//     a vector.  8 compute warps build the A block: warp w the columns of bases 4w..4w+3
//     (thread = face x 8 channels, one 16-byte bary load per sample);
//   * 4 warps write the gradOutput block: each copies 4 of the stage's 16 rows straight from
//     global memory (registers, one stage ahead), splits and stores them -- on warps of their
//     own this work overlaps the compute warps' chains instead of lengthening them (-7 %);
//   * one thread issues tcgen05.mma (M = 128 output channels, N = F*16 in chunks of <= 256,
//     K = 8 faces per instruction) and commits the stage back.
// What bounds it: every 16-byte shared-memory access of a warp costs at least 4 passes of the
// load/store pipe, so the layout of every access is chosen to touch 512 distinct bytes; in
// the hi+lo mode the three MMAs per product read their operands from shared memory three
// times, and that traffic (about 123 KB per stage) is the floor.
// Every 256 stages the accumulator is added to a running sum in global memory and restarted (the
// tensor core's adder truncates; see FLUSH_STAGES).  At the end accumulator + running sum go to
// partial[chunk] (final gradFilter layout); a second kernel adds the chunks in order, so the result
// is deterministic.
// Modes: 1 split (bf16 or tf32 operands) or 2 splits (bf16 or tf32 hi+lo, three MMAs per k-step).
#include <type_traits>
#include "common.cuh"
#include "tc_ptx.cuh"
#include "tc_runtime.cuh"

namespace pb {
namespace tc {

namespace gfilter {

using namespace ptx;

constexpr int UM = 128;                       // output channels (UMMA M), Cout zero-padded
constexpr int CG = 16;                        // input channels per CTA
constexpr int KF = 16;                        // faces per stage (four groups of 4 K-rows, two per instruction)
constexpr int CWARPS = 8;                     // compute warps 0..7: two faces x 16 channels each
constexpr int REC_WARP = CWARPS;              // loader: face records + bary block
constexpr int X_WARP = CWARPS + 1;            // loader: sample rows
constexpr int MMA_WARP = CWARPS + 2;
constexpr int G_WARP = CWARPS + 3;            // first of the warps that write the gradOutput operand
constexpr int GWARPS = 4;
constexpr int GROWS = KF / GWARPS;            // rows of a stage per such warp
constexpr int NTHREADS = (CWARPS + 3 + GWARPS) * 32;
static_assert(CWARPS * 16 == UM && CWARPS * 2 == KF, "one 16-channel gradOutput unit and two faces per compute warp");
constexpr int ATOM_BYTES = 512;               // 4 K-rows x 128 bytes (32 M/N elements)
constexpr int G_SBO = (UM / 32) * ATOM_BYTES; // gradOutput block: [4-face group][32-channel block][atom]
constexpr int G_TILE_BYTES = (KF / 4) * G_SBO;
constexpr int TREG = 4;                       // samples per face on the fast path
// The tensor core adds into its accumulator with truncation, so a long chain of accumulating
// products drifts towards zero (measured: -1.2e-3 relative over the 26 000 stages a CTA walks on a
// 7.4 M-face batch, -1.2e-5 over 256).  Every FLUSH_STAGES stages the accumulator is therefore added
// (round-to-nearest, CUDA cores) to a running sum of the CTA in global memory and restarted.
#ifndef PB_GF_FLUSH_STAGES
#define PB_GF_FLUSH_STAGES 256
#endif
constexpr int FLUSH_STAGES = PB_GF_FLUSH_STAGES;
__host__ __device__ constexpr int at_blocks(int F) { return (F * CG + 31) / 32; }   // 32-column blocks of the A operand

// one raw buffer: what a stage needs from global memory, as it lies there
constexpr int RAW_SAMPLES = 64;               // samples of a stage that are staged (16 faces x 4)
// Sample rows are staged per face: slot fl*4 + t (128 bytes) holds the CTA's 16 channels of
// sample t of face fl as four 16-byte pieces, piece q at chunk q ^ (fl & 7) -- the 8 lanes of
// a quarter warp (8 faces) then read 8 distinct bank groups.
constexpr int RAW_X_SLOT = 128;
constexpr int RAW_X_BYTES = KF * TREG * RAW_X_SLOT;
constexpr int RAW_B_BYTES = (RAW_SAMPLES + TREG) * 32 * 4;            // bary rows padded to Fp <= 32 floats; + rows read (weight 0) by short faces
constexpr int RAW_REC_BYTES = KF * 16 + 32;   // per face {first sample - ks0, T, 1/T, first sample}; then {slow, 0, ks0, ns}
constexpr int RAW_X_OFF = 0;
constexpr int RAW_B_OFF = RAW_X_OFF + RAW_X_BYTES;
constexpr int RAW_REC_OFF = RAW_B_OFF + RAW_B_BYTES;
constexpr int RAW_BYTES = (RAW_REC_OFF + RAW_REC_BYTES + 127) / 128 * 128;
static_assert(RAW_X_OFF % 16 == 0 && RAW_B_OFF % 16 == 0 && RAW_REC_OFF % 16 == 0, "copy destinations are 16-byte aligned");

// 16-byte asynchronous copy global -> shared (no register staging), and the arrival of all
// such copies of the calling thread on an mbarrier (counted in the barrier's expected arrivals)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void sts_i4(uint32_t a, int x, int y, int z, int w) {
    asm volatile("st.shared.v4.s32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ int4 lds_i4(uint32_t a) {
    int4 v;
    asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}

// four operand elements: tf32-rounded (1 split) or hi + lo (2 splits, lo block `lo_off` bytes further)
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

// bf16 operands (MN-major, 128-byte swizzle): a K-row piece of 128 bytes holds 64 columns, an
// atom 8 K-rows; blocks of 64 columns are 1 KB apart, the two 8-face groups of a stage
// `blocks` KB apart.
constexpr int BATOM_BYTES = 1024;
constexpr int BG_SBO = (UM / 64) * BATOM_BYTES;
constexpr int BG_TILE_BYTES = (KF / 8) * BG_SBO;
__host__ __device__ constexpr int at_blocks_b16(int F) { return (F * CG + 63) / 64; }
__device__ __forceinline__ void sts_u2(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sts_u4(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// eight operand elements as bf16 (1 split) or bf16 hi + bf16 lo (2 splits): one 16-byte store each
template <int NSPLIT>
__device__ __forceinline__ void put8_b16(uint32_t a, uint32_t lo_off, const float4& u, const float4& w) {
    uint32_t hi[4], lo[4];
    if (NSPLIT == 1) {
        hi[0] = pack_bf16x2(u.x, u.y); hi[1] = pack_bf16x2(u.z, u.w); hi[2] = pack_bf16x2(w.x, w.y); hi[3] = pack_bf16x2(w.z, w.w);
        sts_u4(a, hi[0], hi[1], hi[2], hi[3]);
    } else {
        split_bf16x2(u.x, u.y, hi[0], lo[0]); split_bf16x2(u.z, u.w, hi[1], lo[1]);
        split_bf16x2(w.x, w.y, hi[2], lo[2]); split_bf16x2(w.z, w.w, hi[3], lo[3]);
        sts_u4(a, hi[0], hi[1], hi[2], hi[3]);
        sts_u4(a + lo_off, lo[0], lo[1], lo[2], lo[3]);
    }
}
// four elements: one 8-byte store each
template <int NSPLIT>
__device__ __forceinline__ void put4_b16(uint32_t a, uint32_t lo_off, const float4& v) {
    uint32_t hi[2], lo[2];
    if (NSPLIT == 1) {
        sts_u2(a, pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    } else {
        split_bf16x2(v.x, v.y, hi[0], lo[0]); split_bf16x2(v.z, v.w, hi[1], lo[1]);
        sts_u2(a, hi[0], hi[1]);
        sts_u2(a + lo_off, lo[0], lo[1]);
    }
}

// one whole warp waits on an mbarrier phase: every lane probes once, then lane 0 waits (bounded)
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity) ? 1 : 0)) return true;
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok) (void)mbar_try_wait(bar, parity);   // every lane observes the completed phase itself
    return ok != 0;
}

// One compute warp's share of a flush: its TMEM lane quadrant, every second group of 32 accumulator
// columns, added to (or, the first time, stored as) the CTA's running sum.  Kept out of line so that its
// 32 staging registers do not count against the operand-building loop it is called from.
__device__ __noinline__ void flush_accumulator(uint32_t tmem_quadrant, float* run, int first_group, int ngroups,
                                               bool add) {
    for (int gi = first_group; gi < ngroups; gi += CWARPS / 4) {
        uint32_t r[32];
        tmem_ld32(tmem_quadrant + (uint32_t)(gi * 32), r);
        tmem_ld_wait();
        float* dst = run + (size_t)(gi * 32) * UM;
        if (add) {
#pragma unroll
            for (int j = 0; j < 32; ++j) dst[(size_t)j * UM] += __uint_as_float(r[j]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) dst[(size_t)j * UM] = __uint_as_float(r[j]);
        }
    }
}

struct Params {
    int64_t Nf;
    int Cin, Cout, F;         // Cin: channels of `in` (a multiple of 16); Cout: output channels of this launch's chunk
    int CinF, CoutF, co0;     // channels of the filter gradient, and the chunk's first output channel
    int Fp;                   // floats per row of the padded bary copy (F rounded up to 4)
    int ncg;                  // channel groups = Cin / 16
    int nchunks;              // face chunks
    int64_t stages_per_chunk; // 16-face stages per chunk
    int nstages;              // operand ring depth
    int nraw;                 // raw ring depth
    const float* gout;
    const float* in;
    const float* bary;        // padded copy: [samples][Fp], pad columns zero
    const int32_t* cum;
    float* partial;           // [nchunks][Cout*Cin*F]
    float* running;           // [CTA][accumulator columns rounded up to 32][128 output channels]
    int* async_err;
    int wait_budget;          // bounded waits give up after this many units of 1024 clocks
};

template <int NSPLIT, bool BF>
__global__ void __launch_bounds__(NTHREADS, 1) f2f_bwd_gfilter_tc_kernel(Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.nstages, NRAW = p.nraw, F = p.F, Cin = p.Cin, Cout = p.Cout;
    const int NR = F * CG;                                   // accumulator columns / A columns
    // A block: [face group][column block][atom]; tf32: groups of 4 faces, blocks of 32 columns, 512-byte
    // atoms; bf16: groups of 8 faces, blocks of 64 columns, 1 KB atoms
    const uint32_t at_sbo = BF ? (uint32_t)at_blocks_b16(F) * BATOM_BYTES : (uint32_t)at_blocks(F) * ATOM_BYTES;
    const size_t at_bytes = (BF ? KF / 8 : KF / 4) * (size_t)at_sbo;
    constexpr uint32_t GT = BF ? BG_TILE_BYTES : G_TILE_BYTES;              // gradOutput block of one split
    const size_t stage_bytes = (size_t)NSPLIT * (GT + at_bytes);             // [g hi][g lo?][A hi][A lo?]
    uint8_t* stages = smem;
    uint8_t* raw = smem + (size_t)S * stage_bytes;            // [NRAW][RAW_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + (size_t)NRAW * RAW_BYTES);
    uint64_t* full = bars;                        // [S]    operands of a stage written by all compute warps
    uint64_t* empty = bars + S;                   // [S]    MMA done with the stage
    uint64_t* raw_ready = bars + 2 * S;           // [NRAW] copies of a raw buffer landed, records written
    uint64_t* raw_free = bars + 2 * S + NRAW;     // [NRAW] all compute warps done with a raw buffer
    uint64_t* acc_done = bars + 2 * S + 2 * NRAW; // all MMAs issued so far complete (once per flush, once at the end)
    uint64_t* acc_free = acc_done + 1;            // all compute warps have read the accumulator out
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], CWARPS + GWARPS); mbar_init(&empty[s], 1); }
        // the sample-row warp's 32 asynchronous-copy arrivals + the record warp's arrival that
        // announces the bulk-copy bytes
        for (int r = 0; r < NRAW; ++r) { mbar_init(&raw_ready[r], 33); mbar_init(&raw_free[r], CWARPS); }
        mbar_init(acc_done, 1);
        mbar_init(acc_free, CWARPS);
        abort_flag[0] = 0;
        abort_flag[1] = p.wait_budget;
        fence_barrier_init();
    }
    // Pad rows and pad columns of the raw buffers are read (their products are masked) but never
    // written by a copy: clear the buffers once so that they hold finite values.  The copies that
    // overwrite them later go through the asynchronous proxy.
    for (int i = tid; i < NRAW * RAW_BYTES / 4; i += NTHREADS) reinterpret_cast<float*>(raw)[i] = 0.f;
    fence_proxy_async();
    if (warp == MMA_WARP) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
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
    const uint32_t raw32 = smem_u32(raw), stages32 = smem_u32(stages);
    // The accumulator is flushed after stage b when (b + 1) is a multiple of FLUSH_STAGES.  The compute
    // warps do it S stages later (before they build stage b + S), so that the operand ring is full
    // when the products resume; a boundary too close to the end of the chunk is left to the final drain.
    // (every role counts stages of the chunk in 32 bits: a chunk has fewer than 2^31 stages)
    const int nst32 = (int)nst;

    if (warp == REC_WARP || warp == X_WARP) {
        // ===================================== loaders =====================================
        // lane l holds cum[f0 - 1 + l] of a stage (l = 0..16): the sample ranges of its 16 faces.
        // Both loader warps keep the values of the next three stages in registers.
        auto load_cum = [&](int64_t st) -> int {
            if (st >= nst || lane > KF) return 0;
            int64_t fi = (st0 + st) * KF - 1 + lane;
            if (fi < 0) return 0;
            if (fi > p.Nf - 1) fi = p.Nf - 1;
            return __ldg(p.cum + fi);
        };
        int cv = load_cum(0), cv1 = load_cum(1), cv2 = load_cum(2);
        int rbuf = 0;
        uint32_t rph = 0;
        for (int64_t st = 0; st < nst; ++st) {
            const int cv3 = load_cum(st + 3);                // in flight for three stages
            if (!warp_wait(&raw_free[rbuf], rph ^ 1u, abort_flag, lane)) break;
            const uint32_t rb32 = raw32 + (uint32_t)rbuf * RAW_BYTES;
            uint64_t* bar = &raw_ready[rbuf];
            const int64_t f0 = (st0 + st) * KF;
            const int nvf = p.Nf - f0 < KF ? (int)(p.Nf - f0) : KF;          // faces of the stage
            const int ks0 = __shfl_sync(0xffffffffu, cv, 0), ks1 = __shfl_sync(0xffffffffu, cv, nvf);
            const int k1 = __shfl_down_sync(0xffffffffu, cv, 1);
            const bool face = lane < nvf;
            const int T = face ? k1 - cv : 0, kloc = face ? cv - ks0 : 0;
            int ns = ks1 - ks0;
            if (ns > RAW_SAMPLES) ns = RAW_SAMPLES;
            const int slow = __any_sync(0xffffffffu, (T > TREG) || (kloc + T > ns)) ? 1 : 0;
            if (warp == REC_WARP) {
                if (lane < KF) sts_i4(rb32 + RAW_REC_OFF + lane * 16, kloc, T, __float_as_int(T > 0 ? 1.f / (float)T : 0.f), cv);
                const int one = __any_sync(0xffffffffu, T > 1) ? 0 : 1;          // no face of the stage has a second sample
                if (lane == KF) sts_i4(rb32 + RAW_REC_OFF + KF * 16, slow, one, ks0, ns);
                __syncwarp();
                if (lane == 0) {
                    // the stage's bary rows: one bulk copy (rows are 16-byte multiples)
                    const uint32_t bbytes = (uint32_t)(ns * p.Fp * 4);
                    mbar_arrive_expect_tx(bar, bbytes);
                    if (bbytes > 0) bulk_g2s(raw + (size_t)rbuf * RAW_BYTES + RAW_B_OFF, p.bary + (int64_t)ks0 * p.Fp, bbytes, bar);
                }
            } else {
                // this CTA's 16 input channels of the first TREG samples of every face:
                // (face, sample, 16-byte quarter) per lane
                const float* xsrc = p.in + cgp * CG;
#pragma unroll
                for (int i = 0; i < KF * TREG * 4 / 32; ++i) {
                    const int idx = lane + i * 32, qd = idx & 3, t = (idx >> 2) & 3, xf = idx >> 4;
                    const int Tf = __shfl_sync(0xffffffffu, T, xf), kf = __shfl_sync(0xffffffffu, cv, xf);
                    if (t < Tf && !slow)
                        cp_async16(rb32 + RAW_X_OFF + (uint32_t)((xf * TREG + t) * RAW_X_SLOT + ((qd ^ (xf & 7)) << 4)),
                                   xsrc + (int64_t)(kf + t) * Cin + qd * 4);
                }
                cp_async_arrive(bar);
            }
            cv = cv1; cv1 = cv2; cv2 = cv3;
            if (++rbuf == NRAW) { rbuf = 0; rph ^= 1u; }
        }
    } else if (warp < CWARPS) {
        // ================================== compute warps ==================================
        // --- A block: warp q builds the columns of bases 4q..4q+3; thread = (face fl, 8 channels).
        // Column n = d*16 + channel; the thread's 8 columns of basis d are 32-byte chunk
        // 2*(d&1) + half of 32-column block d>>1, and chunk j of K-row k is stored at j ^ (k&3).
        // A quarter warp (faces 0..7 or 8..15) covers two 4-face groups whose lanes would meet in
        // the same 16-byte bank group: the lanes with fl & 4 keep their two 4-channel halves
        // swapped in registers (`sw`), so the first store of a pair lands in the other half.
        const int half = lane >> 4, fl = lane & 15;
        // bf16: the thread's 8 columns of basis 4q + dd are 16-byte chunk 2*dd + half of 64-column
        // block q, chunk c of K-row k is stored at c ^ (k & 7): the 8 lanes of a quarter warp hit 8
        // distinct bank groups without any swap.
        const uint32_t sw = BF ? 0u : ((fl & 4) ? 16u : 0u);
        const uint32_t a_row = BF ? (uint32_t)(NSPLIT * GT) + (uint32_t)(fl >> 3) * at_sbo + (uint32_t)(fl & 7) * 128u
                                        + (uint32_t)warp * BATOM_BYTES
                                  : (uint32_t)(NSPLIT * GT) + (uint32_t)(fl >> 2) * at_sbo + (uint32_t)(fl & 3) * 128u
                                        + (uint32_t)(2 * warp) * ATOM_BYTES + sw;
        const uint32_t a_off0 = a_row + (((uint32_t)half ^ (uint32_t)(fl & 3)) << 5);          // tf32, even bases
        const uint32_t a_off1 = a_row + (((2u + (uint32_t)half) ^ (uint32_t)(fl & 3)) << 5);   // tf32, odd bases
        // byte address (inside a stage) of the thread's 8 columns of basis 4q + dd
        auto a_addr = [&](int dd) -> uint32_t {
            if (BF) return a_row + (((uint32_t)(2 * dd + half) ^ (uint32_t)(fl & 7)) << 4);
            return ((dd & 1) ? a_off1 : a_off0) + (uint32_t)(dd >> 1) * ATOM_BYTES;
        };
        // the thread's 8 values of a basis (first four, last four) into the A block
        auto put_a = [&](uint32_t sb32, int dd, const float4& u, const float4& w) {
            const uint32_t da32 = sb32 + a_addr(dd);
            if (BF) put8_b16<NSPLIT>(da32, (uint32_t)at_bytes, u, w);
            else { put4<NSPLIT>(da32, (uint32_t)at_bytes, u); put4<NSPLIT>(da32 ^ 16u, (uint32_t)at_bytes, w); }
        };
        const bool has_unit = 4 * warp < F;
        // --- gradOutput block: warp w copies the rows of faces 2w and 2w+1 straight from global
        // memory (registers, two stages ahead): lane l holds channels 4l..4l+3 of both, so a warp
        // load reads one whole row and the 8 lanes of a quarter warp store 128 consecutive bytes
        // of the face's K-row (16-byte piece l&7 of 32-channel block l>>3).
        // (bf16: 8-byte piece l&15 of 64-channel block l>>4)
        int si = 0, rbuf = 0;
        uint32_t sph = 0, rph = 0, aph = 0;
        bool alive = true, flushed = false;
        const int dq = warp & 3, dhalf = warp >> 2;      // TMEM lane quadrant, half of the 32-column groups
        const int ngroups = (NR + 31) / 32;
        float* run = p.running + ((size_t)blockIdx.x * (size_t)(ngroups * 32)) * UM + (dq * 32 + lane);
        int to_flush = FLUSH_STAGES + S;                 // iterations until the next flush is due here
        for (int st = 0; st < nst32; ++st) {
            if (--to_flush == 0) {                       // stage st - S closed a run of FLUSH_STAGES stages
                to_flush = FLUSH_STAGES;
                // running sum += accumulator (a thread meets the same addresses at every flush)
                if (!warp_wait(acc_done, aph, abort_flag, lane)) { alive = false; break; }
                aph ^= 1u;
                tc_fence_after();
                flush_accumulator(tmem_base + ((uint32_t)(dq * 32) << 16), run, dhalf, ngroups, flushed);
                flushed = true;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_free);
            }
            if (!warp_wait(&raw_ready[rbuf], rph, abort_flag, lane)) { alive = false; break; }
            const uint32_t rb32 = raw32 + (uint32_t)rbuf * RAW_BYTES;
            const int4 rec = lds_i4(rb32 + RAW_REC_OFF + fl * 16);           // {kloc, T, 1/T, first sample}
            const int slow = lds_i32(rb32 + RAW_REC_OFF + KF * 16);
            const int kloc = rec.x, T = rec.y;
            const float invT = __int_as_float(rec.z);
            if (!warp_wait(&empty[si], sph ^ 1u, abort_flag, lane)) { alive = false; break; }
            const uint32_t sb32 = stages32 + (uint32_t)si * (uint32_t)stage_bytes;
            // fast path: every face of the stage has at most TR samples (TR = 1: one product per operand element
            // instead of TREG multiply-adds), all of them staged.
            // (Rows behind a face's last sample belong to other faces or are stale: their weight
            // is zero, so they only matter if the input holds non-finite values.)
            auto fast = [&](auto trc) {
                constexpr int TR = decltype(trc)::value;
                float2 x[TR][4];
                float4 b[TR];
                {
                    const uint32_t xa = rb32 + RAW_X_OFF + (uint32_t)fl * (TREG * RAW_X_SLOT);
                    const uint32_t qu = 2u * (uint32_t)half + (sw >> 4);            // 16-byte quarter held first
                    const uint32_t xu = xa + ((qu ^ (uint32_t)(fl & 7)) << 4), xw = xa + (((qu ^ 1u) ^ (uint32_t)(fl & 7)) << 4);
                    const uint32_t ba = rb32 + RAW_B_OFF + (uint32_t)(kloc * p.Fp + 4 * warp) * 4u;
#pragma unroll
                    for (int t = 0; t < TR; ++t) {
                        const float4 u = lds_f4(xu + t * RAW_X_SLOT), w = lds_f4(xw + t * RAW_X_SLOT);
                        b[t] = lds_f4(ba + (uint32_t)(t * p.Fp) * 4u);
                        const float wt = t < T ? invT : 0.f;
                        x[t][0] = make_float2(u.x * wt, u.y * wt); x[t][1] = make_float2(u.z * wt, u.w * wt);
                        x[t][2] = make_float2(w.x * wt, w.y * wt); x[t][3] = make_float2(w.z * wt, w.w * wt);
                    }
                }
#pragma unroll
                for (int dd = 0; dd < 4; ++dd) {
                    if (4 * warp + dd < F) {
                        float2 a[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) a[j] = make_float2(0.f, 0.f);
#pragma unroll
                        for (int t = 0; t < TR; ++t) {
                            const float bv = dd == 0 ? b[t].x : dd == 1 ? b[t].y : dd == 2 ? b[t].z : b[t].w;
                            const float2 b2 = make_float2(bv, bv);
#pragma unroll
                            for (int j = 0; j < 4; ++j) a[j] = TR == 1 ? __fmul2_rn(b2, x[t][j]) : __ffma2_rn(b2, x[t][j], a[j]);
                        }
                        put_a(sb32, dd, make_float4(a[0].x, a[0].y, a[1].x, a[1].y), make_float4(a[2].x, a[2].y, a[3].x, a[3].y));
                    }
                }
            };
            if (has_unit && !slow) {
                if (lds_i32(rb32 + RAW_REC_OFF + KF * 16 + 4)) fast(std::integral_constant<int, 1>{});
                else fast(std::integral_constant<int, TREG>{});
            } else if (has_unit) {
                // generic path, straight from global memory (halves swapped where sw is set)
                const int k0 = rec.w, jsw = (int)(sw >> 2);
                for (int dd = 0; dd < 4; ++dd) {
                    const int d = 4 * warp + dd;
                    if (d >= F) break;
                    float a[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) a[j] = 0.f;
                    for (int t = 0; t < T; ++t) {
                        const float bv = __ldg(p.bary + (int64_t)(k0 + t) * p.Fp + d) * invT;
                        const float* xr = p.in + (int64_t)(k0 + t) * Cin + cgp * CG + half * 8;
#pragma unroll
                        for (int j = 0; j < 8; ++j) a[j] = fmaf(bv, __ldg(xr + (j ^ jsw)), a[j]);
                    }
                    put_a(sb32, dd, make_float4(a[0], a[1], a[2], a[3]), make_float4(a[4], a[5], a[6], a[7]));
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&full[si]); mbar_arrive(&raw_free[rbuf]); }
            if (++si == S) { si = 0; sph ^= 1u; }
            if (++rbuf == NRAW) { rbuf = 0; rph ^= 1u; }
        }
        // ==================================== drain ====================================
        if (alive && warp_wait(acc_done, aph, abort_flag, lane)) {
            tc_fence_after();
            const int co = dq * 32 + lane;
            float* out = p.partial + (int64_t)chunk * p.CoutF * p.CinF * F;
            for (int gi = dhalf; gi < ngroups; gi += CWARPS / 4) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(dq * 32) << 16) + (uint32_t)(gi * 32), r);
                tmem_ld_wait();
                const float* src = run + (size_t)(gi * 32) * UM;
                if (co < Cout) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        int col = gi * 32 + j;
                        if (col < NR) {
                            const int d = col / CG, kk = col - d * CG, ci = cgp * CG + kk;
                            if (ci < p.CinF) {
                                float v = nst > 0 ? __uint_as_float(r[j]) : 0.f;
                                if (flushed) v += src[(size_t)j * UM];
                                out[((int64_t)(p.co0 + co) * p.CinF + ci) * F + d] = v;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
        }
    } else if (warp >= G_WARP) {
        const int gw = warp - G_WARP;
        // ================================ gradOutput operand ================================
        // lane l holds channels 4l..4l+3 of the stage's 16 rows (one stage ahead in registers) and writes
        // them as K-rows of the MN-major operand: 16-byte piece l&7 of 32-channel block l>>3 (tf32),
        // 8-byte piece l&15 of 64-channel block l>>4 (bf16)
        auto g_row_off = [&](int k) -> uint32_t {
            if (BF)
                return (uint32_t)(k >> 3) * BG_SBO + (uint32_t)(k & 7) * 128u + (uint32_t)(lane >> 4) * BATOM_BYTES
                       + ((((uint32_t)(lane & 15) >> 1) ^ (uint32_t)(k & 7)) << 4) + (uint32_t)(lane & 1) * 8u;
            return (uint32_t)(k >> 2) * G_SBO + (uint32_t)(k & 3) * 128u + (uint32_t)(lane >> 3) * ATOM_BYTES
                   + ((((uint32_t)(lane & 7) >> 1) ^ (uint32_t)(k & 3)) << 5) + (uint32_t)(lane & 1) * 16u;
        };
        float4 cur[GROWS], nxt[GROWS];
        auto load_rows = [&](int64_t st, float4 (&dst)[GROWS]) {
#pragma unroll
            for (int k = 0; k < GROWS; ++k) {
                dst[k] = zero4();
                const int64_t f = (st0 + st) * KF + gw * GROWS + k;
                if (st < nst && 4 * lane < Cout && f < p.Nf)
                    dst[k] = ldg4(reinterpret_cast<const float4*>(p.gout + f * p.CoutF + p.co0) + lane);
            }
        };
        load_rows(0, cur);
        int si = 0;
        uint32_t sph = 0;
        for (int64_t st = 0; st < nst; ++st) {
            load_rows(st + 1, nxt);
            if (!warp_wait(&empty[si], sph ^ 1u, abort_flag, lane)) break;
            const uint32_t sb32 = stages32 + (uint32_t)si * (uint32_t)stage_bytes;
#pragma unroll
            for (int k = 0; k < GROWS; ++k) {
                if (BF) put4_b16<NSPLIT>(sb32 + g_row_off(gw * GROWS + k), GT, cur[k]);
                else put4<NSPLIT>(sb32 + g_row_off(gw * GROWS + k), GT, cur[k]);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[si]);
#pragma unroll
            for (int k = 0; k < GROWS; ++k) cur[k] = nxt[k];
            if (++si == S) { si = 0; sph ^= 1u; }
        }
    } else {
        // ==================================== MMA issuer ====================================
        if (lane == 0) {
            const int n1 = NR < 256 ? NR : 256, n2 = NR - n1;
            const uint32_t idesc1 = instr_desc_mnmajor(BF ? FMT_BF16 : FMT_TF32, UM, (uint32_t)n1);
            const uint32_t idesc2 = instr_desc_mnmajor(BF ? FMT_BF16 : FMT_TF32, UM, (uint32_t)(n2 > 0 ? n2 : 16));
            const uint64_t dbase_g = BF ? smem_desc_mnmajor_b16(stages32, BATOM_BYTES, BG_SBO)
                                        : smem_desc_mnmajor_b32(stages32, ATOM_BYTES, G_SBO);
            const uint64_t dbase_a = BF ? smem_desc_mnmajor_b16(stages32 + NSPLIT * GT, BATOM_BYTES, at_sbo)
                                        : smem_desc_mnmajor_b32(stages32 + NSPLIT * GT, ATOM_BYTES, at_sbo);
            // tf32: one instruction = 8 faces = two 4-face groups, two per stage; bf16: one
            // instruction = 16 faces = two 8-face groups, one per stage
            constexpr int KSTEPS = BF ? 1 : 2;
            const uint32_t g_kstep = 2 * G_SBO, a_kstep = 2 * at_sbo;
            const uint32_t n_chunk = BF ? 4u * BATOM_BYTES : 8u * ATOM_BYTES;      // 256 columns further on
            int si = 0;
            uint32_t sph = 0, fph = 0;
            bool alive = true, fresh = true;                 // fresh: the next product overwrites the accumulator
            int run_len = 0;                                 // stages added to the accumulator since it was restarted
            bool wait_free = false;
            for (int st = 0; st < nst32; ++st) {
                if (!mbar_wait(&full[si], sph, abort_flag)) { alive = false; break; }
                if (wait_free) {                             // the compute warps have read the accumulator out
                    wait_free = false;
                    if (!mbar_wait(acc_free, fph, abort_flag)) { alive = false; break; }
                    fph ^= 1u;
                    fresh = true;
                }
                tc_fence_after();
                const uint64_t soff = (uint64_t)(((uint32_t)si * (uint32_t)stage_bytes) >> 4);
                const uint64_t dg_hi0 = dbase_g + soff, da_hi0 = dbase_a + soff;
#pragma unroll
                for (int k2 = 0; k2 < KSTEPS; ++k2) {
                    const uint32_t first = (!fresh || k2 != 0) ? 1u : 0u;
                    for (int c = 0; c < (n2 > 0 ? 2 : 1); ++c) {
                        const uint32_t d_tmem = tmem_base + (uint32_t)(c * 256);
                        const uint32_t idesc = c == 0 ? idesc1 : idesc2;
                        const uint64_t dg_hi = dg_hi0 + (uint64_t)(((uint32_t)k2 * g_kstep) >> 4);
                        const uint64_t da_hi = da_hi0 + (uint64_t)(((uint32_t)k2 * a_kstep + (uint32_t)c * n_chunk) >> 4);
                        auto mma = [&](uint64_t a, uint64_t b, uint32_t acc) {
                            if (BF) mma_f16(d_tmem, a, b, idesc, acc); else mma_tf32(d_tmem, a, b, idesc, acc);
                        };
                        if (NSPLIT == 1) {
                            mma(dg_hi, da_hi, first);
                        } else {
                            const uint64_t dg_lo = dg_hi + (uint64_t)(GT >> 4);
                            const uint64_t da_lo = da_hi + (uint64_t)(at_bytes >> 4);
                            mma(dg_lo, da_hi, first);
                            mma(dg_hi, da_lo, 1u);
                            mma(dg_hi, da_hi, 1u);
                        }
                    }
                }
                fresh = false;
                tc_commit(&empty[si]);
                if (++run_len == FLUSH_STAGES) {
                    run_len = 0;
                    if (st + S < nst32) { tc_commit(acc_done); wait_free = true; }
                }
                if (++si == S) { si = 0; sph ^= 1u; }
            }
            if (alive) tc_commit(acc_done);
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, 512);
    if (tid == 0 && *abort_flag && p.async_err) {
        *p.async_err = 3;
        __threadfence_system();
    }
}

// bary rows padded to Fp = F rounded up to 4 floats (pad columns zero): rows start on 16-byte
// boundaries, so a stage's block is one bulk copy and a thread reads 4 bases per 16-byte load
// (thread = one 16-byte piece of a padded row)
__global__ void pad_bary_kernel(int64_t n, int F, int Fp, const float* __restrict__ src, float* __restrict__ dst) {
    const int q = Fp / 4;                                    // pieces per row
    const int64_t total = n * q;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t s;
        int d;
        if (total < (int64_t)1 << 32) { const uint32_t u = (uint32_t)i; s = u / (uint32_t)q; d = 4 * (int)(u - (uint32_t)s * (uint32_t)q); }
        else { s = i / q; d = 4 * (int)(i - s * q); }
        const float* r = src + s * F + d;
        float4 v;
        v.x = __ldg(r);                                       // d < F always: Fp - F < 4
        v.y = d + 1 < F ? __ldg(r + 1) : 0.f;
        v.z = d + 2 < F ? __ldg(r + 2) : 0.f;
        v.w = d + 3 < F ? __ldg(r + 3) : 0.f;
        reinterpret_cast<float4*>(dst)[i] = v;
    }
}

// ---------------------------------------------------------------------------- host side
struct Plan { int nsplit, bf, ncg, nchunks, nstages, nraw; int64_t stages_per_chunk; size_t smem, partial_bytes, running_bytes; };

// every channel count: `input` must come with its channels padded to a multiple of 16 (tc::pad_input),
// output channels are walked in chunks of 128; rows of gradOutput are read 16 bytes at a time
bool supported(int Cin, int Cout, int F) {
    return Cin >= 1 && Cout % 4 == 0 && Cout >= 4 && F >= 1 && F <= 32;   // F*16 <= 512 columns
}

Plan plan(int64_t Nf, int Cin, int Cout, int F, int precision) {
    Plan pl;
    const OperandMode om = operand_mode(precision);
    pl.nsplit = om.nsplit;
    pl.bf = om.bf;
    pl.ncg = (Cin + CG - 1) / CG;
    int64_t total_stages = ceil_div(Nf > 0 ? Nf : 1, KF);
    int nch = sm_count() / pl.ncg;
    if (nch < 1) nch = 1;
    if (nch > total_stages) nch = (int)total_stages;
    pl.stages_per_chunk = ceil_div(total_stages, nch);
    pl.nchunks = (int)ceil_div(total_stages, pl.stages_per_chunk);
    const size_t stage = pl.bf ? (size_t)pl.nsplit * (BG_TILE_BYTES + (KF / 8) * (size_t)at_blocks_b16(F) * BATOM_BYTES)
                               : (size_t)pl.nsplit * (G_TILE_BYTES + (KF / 4) * (size_t)at_blocks(F) * ATOM_BYTES);
    const size_t budget = 224 * 1024, fixed = 1024 + 256;
    // operand ring as deep as fits beside a raw ring of 2 (at most 4), then the raw ring as deep as fits
    int S = 4, R = 4;
    while (S > 2 && (size_t)S * stage + 2 * (size_t)RAW_BYTES + fixed > budget) --S;
    while (R > 2 && (size_t)S * stage + (size_t)R * RAW_BYTES + fixed > budget) --R;
    pl.nstages = S;
    pl.nraw = R;
    pl.smem = (size_t)S * stage + (size_t)R * RAW_BYTES + fixed;
    pl.partial_bytes = align_up((size_t)pl.nchunks * Cout * Cin * F * sizeof(float), 256);
    pl.running_bytes = (size_t)pl.ncg * pl.nchunks * (size_t)((F * CG + 31) / 32 * 32) * UM * sizeof(float);
    return pl;
}

bool fits(int64_t Nf, int Cin, int Cout, int F, int precision) {
    return plan(Nf, Cin, Cout, F, precision).smem <= 227 * 1024;
}

size_t workspace_bytes(int64_t Nf, int Cin, int Cout, int F, int precision) {
    const Plan pl = plan(Nf, Cin, Cout, F, precision);
    return align_up(pl.partial_bytes + pl.running_bytes, 256);
}

// `bary_p`: bary with rows of `Fp` floats (F rounded up to 4, pad columns zero; see tc::pad_bary);
// `input_p`: input with rows of Cin rounded up to 16 floats (pad channels zero; see tc::pad_input)
int backward_filter(int64_t Nf, int Cin, int Cout, int F, const float* gout, const float* input_p, const float* bary_p,
                    int Fp, const int32_t* cum, float* gfilter, int precision, void* ws, cudaStream_t stream) {
    int rc = check_async_error("facet2facet_backward");
    if (rc) return rc;
    Plan pl = plan(Nf, Cin, Cout, F, precision);
    Params p;
    p.Nf = Nf; p.Cin = pl.ncg * CG; p.F = F; p.Fp = Fp;
    p.CinF = Cin; p.CoutF = Cout;
    p.ncg = pl.ncg; p.nchunks = pl.nchunks; p.stages_per_chunk = pl.stages_per_chunk;
    p.nstages = pl.nstages; p.nraw = pl.nraw;
    p.gout = gout; p.in = input_p; p.cum = cum; p.partial = (float*)ws;
    p.running = (float*)((char*)ws + pl.partial_bytes);
    p.bary = bary_p;
    p.async_err = async_error_word();
    p.wait_budget = wait_budget_kclocks();
    int grid = pl.ncg * pl.nchunks;
#define PB_GF_LAUNCH(NS, BFV)                                                                                       \
    do {                                                                                                              \
        PB_CUDA(cudaFuncSetAttribute(f2f_bwd_gfilter_tc_kernel<NS, BFV>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                     (int)pl.smem));                                                                  \
        PB_LAUNCH("f2f_bwd_gfilter_tc", (f2f_bwd_gfilter_tc_kernel<NS, BFV>), grid, NTHREADS, pl.smem, stream, p);    \
    } while (0)
    for (int co0 = 0; co0 < Cout; co0 += UM) {          // every launch writes its rows of every face chunk's partial
        p.co0 = co0;
        p.Cout = Cout - co0 < UM ? Cout - co0 : UM;
        if (pl.nsplit == 2 && pl.bf) PB_GF_LAUNCH(2, true);
        else if (pl.nsplit == 2) PB_GF_LAUNCH(2, false);
        else if (pl.bf) PB_GF_LAUNCH(1, true);
        else PB_GF_LAUNCH(1, false);
    }
#undef PB_GF_LAUNCH
    return reduce_partials((const float*)ws, pl.nchunks, (int64_t)Cout * Cin * F, gfilter, stream);
}

}  // namespace gfilter

// bary rows padded to a multiple of 4 floats, shared by the two backward kernels
int padded_F(int F) { return (F + 3) / 4 * 4; }
size_t padded_bary_bytes(int64_t NiK, int F) {
    return F % 4 == 0 ? 0 : align_up((size_t)(NiK > 0 ? NiK : 1) * padded_F(F) * sizeof(float), 256);
}
int pad_bary(int64_t NiK, int F, const float* bary, float* dst, cudaStream_t stream) {
    if (NiK <= 0) return PB200_OK;
    const int Fp = padded_F(F);
    PB_LAUNCH("f2f_pad_bary", gfilter::pad_bary_kernel, persistent_blocks(NiK * (Fp / 4), 256, 8), 256, 0, stream, NiK, F, Fp,
              bary, dst);
    return PB200_OK;
}
}  // namespace tc
}  // namespace pb

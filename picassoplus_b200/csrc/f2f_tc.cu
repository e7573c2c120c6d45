// facet2facet forward on the 5th-generation tensor cores (tcgen05 + TMEM), one fused kernel:
//
//   out^T[co, f] = sum_{q=(c16,d,kk)}  W[co, q] * A[f, q],   A[f,(d,ci)] = (1/T_f) sum_k bary[k,d]*in[k,ci]
//
// Per CTA (persistent, one per SM) and per tile of 256 faces:
//   * 16 producer warps build the A operand on the fly: a thread keeps the (pre-scaled)
//     input values of its face for 8 channels in registers, walks the F bases, and writes
//     one 64-byte swizzled K-major row segment per stage straight into shared memory
//     (A is never materialised in HBM: at 128 channels x 25 bases it would be 12.8 KB/face);
//   * one thread streams the pre-swizzled filter blocks (8 KB, or hi+lo 16 KB) with 1-D bulk
//     copies of the TMA engine, completion counted on the stage's mbarrier;
//   * one thread issues tcgen05.mma (M = 128 filter rows, N = 256 faces, K = 8 per
//     instruction, tf32 operands, fp32 accumulation in TMEM) and commits stages back;
//   * the producer warps drain the 128 x 256 accumulator with tcgen05.ld and store
//     out[f, co] coalesced along co.
// Operand formats (template BF): tf32 -- a 64-byte operand row holds 16 values = one k-block
// (16 channels x 1 basis) -- or bf16 -- a row holds 32 values = two bases of the 16 channels,
// so a stage carries twice the work in the same bytes and its MMAs (kind::f16, K = 16) run at
// twice the tf32 rate.
// Precision modes: 1 split  = operands rounded to the format;
//                  2 splits = every operand as hi + lo of the format, three MMAs per k-step
//                             (hi*hi + hi*lo + lo*hi).  bf16 hi+lo keeps 16 mantissa bits per
//                             operand (products good to about 2^-16), tf32 hi+lo about 21.
// All waits are bounded (tc_ptx.cuh); on a time-out the block unwinds, frees its TMEM and
// raises the library's asynchronous error word.
#include "common.cuh"
#include <type_traits>
#include "tc_ptx.cuh"
#include "tc_runtime.cuh"

namespace pb {
namespace tc {

using namespace ptx;

constexpr int TILE_F = 256;                 // faces per tile  (UMMA N)
constexpr int UM = 128;                     // filter rows     (UMMA M), Cout zero-padded to it
constexpr int KS = 16;                      // floats per operand row per stage (64 B)
constexpr int PWARPS = 16;                  // producer / epilogue warps, 16 faces each
constexpr int NTHREADS = (PWARPS + 2) * 32; // + bulk-copy warp + MMA warp
constexpr int FACE_TILE_BYTES = TILE_F * 64;
constexpr int FILT_TILE_BYTES = UM * 64;
constexpr int TREG = 4;                     // samples per face whose inputs stay in registers
constexpr int TMEM_COLS = 256;

// ---- bf16 filter image: Wimg[kb][split][co 0..127][32 bf16, 64B-swizzled], kb = c16*ceil(F/2) + dp,
//      element (co, j*16 + kk) = filter[co][c16*16 + kk][2*dp + j]  (0 for a basis >= F)
//      Cin = channels padded to 16 (CinF = channels of the filter; padded ones are 0); the image holds
//      output channels co0 .. co0 + Cout - 1 of the filter.
__global__ void f2f_tc_prep_filter_bf16_kernel(int F, int Cin, int CinF, int co0, int Cout, int nsplit,
                                               const float* __restrict__ filter, uint8_t* __restrict__ wimg) {
    const int nd2 = (F + 1) / 2;
    const int nkb = (Cin / 16) * nd2;
    int64_t total = (int64_t)nkb * 128 * 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i & 3);                   // 16-byte chunk: basis j = c >> 1, channels 8*(c&1)..+7
        const int co = (int)((i >> 2) % 128);
        const int kb = (int)(i / (4 * 128));
        const int c16 = kb / nd2, d = 2 * (kb - c16 * nd2) + (c >> 1);
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int ci = c16 * 16 + (c & 1) * 8 + 2 * j + e;
                v[e] = (co < Cout && d < F && ci < CinF) ? __ldg(filter + ((int64_t)(co0 + co) * CinF + ci) * F + d) : 0.f;
            }
            if (nsplit == 1) { hi[j] = pack_bf16x2(v[0], v[1]); lo[j] = 0u; }
            else split_bf16x2(v[0], v[1], hi[j], lo[j]);
        }
        uint8_t* base = wimg + (int64_t)kb * nsplit * (128 * 64);
        const uint32_t off = swz64_offset((uint32_t)co, (uint32_t)c);
        *reinterpret_cast<uint4*>(base + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        if (nsplit == 2) *reinterpret_cast<uint4*>(base + 128 * 64 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// ---- filter image: Wimg[kb][split][co 0..127][16 floats, 64B-swizzled], kb = c16*F + d,
//      element (co, kk) = filter[co][c16*16 + kk][d]
__global__ void f2f_tc_prep_filter_kernel(int F, int Cin, int CinF, int co0, int Cout, int nsplit,
                                          const float* __restrict__ filter, uint8_t* __restrict__ wimg) {
    const int nkb = (Cin / KS) * F;
    int64_t total = (int64_t)nkb * UM * 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int c = (int)(i & 3);
        int co = (int)((i >> 2) % UM);
        int kb = (int)(i / (4 * UM));
        int c16 = kb / F, d = kb - c16 * F;
        float v[4], hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ci = c16 * KS + c * 4 + j;
            v[j] = (co < Cout && ci < CinF) ? __ldg(filter + ((int64_t)(co0 + co) * CinF + ci) * F + d) : 0.f;
            if (nsplit == 1) { hi[j] = to_tf32_rna(v[j]); lo[j] = 0.f; }
            else { hi[j] = tf32_hi(v[j]); lo[j] = v[j] - hi[j]; }
        }
        uint8_t* base = wimg + (int64_t)kb * nsplit * FILT_TILE_BYTES;
        uint32_t off = swz64_offset((uint32_t)co, (uint32_t)c);
        *reinterpret_cast<float4*>(base + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        if (nsplit == 2)
            *reinterpret_cast<float4*>(base + FILT_TILE_BYTES + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
}

struct FwdParams {
    int64_t Nf;
    int Cin, Cout, F;
    int nstages;          // pipeline depth
    int smaxw;            // bary rows staged per producer warp
    int bpitch;           // floats per staged bary row: multiple of 4 and = 4 (mod 8) -> aligned, conflict-free
    const float* in;
    const float* bary;
    const int32_t* cum;
    const uint8_t* wimg;
    float* out;           // first output channel of this launch's chunk
    int out_stride;       // floats per output row (all output channels of the operator)
    int* async_err;
    int wait_budget;      // bounded waits give up after this many units of 1024 clocks
    int silent_filter;    // test switch: the filter stream issues nothing, so every wait runs out
};

__host__ __device__ inline size_t fwd_stage_bytes(int nsplit) {
    return (size_t)nsplit * (FACE_TILE_BYTES + FILT_TILE_BYTES);
}

template <int NSPLIT, bool BF>
__global__ void __launch_bounds__(NTHREADS, 1) f2f_fwd_tc_kernel(FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.nstages;
    const int F = p.F, Cin = p.Cin, Cout = p.Cout;
    const int FP = p.bpitch;
    const size_t stage_bytes = fwd_stage_bytes(NSPLIT);
    // stage layout: [face hi][face lo?][filter hi][filter lo?]
    uint8_t* stages = smem;
    float* bary_s = reinterpret_cast<float*>(smem + (size_t)S * stage_bytes);
    uint8_t* tail = reinterpret_cast<uint8_t*>(bary_s + (size_t)PWARPS * p.smaxw * FP);
    uint64_t* bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(tail) + 15) & ~(uintptr_t)15);
    uint64_t* full = bars;                 // [S]  producers (16 warps) + filter bytes
    uint64_t* empty = bars + S;            // [S]  MMA done with the stage
    uint64_t* acc_full = bars + 2 * S;     // [1]  accumulator of the tile complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], PWARPS + 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        abort_flag[0] = 0;
        abort_flag[1] = p.wait_budget;
        fence_barrier_init();
    }
    if (warp == PWARPS) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t ntiles = (p.Nf + TILE_F - 1) / TILE_F;
    const int nkb = (Cin / KS) * (BF ? (F + 1) / 2 : F);     // stages per tile

    if (warp < PWARPS) {
        // ================================ producers + epilogue ================================
        const int ml = lane >> 1, h = lane & 1;               // face within the warp's 16, 8-channel half
        const int m = warp * 16 + ml;                         // row of the face operand tile
        float* wb = bary_s + (size_t)warp * p.smaxw * FP;     // this warp's staged bary rows
        for (int i = lane; i < p.smaxw * FP; i += 32) wb[i] = 0.f;
        const uint32_t off0 = swz64_offset((uint32_t)m, (uint32_t)(2 * h));
        const uint32_t off1 = swz64_offset((uint32_t)m, (uint32_t)(2 * h + 1));
        // bf16 rows: chunk 2*j + h holds the thread's 8 channels of basis j of the stage's pair
        const uint32_t offb0 = swz64_offset((uint32_t)m, (uint32_t)h), offb1 = swz64_offset((uint32_t)m, (uint32_t)(2 + h));
        const uint32_t stages32 = smem_u32(stages), wb32 = smem_u32(wb);
        int st_i = 0;                                         // running stage index and phase
        uint32_t st_ph = 0;
        uint32_t tcount = 0;
        bool alive = true;

        // publish one operand row segment (a0, a1 = 8 channels of A[f, d, :]) into the current stage;
        // a bf16 stage takes two bases (d even, then d odd; an odd F ends with a zero partner)
        auto publish = [&](const float4& a0, const float4& a1, int d) -> bool {
            if (!BF || (d & 1) == 0) {
                if (!mbar_try_wait(&empty[st_i], st_ph ^ 1u)) {
                    int ok = 1;
                    if (lane == 0) ok = mbar_wait(&empty[st_i], st_ph ^ 1u, abort_flag) ? 1 : 0;
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) return false;
                }
            }
            const uint32_t st = stages32 + (uint32_t)st_i * (uint32_t)stage_bytes;
            if (BF) {
                uint32_t hi[4], lo[4];
                if (NSPLIT == 1) {
                    hi[0] = pack_bf16x2(a0.x, a0.y); hi[1] = pack_bf16x2(a0.z, a0.w);
                    hi[2] = pack_bf16x2(a1.x, a1.y); hi[3] = pack_bf16x2(a1.z, a1.w);
                } else {
                    split_bf16x2(a0.x, a0.y, hi[0], lo[0]); split_bf16x2(a0.z, a0.w, hi[1], lo[1]);
                    split_bf16x2(a1.x, a1.y, hi[2], lo[2]); split_bf16x2(a1.z, a1.w, hi[3], lo[3]);
                }
                const uint32_t ob = (d & 1) ? offb1 : offb0;
                sts_f4(st + ob, make_float4(__uint_as_float(hi[0]), __uint_as_float(hi[1]), __uint_as_float(hi[2]), __uint_as_float(hi[3])));
                if (NSPLIT == 2)
                    sts_f4(st + FACE_TILE_BYTES + ob, make_float4(__uint_as_float(lo[0]), __uint_as_float(lo[1]), __uint_as_float(lo[2]), __uint_as_float(lo[3])));
                if ((d & 1) == 0) {
                    if (d + 1 < F) return true;                // the stage is complete with the next basis
                    sts_f4(st + offb1, zero4());
                    if (NSPLIT == 2) sts_f4(st + FACE_TILE_BYTES + offb1, zero4());
                }
            } else if (NSPLIT == 1) {
                sts_f4(st + off0, make_float4(to_tf32_rna(a0.x), to_tf32_rna(a0.y), to_tf32_rna(a0.z), to_tf32_rna(a0.w)));
                sts_f4(st + off1, make_float4(to_tf32_rna(a1.x), to_tf32_rna(a1.y), to_tf32_rna(a1.z), to_tf32_rna(a1.w)));
            } else {
                const float4 h0 = make_float4(tf32_hi(a0.x), tf32_hi(a0.y), tf32_hi(a0.z), tf32_hi(a0.w));
                const float4 h1 = make_float4(tf32_hi(a1.x), tf32_hi(a1.y), tf32_hi(a1.z), tf32_hi(a1.w));
                sts_f4(st + off0, h0);
                sts_f4(st + off1, h1);
                sts_f4(st + FACE_TILE_BYTES + off0, make_float4(a0.x - h0.x, a0.y - h0.y, a0.z - h0.z, a0.w - h0.w));
                sts_f4(st + FACE_TILE_BYTES + off1, make_float4(a1.x - h1.x, a1.y - h1.y, a1.z - h1.z, a1.w - h1.w));
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[st_i]);
            if (++st_i == S) { st_i = 0; st_ph ^= 1u; }
            return true;
        };

        for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++tcount) {
            const int64_t f0 = tile * TILE_F;
            const int64_t fw0 = f0 + warp * 16;               // first face of this warp
            const int64_t f = fw0 + ml;
            const bool valid = f < p.Nf;
            int k0 = 0, k1 = 0;
            if (valid) { k0 = f > 0 ? __ldg(p.cum + f - 1) : 0; k1 = __ldg(p.cum + f); }
            const int T = k1 - k0;
            // sample range of the warp's faces, staged (as far as it fits) in the warp's region
            int kw0 = 0, kw1 = 0;
            if (fw0 < p.Nf) {
                int64_t fl = fw0 + 16 < p.Nf ? fw0 + 16 : p.Nf;
                kw0 = fw0 > 0 ? __ldg(p.cum + fw0 - 1) : 0;
                kw1 = __ldg(p.cum + fl - 1);
            }
            int nS = kw1 - kw0;
            if (nS > p.smaxw) nS = p.smaxw;
            // a warp whose faces all have <= TREG samples and fit the staged rows takes the lean path
            const bool slow = __any_sync(0xffffffffu, (T > TREG) || (kw1 - kw0 > p.smaxw));
            __syncwarp();
            {
                const float* src = p.bary + (int64_t)kw0 * F;
                for (int i = lane; i < nS * F; i += 32) {
                    int sr = i / F;
                    wb[sr * FP + (i - sr * F)] = __ldg(src + i);
                }
            }
            __syncwarp();
            const float invT = T > 0 ? 1.f / (float)T : 0.f;
            const int kloc = valid ? k0 - kw0 : 0;            // row of the face's first sample in wb
            // the lean path for TR sample slots per face (TR = 1 when no face of the warp has a second sample:
            // one product per operand element instead of TREG multiply-adds)
            auto lean = [&](auto trc) {
                constexpr int TR = decltype(trc)::value;
                // rows of the face's samples; unused slots point at a valid row and meet x == 0
                uint32_t bp[TR];
#pragma unroll
                for (int t = 0; t < TR; ++t) {
                    int row = kloc + (t < T ? t : (T > 0 ? T - 1 : 0));
                    if (row >= p.smaxw) row = 0;
                    bp[t] = wb32 + (uint32_t)(row * FP) * 4u;
                }
                for (int c16 = 0; c16 < Cin / KS && alive; ++c16) {
                    float4 x[TR][2];
#pragma unroll
                    for (int t = 0; t < TR; ++t) {
                        if (t < T) {
                            const float4* src =
                                reinterpret_cast<const float4*>(p.in + (int64_t)(k0 + t) * Cin + c16 * KS + h * 8);
                            x[t][0] = scale4(ldg4(src), invT);
                            x[t][1] = scale4(ldg4(src + 1), invT);
                        } else {
                            x[t][0] = zero4(); x[t][1] = zero4();
                        }
                    }
                    for (int d4 = 0; d4 < F && alive; d4 += 4) {
                        float4 b[TR];
#pragma unroll
                        for (int t = 0; t < TR; ++t) b[t] = lds_f4(bp[t] + (uint32_t)d4 * 4u);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (d4 + j < F) {
                                // packed f32x2 FMAs: half the instructions of the scalar form
                                float2 s0 = make_float2(0.f, 0.f), s1 = s0, s2 = s0, s3 = s0;
#pragma unroll
                                for (int t = 0; t < TR; ++t) {
                                    const float bj = j == 0 ? b[t].x : (j == 1 ? b[t].y : (j == 2 ? b[t].z : b[t].w));
                                    const float2 b2 = make_float2(bj, bj);
                                    if (TR == 1) {
                                        s0 = __fmul2_rn(b2, make_float2(x[t][0].x, x[t][0].y));
                                        s1 = __fmul2_rn(b2, make_float2(x[t][0].z, x[t][0].w));
                                        s2 = __fmul2_rn(b2, make_float2(x[t][1].x, x[t][1].y));
                                        s3 = __fmul2_rn(b2, make_float2(x[t][1].z, x[t][1].w));
                                    } else {
                                        s0 = __ffma2_rn(b2, make_float2(x[t][0].x, x[t][0].y), s0);
                                        s1 = __ffma2_rn(b2, make_float2(x[t][0].z, x[t][0].w), s1);
                                        s2 = __ffma2_rn(b2, make_float2(x[t][1].x, x[t][1].y), s2);
                                        s3 = __ffma2_rn(b2, make_float2(x[t][1].z, x[t][1].w), s3);
                                    }
                                }
                                const float4 a0 = make_float4(s0.x, s0.y, s1.x, s1.y), a1 = make_float4(s2.x, s2.y, s3.x, s3.y);
                                if (!publish(a0, a1, d4 + j)) { alive = false; break; }
                            }
                        }
                    }
                }
            };
            if (!slow) {
                if (__any_sync(0xffffffffu, T > 1)) lean(std::integral_constant<int, TREG>{});
                else lean(std::integral_constant<int, 1>{});
            } else {
                for (int c16 = 0; c16 < Cin / KS && alive; ++c16) {
                    for (int d = 0; d < F; ++d) {
                        float4 a0 = zero4(), a1 = zero4();
                        for (int t = 0; t < T; ++t) {
                            int row = kloc + t;
                            float b = (row < p.smaxw ? wb[row * FP + d] : __ldg(p.bary + (int64_t)(k0 + t) * F + d)) * invT;
                            const float4* src =
                                reinterpret_cast<const float4*>(p.in + (int64_t)(k0 + t) * Cin + c16 * KS + h * 8);
                            fma4s(a0, b, ldg4(src));
                            fma4s(a1, b, ldg4(src + 1));
                        }
                        if (!publish(a0, a1, d)) { alive = false; break; }
                    }
                }
            }
            if (!alive) break;
            // ---- epilogue: drain the accumulator (rows = co, columns = faces of the tile)
            int ok = 1;
            if (lane == 0) ok = mbar_wait(acc_full, tcount & 1u, abort_flag) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { alive = false; break; }
            tc_fence_after();
            const int q = warp & 3, g = warp >> 2;
            const int co = q * 32 + lane;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                const int col = g * 64 + half * 32;
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)col, r);
                tmem_ld_wait();
                if (co < Cout) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        int64_t fo = f0 + col + j;
                        if (fo < p.Nf) __stcs(p.out + fo * p.out_stride + co, __uint_as_float(r[j]));
                    }
                }
            }
            tc_fence_before();
        }
    } else if (warp == PWARPS) {
        // ================================ filter loader (TMA engine) ==========================
        if (lane == 0) {
            const uint32_t bytes = (uint32_t)(NSPLIT * FILT_TILE_BYTES);
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { alive = false; break; }
                    if (p.silent_filter) continue;          // test switch: `full` never completes
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_g2s(stages + (size_t)s * stage_bytes + (size_t)NSPLIT * FACE_TILE_BYTES,
                             p.wimg + (size_t)kb * bytes, bytes, &full[s]);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
            if (!alive) {                       // let copies in flight land before shared memory is released
                long long t0 = clock64();
                while (clock64() - t0 < 2000000) { }
            }
        }
    } else {
        // ================================ MMA issuer =========================================
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BF ? FMT_BF16 : FMT_TF32, UM, TILE_F);
            const uint64_t dbase = smem_desc_kmajor(smem_u32(stages), 64, SWZ_64B);
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!mbar_wait(&full[s], ph, abort_flag)) { alive = false; break; }
                    tc_fence_after();
                    // descriptors differ only in the 16-byte-unit start address: add offsets to one base
                    const uint64_t face_hi = dbase + (uint64_t)(((uint32_t)s * (uint32_t)stage_bytes) >> 4);
                    const uint64_t filt_hi = face_hi + (uint64_t)((NSPLIT * FACE_TILE_BYTES) >> 4);
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) {          // 2 x 32 bytes of K (8 tf32 or 16 bf16)
                        const uint64_t adv = (uint64_t)(ks * 2);
                        const uint32_t first = (kb | ks) != 0;
                        auto mma = [&](uint64_t a, uint64_t b, uint32_t acc) {
                            if (BF) mma_f16(tmem_base, a, b, idesc, acc); else mma_tf32(tmem_base, a, b, idesc, acc);
                        };
                        if (NSPLIT == 1) {
                            mma(filt_hi + adv, face_hi + adv, first);
                        } else {
                            const uint64_t face_lo = face_hi + (uint64_t)(FACE_TILE_BYTES >> 4);
                            const uint64_t filt_lo = filt_hi + (uint64_t)(FILT_TILE_BYTES >> 4);
                            mma(filt_lo + adv, face_hi + adv, first);
                            mma(filt_hi + adv, face_lo + adv, 1u);
                            mma(filt_hi + adv, face_hi + adv, 1u);
                        }
                    }
                    tc_commit(&empty[s]);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (alive) tc_commit(acc_full);
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == PWARPS) tmem_dealloc(tmem_base, TMEM_COLS);
    if (tid == 0 && *abort_flag && p.async_err) {
        *p.async_err = 1;
        __threadfence_system();
    }
}

// rows of C floats -> rows of Cp >= C floats, pad columns zero (thread = one float of the padded row)
__global__ void pad_rows_kernel(int64_t n, int C, int Cp, const float* __restrict__ src, float* __restrict__ dst) {
    const int64_t total = n * Cp;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / Cp;
        const int c = (int)(i - r * Cp);
        dst[i] = c < C ? __ldg(src + r * C + c) : 0.f;
    }
}

int padded_channels(int Cin) { return (Cin + KS - 1) / KS * KS; }
size_t padded_input_bytes(int64_t NiK, int Cin) {
    return Cin % KS == 0 ? 0 : align_up((size_t)(NiK > 0 ? NiK : 1) * padded_channels(Cin) * sizeof(float), 256);
}
int pad_input(int64_t NiK, int Cin, const float* input, float* dst, cudaStream_t stream) {
    if (NiK <= 0) return PB200_OK;
    const int Cp = padded_channels(Cin);
    PB_LAUNCH("f2f_pad_input", pad_rows_kernel, persistent_blocks(NiK * Cp, 256, 8), 256, 0, stream, NiK, Cin, Cp, input, dst);
    return PB200_OK;
}

// ---------------------------------------------------------------------------- host side
struct FwdPlan { int nsplit, bf, nkb, nstages, smaxw, bpitch; size_t smem; size_t wimg_bytes; };

// every channel count: input channels are zero-padded to a multiple of 16 (a copy in the workspace),
// output channels are walked in chunks of 128 (one launch each over the same input)
bool fwd_supported(int Cin, int Cout, int F) { return Cin >= 1 && Cout >= 1 && F >= 1 && F <= 50; }

FwdPlan fwd_plan(int Cin, int Cout, int F, int precision) {
    FwdPlan pl;
    const OperandMode om = operand_mode(precision);
    pl.nsplit = om.nsplit;
    pl.bf = om.bf;
    pl.nkb = (Cin / KS) * (pl.bf ? (F + 1) / 2 : F);
    pl.nstages = pl.nsplit == 2 ? 2 : 4;
    const int FP = ((F + 3) / 4 * 4) | 4;
    pl.bpitch = FP;
    const size_t budget = 220 * 1024;
    size_t fixed = (size_t)pl.nstages * fwd_stage_bytes(pl.nsplit) + 1024 /*alignment*/ + 256 /*barriers*/;
    int smaxw = (int)((budget - fixed) / ((size_t)PWARPS * FP * 4));
    if (smaxw > 64) smaxw = 64;             // 16 faces x 4 samples
    if (smaxw < 0) smaxw = 0;
    pl.smaxw = smaxw;
    pl.smem = fixed + (size_t)PWARPS * smaxw * FP * 4;
    pl.wimg_bytes = (size_t)pl.nkb * pl.nsplit * FILT_TILE_BYTES;
    return pl;
}

size_t fwd_workspace_bytes(int64_t NiK, int Cin, int Cout, int F, int precision) {
    return align_up(fwd_plan(padded_channels(Cin), Cout, F, precision).wimg_bytes, 256) + padded_input_bytes(NiK, Cin);
}

int forward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* input, const float* filter,
            const float* bary, const int32_t* cum, float* output, int precision, void* ws, cudaStream_t stream) {
    int rc = check_async_error("facet2facet_forward");
    if (rc) return rc;
    const int CinP = padded_channels(Cin);
    FwdPlan pl = fwd_plan(CinP, Cout, F, precision);
    uint8_t* wimg = (uint8_t*)ws;
    if (CinP != Cin) {
        float* xp = (float*)((char*)ws + align_up(pl.wimg_bytes, 256));
        rc = pad_input(NiK, Cin, input, xp, stream);
        if (rc) return rc;
        input = xp;
    }
    const int64_t prep_items = (int64_t)pl.nkb * UM * 4;
    const int64_t ntiles = ceil_div(Nf, TILE_F);
    const int grid = (int)(ntiles < sm_count() ? ntiles : sm_count());
    for (int co0 = 0; co0 < Cout; co0 += UM) {
        const int cchunk = Cout - co0 < UM ? Cout - co0 : UM;
        if (pl.bf) {
            PB_LAUNCH("f2f_tc_prep_filter", f2f_tc_prep_filter_bf16_kernel, persistent_blocks(prep_items, 256, 8), 256, 0,
                      stream, F, CinP, Cin, co0, cchunk, pl.nsplit, filter, wimg);
        } else {
            PB_LAUNCH("f2f_tc_prep_filter", f2f_tc_prep_filter_kernel, persistent_blocks(prep_items, 256, 8), 256, 0, stream,
                      F, CinP, Cin, co0, cchunk, pl.nsplit, filter, wimg);
        }
        FwdParams p;
        p.Nf = Nf; p.Cin = CinP; p.Cout = cchunk; p.F = F;
        p.nstages = pl.nstages; p.smaxw = pl.smaxw; p.bpitch = pl.bpitch;
        p.in = input; p.bary = bary; p.cum = cum; p.wimg = wimg; p.out = output + co0; p.out_stride = Cout;
        p.async_err = async_error_word();
        p.wait_budget = wait_budget_kclocks();
        p.silent_filter = test_skip_filter_stream();
#define PB_FWD_LAUNCH(NS, BFV)                                                                                      \
    do {                                                                                                              \
        PB_CUDA(cudaFuncSetAttribute(f2f_fwd_tc_kernel<NS, BFV>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                     (int)pl.smem));                                                                  \
        PB_LAUNCH("f2f_fwd_tc", (f2f_fwd_tc_kernel<NS, BFV>), grid, NTHREADS, pl.smem, stream, p);                    \
    } while (0)
        if (pl.nsplit == 2 && pl.bf) PB_FWD_LAUNCH(2, true);
        else if (pl.nsplit == 2) PB_FWD_LAUNCH(2, false);
        else if (pl.bf) PB_FWD_LAUNCH(1, true);
        else PB_FWD_LAUNCH(1, false);
#undef PB_FWD_LAUNCH
    }
    return PB200_OK;
}

}  // namespace tc
}  // namespace pb

// Module-level fusion of the two HBM-bound mesh operators with the pointwise stage that follows
// them in the layer modules (picasso/mesh/layers.py:109-120 V2FConv3d.forward, :166-175
// F2VConv3d.forward: operator -> matmul(depth_weights) -> + bias -> ReLU):
//
//   out^T[co, row] = act( sum_c  Wd[c, co] * feat[row, c]  + bias[co] )
//
// where feat[row, :] is never written to HBM.  The rows of `feat` are produced on the fly:
//   vertex2facet:  feat[f, c] = sum_{k<3} filter[k, c] * input[face[f, k], c]        (r = 1)
//   facet2vertex:  feat[v, c] = (sum over the CSR entries (f, corner) of v of wx[f, c]) / nfCount[v]
//                  (wx = the per-face products of the facet2vertex forward pass)
// Per CTA (persistent) and per tile of 256 rows, the same roles as the facet2facet forward kernel:
// 16 producer warps gather and combine the operand rows (thread = row x 8 channels) and write them
// as 64-byte swizzled K-major bf16 rows (one stage = 32 channels); one thread streams the
// pre-swizzled weight blocks with 1-D bulk copies; one thread issues tcgen05.mma (M = 128 output
// channels, N = 256 rows, K = 16 per instruction, fp32 accumulation in TMEM); the producer warps
// drain the accumulator, add the bias, apply the activation and store out[row, co] coalesced.
// Precision modes: bf16 operands (one product per term) or bf16 hi + lo operands (three products,
// about 1e-5 relative: the fp32 mode).  All waits are bounded (tc_ptx.cuh).
#include "common.cuh"
#include "tc_ptx.cuh"
#include "tc_runtime.cuh"

namespace pb {

// per-face products of the facet2vertex forward pass (f2v.cu): wx[f, :] = (coeff[f] @ filter) * input[f]
int f2v_face_products(int64_t Nf, int C, int K, const float* input, const float* filter, const float* coeff, float* wx,
                      cudaStream_t stream);
bool f2v_face_products_supported(int C, int K);

namespace pw {

using namespace ptx;

constexpr int TILE_R = 256;                 // rows per tile (UMMA N)
constexpr int UM = 128;                     // output channels per launch (UMMA M), zero-padded
constexpr int PWARPS = 16;
constexpr int NTHREADS = (PWARPS + 2) * 32;
constexpr int ROW_TILE_BYTES = TILE_R * 64;
constexpr int W_TILE_BYTES = UM * 64;
constexpr int KB = 32;                      // channels per stage (one 64-byte bf16 operand row)

// weight image: Wimg[kb][split][co 0..127][32 bf16, 64B-swizzled], element (co, k) = Wd[kb*32 + k][co0 + co]
__global__ void pw_prep_weights_kernel(int Cmid, int Cout, int co0, int cchunk, int nkb, int nsplit,
                                       const float* __restrict__ wd, uint8_t* __restrict__ wimg) {
    const int64_t total = (int64_t)nkb * UM * 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i & 3);                   // 16-byte chunk = 8 channels
        const int co = (int)((i >> 2) % UM);
        const int kb = (int)(i / (4 * UM));
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int ci = kb * KB + c * 8 + 2 * j + e;
                v[e] = (co < cchunk && ci < Cmid) ? __ldg(wd + (int64_t)ci * Cout + co0 + co) : 0.f;
            }
            if (nsplit == 1) { hi[j] = pack_bf16x2(v[0], v[1]); lo[j] = 0u; }
            else split_bf16x2(v[0], v[1], hi[j], lo[j]);
        }
        uint8_t* base = wimg + (int64_t)kb * nsplit * W_TILE_BYTES;
        const uint32_t off = swz64_offset((uint32_t)co, (uint32_t)c);
        *reinterpret_cast<uint4*>(base + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        if (nsplit == 2) *reinterpret_cast<uint4*>(base + W_TILE_BYTES + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

struct Params {
    int64_t Nrows;            // faces (vertex2facet) or output vertices (facet2vertex)
    int C;                    // channels of the gathered rows (a multiple of 8)
    int Cout;                 // output channels of this launch's chunk (<= 128)
    int out_stride;           // floats per output row
    int nkb;                  // 32-channel stages per tile
    int nstages;
    int relu;
    // vertex2facet rows
    const float* vin;         // (Nv, C)
    const float* vfilt;       // (3, C)
    const int32_t* face;      // (Nrows, 3)
    int64_t Nv;
    // facet2vertex rows
    const float* wx;          // (Nf, C) per-face products
    const int32_t* rowptr;
    const int32_t* entries;
    const int32_t* nfCount;
    // masked rows (backward of the pointwise stage)
    const float* rows;        // (Nrows, C) upstream gradient
    const float* mask;        // (Nrows, C) activated output: the gradient passes where it is > 0; NULL = no mask
    float* masked_out;        // (Nrows, C) the masked gradient, written as a by-product; NULL = not wanted
    const uint8_t* wimg;
    const float* bias;        // (Cout chunk) or NULL
    float* out;               // first output channel of the chunk
    int* async_err;
    int wait_budget;
};

__host__ __device__ inline size_t stage_bytes(int nsplit) { return (size_t)nsplit * (ROW_TILE_BYTES + W_TILE_BYTES); }

// MODE 0: vertex2facet rows, MODE 1: facet2vertex rows, MODE 2: rows of a gradient masked by an activation
template <int NSPLIT, int MODE>
__global__ void __launch_bounds__(NTHREADS, 1) rows_pointwise_tc_kernel(Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.nstages, C = p.C, Cout = p.Cout;
    const size_t sbytes = stage_bytes(NSPLIT);
    uint8_t* stages = smem;                       // stage: [rows hi][rows lo?][weights hi][weights lo?]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)S * sbytes);
    uint64_t* full = bars;                        // [S] producers (16 warps) + weight bytes
    uint64_t* empty = bars + S;                   // [S] MMA done with the stage
    uint64_t* acc_full = bars + 2 * S;            // accumulator of the tile complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (tid == 0) {
        for (int s = 0; s < S; ++s) { mbar_init(&full[s], PWARPS + 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        abort_flag[0] = 0;
        abort_flag[1] = p.wait_budget;
        fence_barrier_init();
    }
    if (warp == PWARPS) { tmem_alloc(tmem_slot, TILE_R); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int64_t ntiles = (p.Nrows + TILE_R - 1) / TILE_R;

    if (warp < PWARPS) {
        // ================================ producers + epilogue ================================
        const int ml = lane >> 1, h = lane & 1;               // row within the warp's 16, 8-channel half
        const int m = warp * 16 + ml;
        const uint32_t offb0 = swz64_offset((uint32_t)m, (uint32_t)h), offb1 = swz64_offset((uint32_t)m, (uint32_t)(2 + h));
        const uint32_t stages32 = smem_u32(stages);
        int st_i = 0;
        uint32_t st_ph = 0, tcount = 0;
        bool alive = true;

        // 8 channels of 16-channel block `b16` of the row into the current stage (two blocks per stage)
        auto publish = [&](const float4& a0, const float4& a1, int b16) -> bool {
            if ((b16 & 1) == 0) {
                if (!mbar_try_wait(&empty[st_i], st_ph ^ 1u)) {
                    int ok = 1;
                    if (lane == 0) ok = mbar_wait(&empty[st_i], st_ph ^ 1u, abort_flag) ? 1 : 0;
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) return false;
                }
            }
            const uint32_t st = stages32 + (uint32_t)st_i * (uint32_t)sbytes;
            uint32_t hi[4], lo[4];
            if (NSPLIT == 1) {
                hi[0] = pack_bf16x2(a0.x, a0.y); hi[1] = pack_bf16x2(a0.z, a0.w);
                hi[2] = pack_bf16x2(a1.x, a1.y); hi[3] = pack_bf16x2(a1.z, a1.w);
            } else {
                split_bf16x2(a0.x, a0.y, hi[0], lo[0]); split_bf16x2(a0.z, a0.w, hi[1], lo[1]);
                split_bf16x2(a1.x, a1.y, hi[2], lo[2]); split_bf16x2(a1.z, a1.w, hi[3], lo[3]);
            }
            const uint32_t ob = (b16 & 1) ? offb1 : offb0;
            sts_f4(st + ob, make_float4(__uint_as_float(hi[0]), __uint_as_float(hi[1]), __uint_as_float(hi[2]), __uint_as_float(hi[3])));
            if (NSPLIT == 2)
                sts_f4(st + ROW_TILE_BYTES + ob, make_float4(__uint_as_float(lo[0]), __uint_as_float(lo[1]), __uint_as_float(lo[2]), __uint_as_float(lo[3])));
            if ((b16 & 1) == 0) return true;                  // the stage is complete with the odd block
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[st_i]);
            if (++st_i == S) { st_i = 0; st_ph ^= 1u; }
            return true;
        };

        for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x, ++tcount) {
            const int64_t r0 = tile * TILE_R;
            const int64_t row = r0 + m;
            const bool valid = row < p.Nrows;
            int v0 = -1, v1 = -1, v2 = -1, beg = 0, end = 0;
            float inv_n = 0.f;
            if (MODE == 0) {
                if (valid) {
                    v0 = __ldg(p.face + 3 * row); v1 = __ldg(p.face + 3 * row + 1); v2 = __ldg(p.face + 3 * row + 2);
                    if (v0 < 0 || v0 >= p.Nv) v0 = -1;            // a bad index contributes nothing
                    if (v1 < 0 || v1 >= p.Nv) v1 = -1;
                    if (v2 < 0 || v2 >= p.Nv) v2 = -1;
                }
            } else if (valid) {
                beg = __ldg(p.rowptr + row); end = __ldg(p.rowptr + row + 1);
                if (end > beg) inv_n = 1.f / (float)__ldg(p.nfCount + row);
            }
            for (int b16 = 0; b16 < 2 * p.nkb && alive; ++b16) {
                const int c = b16 * 16 + h * 8;
                float4 a0 = zero4(), a1 = zero4();
                if (c < C) {
                    if (MODE == 0) {
                        // the k-ascending FMA chain of the stand-alone vertex2facet kernel
                        const int vs[3] = {v0, v1, v2};
#pragma unroll
                        for (int k = 0; k < 3; ++k) {
                            if (vs[k] >= 0) {
                                const float4* x = reinterpret_cast<const float4*>(p.vin + (int64_t)vs[k] * C + c);
                                const float4* f = reinterpret_cast<const float4*>(p.vfilt + (int64_t)k * C + c);
                                fma4(a0, ldg4(f), ldg4(x));
                                fma4(a1, ldg4(f + 1), ldg4(x + 1));
                            }
                        }
                    } else if (MODE == 2) {
                        if (valid) {
                            const float4* x = reinterpret_cast<const float4*>(p.rows + row * C + c);
                            a0 = ldg4(x); a1 = ldg4(x + 1);
                            if (p.mask) {
                                const float4* mk = reinterpret_cast<const float4*>(p.mask + row * C + c);
                                const float4 m0 = ldg4(mk), m1 = ldg4(mk + 1);
                                a0 = make_float4(m0.x > 0.f ? a0.x : 0.f, m0.y > 0.f ? a0.y : 0.f, m0.z > 0.f ? a0.z : 0.f,
                                                 m0.w > 0.f ? a0.w : 0.f);
                                a1 = make_float4(m1.x > 0.f ? a1.x : 0.f, m1.y > 0.f ? a1.y : 0.f, m1.z > 0.f ? a1.z : 0.f,
                                                 m1.w > 0.f ? a1.w : 0.f);
                            }
                            if (p.masked_out) {
                                float4* mo = reinterpret_cast<float4*>(p.masked_out + row * C + c);
                                mo[0] = a0; mo[1] = a1;
                            }
                        }
                    } else {
                        // ascending CSR entries, then one scaling: the arithmetic of the stand-alone gather kernel
                        for (int e = beg; e < end; ++e) {
                            const int64_t f = __ldg(p.entries + e) >> 2;
                            const float4* x = reinterpret_cast<const float4*>(p.wx + f * C + c);
                            add4(a0, ldg4(x));
                            add4(a1, ldg4(x + 1));
                        }
                        if (end > beg) { a0 = scale4(a0, inv_n); a1 = scale4(a1, inv_n); }
                    }
                }
                if (!publish(a0, a1, b16)) { alive = false; break; }
            }
            if (!alive) break;
            // ---- epilogue: accumulator rows = output channels, columns = rows of the tile
            int ok = 1;
            if (lane == 0) ok = mbar_wait(acc_full, tcount & 1u, abort_flag) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { alive = false; break; }
            tc_fence_after();
            const int q = warp & 3, g = warp >> 2;
            const int co = q * 32 + lane;
            const float bv = (p.bias && co < Cout) ? __ldg(p.bias + co) : 0.f;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                const int col = g * 64 + half * 32;
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)col, r);
                tmem_ld_wait();
                if (co < Cout) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int64_t ro = r0 + col + j;
                        float v = __uint_as_float(r[j]) + bv;
                        if (p.relu) v = fmaxf(v, 0.f);
                        if (ro < p.Nrows) __stcs(p.out + ro * p.out_stride + co, v);
                    }
                }
            }
            tc_fence_before();
        }
    } else if (warp == PWARPS) {
        // ================================ weight loader (TMA engine) ==========================
        if (lane == 0) {
            const uint32_t bytes = (uint32_t)(NSPLIT * W_TILE_BYTES);
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
                for (int kb = 0; kb < p.nkb; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { alive = false; break; }
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_g2s(stages + (size_t)s * sbytes + (size_t)NSPLIT * ROW_TILE_BYTES, p.wimg + (size_t)kb * bytes, bytes,
                             &full[s]);
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
            constexpr uint32_t idesc = instr_desc(FMT_BF16, UM, TILE_R);
            const uint64_t dbase = smem_desc_kmajor(smem_u32(stages), 64, SWZ_64B);
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && alive; tile += gridDim.x) {
                for (int kb = 0; kb < p.nkb; ++kb) {
                    if (!mbar_wait(&full[s], ph, abort_flag)) { alive = false; break; }
                    tc_fence_after();
                    const uint64_t rows_hi = dbase + (uint64_t)(((uint32_t)s * (uint32_t)sbytes) >> 4);
                    const uint64_t w_hi = rows_hi + (uint64_t)((NSPLIT * ROW_TILE_BYTES) >> 4);
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) {          // 2 x 32 bytes of K (16 bf16 each)
                        const uint64_t adv = (uint64_t)(ks * 2);
                        const uint32_t first = (kb | ks) != 0;
                        if (NSPLIT == 1) {
                            mma_f16(tmem_base, w_hi + adv, rows_hi + adv, idesc, first);
                        } else {
                            const uint64_t rows_lo = rows_hi + (uint64_t)(ROW_TILE_BYTES >> 4);
                            const uint64_t w_lo = w_hi + (uint64_t)(W_TILE_BYTES >> 4);
                            mma_f16(tmem_base, w_lo + adv, rows_hi + adv, idesc, first);
                            mma_f16(tmem_base, w_hi + adv, rows_lo + adv, idesc, 1u);
                            mma_f16(tmem_base, w_hi + adv, rows_hi + adv, idesc, 1u);
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
    if (warp == PWARPS) tmem_dealloc(tmem_base, TILE_R);
    if (tid == 0 && abort_flag[0] && p.async_err) {
        *p.async_err = 4;
        __threadfence_system();
    }
}

// ---------------------------------------------------------------------------- host side
struct Plan { int nsplit, nkb, nstages; size_t smem, wimg_bytes; };

static Plan plan(int C, int precision) {
    Plan pl;
    pl.nsplit = precision == PB200_PREC_BF16 ? 1 : 2;
    pl.nkb = (C + KB - 1) / KB;
    pl.nstages = pl.nsplit == 2 ? 4 : 6;
    pl.smem = (size_t)pl.nstages * stage_bytes(pl.nsplit) + 1024 + 256;
    pl.wimg_bytes = (size_t)pl.nkb * pl.nsplit * W_TILE_BYTES;
    return pl;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int MODE>
static int run(Params p, int Cout, const float* wd, const float* bias, float* out, int precision, void* ws,
               cudaStream_t stream) {
    int rc = tc::check_async_error("pointwise fusion");
    if (rc) return rc;
    const Plan pl = plan(p.C, precision);
    uint8_t* wimg = (uint8_t*)ws;
    p.nkb = pl.nkb; p.nstages = pl.nstages; p.out_stride = Cout;
    p.async_err = tc::async_error_word();
    p.wait_budget = tc::wait_budget_kclocks();
    const int64_t ntiles = ceil_div(p.Nrows, TILE_R);
    const int grid = (int)(ntiles < sm_count() ? ntiles : sm_count());
    for (int co0 = 0; co0 < Cout; co0 += UM) {
        const int cchunk = Cout - co0 < UM ? Cout - co0 : UM;
        PB_LAUNCH("pw_prep_weights", pw_prep_weights_kernel, persistent_blocks((int64_t)pl.nkb * UM * 4, 256, 8), 256, 0, stream,
                  p.C, Cout, co0, cchunk, pl.nkb, pl.nsplit, wd, wimg);
        p.Cout = cchunk; p.wimg = wimg; p.bias = bias ? bias + co0 : nullptr; p.out = out + co0;
        const char* label = MODE == 0 ? "v2f_pointwise_tc" : (MODE == 1 ? "f2v_pointwise_tc" : "masked_rows_tc");
        if (MODE == 2 && co0 > 0) p.masked_out = nullptr;      // the by-product is written by the first chunk's launch
        if (pl.nsplit == 2) {
            PB_CUDA(cudaFuncSetAttribute(rows_pointwise_tc_kernel<2, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
            PB_LAUNCH(label, (rows_pointwise_tc_kernel<2, MODE>), grid, NTHREADS, pl.smem, stream, p);
        } else {
            PB_CUDA(cudaFuncSetAttribute(rows_pointwise_tc_kernel<1, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
            PB_LAUNCH(label, (rows_pointwise_tc_kernel<1, MODE>), grid, NTHREADS, pl.smem, stream, p);
        }
    }
    return PB200_OK;
}

}  // namespace pw
}  // namespace pb

using namespace pb;

extern "C" {

size_t pb200_vertex2facet_pointwise_workspace_bytes(int C, int precision) {
    if (C <= 0) return 0;
    return align_up(pw::plan(C, precision).wimg_bytes, 256);
}

int pb200_vertex2facet_pointwise_forward(int64_t Nf, int64_t Nv, int C, int Cout, const float* input, const float* filter,
                                         const int32_t* face, const float* depthWeights, const float* bias, int relu,
                                         float* output, int precision, void* workspace, size_t workspace_bytes,
                                         void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && Nv >= 0 && C > 0 && Cout > 0 && C % 8 == 0 && Nf < (1LL << 31) && Nv < (1LL << 31), PB200_EINVAL,
               "vertex2facet_pointwise_forward: bad sizes (channels must be a multiple of 8)");
    PB_REQUIRE(precision == PB200_PREC_FP32 || precision == PB200_PREC_BF16, PB200_EINVAL,
               "vertex2facet_pointwise_forward: precision must be PB200_PREC_FP32 or PB200_PREC_BF16");
    if (Nf == 0) return PB200_OK;
    PB_REQUIRE(input && filter && face && depthWeights && output, PB200_EINVAL, "vertex2facet_pointwise_forward: null pointer");
    PB_REQUIRE(pw::aligned16(input) && pw::aligned16(filter) && pw::aligned16(workspace), PB200_EINVAL,
               "vertex2facet_pointwise_forward: input, filter and workspace must be 16-byte aligned");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_vertex2facet_pointwise_workspace_bytes(C, precision), PB200_EWORKSPACE,
               "vertex2facet_pointwise_forward: workspace too small");
    pw::Params p = {};
    p.Nrows = Nf; p.C = C; p.relu = relu;
    p.vin = input; p.vfilt = filter; p.face = face; p.Nv = Nv;
    return pw::run<0>(p, Cout, depthWeights, bias, output, precision, workspace, stream);
}

size_t pb200_facet2vertex_pointwise_workspace_bytes(int64_t Nf, int C, int precision) {
    if (C <= 0 || Nf < 0) return 0;
    return align_up(pw::plan(C, precision).wimg_bytes, 256) + align_up(sizeof(float) * (size_t)(Nf > 0 ? Nf : 1) * C, 256);
}

int pb200_facet2vertex_pointwise_forward(int64_t Nf, int64_t NvOut, int C, int K, int Cout, const float* input,
                                         const float* filter, const float* coeff, const int32_t* nfCount,
                                         const int32_t* rowptr, const int32_t* entries, const float* depthWeights,
                                         const float* bias, int relu, float* output, int precision, void* workspace,
                                         size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NvOut >= 0 && C > 0 && K > 0 && Cout > 0 && C % 8 == 0 && f2v_face_products_supported(C, K) &&
                   Nf < (1LL << 29) && NvOut < (1LL << 31),
               PB200_EINVAL, "facet2vertex_pointwise_forward: bad sizes (channels must be a multiple of 8)");
    PB_REQUIRE(precision == PB200_PREC_FP32 || precision == PB200_PREC_BF16, PB200_EINVAL,
               "facet2vertex_pointwise_forward: precision must be PB200_PREC_FP32 or PB200_PREC_BF16");
    if (NvOut == 0) return PB200_OK;
    PB_REQUIRE(rowptr && nfCount && depthWeights && output && (Nf == 0 || (input && filter && coeff && entries)), PB200_EINVAL,
               "facet2vertex_pointwise_forward: null pointer");
    PB_REQUIRE(workspace && pw::aligned16(workspace) &&
                   workspace_bytes >= pb200_facet2vertex_pointwise_workspace_bytes(Nf, C, precision),
               PB200_EWORKSPACE, "facet2vertex_pointwise_forward: workspace missing, misaligned or too small");
    PB_REQUIRE(Nf == 0 || (pw::aligned16(input) && pw::aligned16(filter)), PB200_EINVAL,
               "facet2vertex_pointwise_forward: input and filter must be 16-byte aligned");
    float* wx = (float*)((char*)workspace + align_up(pw::plan(C, precision).wimg_bytes, 256));
    if (Nf > 0) {
        int rc = f2v_face_products(Nf, C, K, input, filter, coeff, wx, stream);
        if (rc) return rc;
    }
    pw::Params p = {};
    p.Nrows = NvOut; p.C = C; p.relu = relu;
    p.wx = wx; p.rowptr = rowptr; p.entries = entries; p.nfCount = nfCount;
    return pw::run<1>(p, Cout, depthWeights, bias, output, precision, workspace, stream);
}

size_t pb200_masked_rows_matmul_workspace_bytes(int C, int precision) {
    if (C <= 0) return 0;
    return align_up(pw::plan(C, precision).wimg_bytes, 256);
}

int pb200_rows_pointwise_forward(int64_t Nrows, int C, int Cout, const float* rows, const float* weights, const float* bias,
                                 int relu, float* output, int precision, void* workspace, size_t workspace_bytes,
                                 void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nrows >= 0 && C > 0 && Cout > 0 && C % 8 == 0 && Nrows < (1LL << 31), PB200_EINVAL,
               "rows_pointwise_forward: bad sizes (the row width must be a multiple of 8)");
    PB_REQUIRE(precision == PB200_PREC_FP32 || precision == PB200_PREC_BF16, PB200_EINVAL,
               "rows_pointwise_forward: precision must be PB200_PREC_FP32 or PB200_PREC_BF16");
    if (Nrows == 0) return PB200_OK;
    PB_REQUIRE(rows && weights && output, PB200_EINVAL, "rows_pointwise_forward: null pointer");
    PB_REQUIRE(pw::aligned16(rows) && pw::aligned16(workspace), PB200_EINVAL,
               "rows_pointwise_forward: rows and workspace must be 16-byte aligned");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_masked_rows_matmul_workspace_bytes(C, precision), PB200_EWORKSPACE,
               "rows_pointwise_forward: workspace too small");
    pw::Params p = {};
    p.Nrows = Nrows; p.C = C; p.relu = relu;
    p.rows = rows;
    return pw::run<2>(p, Cout, weights, bias, output, precision, workspace, stream);
}

int pb200_masked_rows_matmul(int64_t Nrows, int C, int Cout, const float* rows, const float* mask, const float* weights,
                             float* output, float* maskedRows, int precision, void* workspace, size_t workspace_bytes,
                             void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nrows >= 0 && C > 0 && Cout > 0 && C % 8 == 0 && Nrows < (1LL << 31), PB200_EINVAL,
               "masked_rows_matmul: bad sizes (the row width must be a multiple of 8)");
    PB_REQUIRE(precision == PB200_PREC_FP32 || precision == PB200_PREC_BF16, PB200_EINVAL,
               "masked_rows_matmul: precision must be PB200_PREC_FP32 or PB200_PREC_BF16");
    if (Nrows == 0) return PB200_OK;
    PB_REQUIRE(rows && weights && output, PB200_EINVAL, "masked_rows_matmul: null pointer");
    PB_REQUIRE(pw::aligned16(rows) && pw::aligned16(mask) && pw::aligned16(maskedRows) && pw::aligned16(workspace), PB200_EINVAL,
               "masked_rows_matmul: rows, mask, maskedRows and workspace must be 16-byte aligned");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_masked_rows_matmul_workspace_bytes(C, precision), PB200_EWORKSPACE,
               "masked_rows_matmul: workspace too small");
    pw::Params p = {};
    p.Nrows = Nrows; p.C = C; p.relu = 0;
    p.rows = rows; p.mask = mask; p.masked_out = maskedRows;
    return pw::run<2>(p, Cout, weights, nullptr, output, precision, workspace, stream);
}

}  // extern "C"

// Contraction of two row-major matrices over their rows on tcgen05 + TMEM:
//
//     out[m, n]  = sum_rows A[row, m] * B[row, n]        A (Nrows, M), B (Nrows, N), out (M, N)
//     colsum[n]  = sum_rows B[row, n]                    (optional)
//
// This is the weight gradient (and, with colsum, the bias gradient) of a pointwise stage
// out = act(feats @ W + b): A = feats, B = the masked upstream gradient.  The reference's modules
// leave it to autograd, which runs an fp32 SIMT GEMM with a contraction length of millions
// (picasso/mesh/layers.py:109-120,166-175 are the forward it differentiates).
//
// Rows are the K dimension of the product, and both matrices already lie in memory as the
// MN-major operands want them (a row = a K-row whose M / N elements are contiguous), so the
// producers only convert: 8 warps read 4 rows each per stage of 32 rows (a lane = 4 channels of A
// and 4 or 8 of B), split them into bf16 hi + lo and store 8-byte pieces of 128-byte-swizzled
// K-rows; one thread issues tcgen05.mma (M = 128 columns of A, N <= 256 columns of B, K = 16 rows
// per instruction, three products per term in the hi+lo mode) into a TMEM accumulator.
// The tensor core's adder truncates, so one CTA sums at most 4096 rows (768 accumulating
// instructions, drift 1e-5), fewer when that gives the GPU more CTAs to run (two per SM); the
// per-CTA partial results are added in CTA order by a second kernel, which also makes the result
// independent of scheduling.  All waits are bounded.
#include "common.cuh"
#include "tc_ptx.cuh"
#include "tc_runtime.cuh"

namespace pb {
namespace tc {
namespace rc {

using namespace ptx;

constexpr int UM = 128;                       // columns of A per launch (UMMA M)
constexpr int UN = 256;                       // columns of B per launch (UMMA N), at most
constexpr int RS = 32;                        // rows per stage (two K-steps of 16)
constexpr int PWARPS = 8;
constexpr int NTHREADS = (PWARPS + 1) * 32;
constexpr int MAX_ROWS_PER_CTA = 4096;        // longest accumulator chain: 768 instructions
constexpr int MIN_ROWS_PER_CTA = 256;
constexpr int ATOM = 1024;                    // 8 K-rows x 128 bytes (64 bf16 columns)
constexpr int SBO_A = (UM / 64) * ATOM;       // next 8 rows of the A tile
constexpr int SBO_B = (UN / 64) * ATOM;
constexpr int A_TILE = (RS / 8) * SBO_A;      // one split of the A tile of a stage
constexpr int B_TILE = (RS / 8) * SBO_B;
constexpr int NSTAGES = 2;                    // 2 stages -> two CTAs per SM

struct Params {
    int64_t Nrows;
    int M, N;                 // full widths (= row strides) of A and B
    int m0, n0, Mw, Nw;       // this launch's chunk of columns
    const float* A;
    const float* B;
    float* partial;           // [gridDim.x][M][N]
    float* colsum_partial;    // [gridDim.x][N] or NULL
    int rows_per_cta;
    int* async_err;
    int wait_budget;
};

__host__ __device__ constexpr size_t stage_bytes(int nsplit) { return (size_t)nsplit * (A_TILE + B_TILE); }

__device__ __forceinline__ void sts_u2(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
// four consecutive columns of a K-row: one 8-byte piece in the hi tile (and in the lo tile)
template <int NSPLIT>
__device__ __forceinline__ void put4(uint32_t a, uint32_t lo_off, const float4& v) {
    if (NSPLIT == 1) {
        sts_u2(a, pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    } else {
        uint32_t hi[2], lo[2];
        split_bf16x2(v.x, v.y, hi[0], lo[0]); split_bf16x2(v.z, v.w, hi[1], lo[1]);
        sts_u2(a, hi[0], hi[1]);
        sts_u2(a + lo_off, lo[0], lo[1]);
    }
}
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok) (void)mbar_try_wait(bar, parity);
    return ok != 0;
}

template <int NSPLIT>
__global__ void __launch_bounds__(NTHREADS, 2) rows_contract_tc_kernel(Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr size_t SB = stage_bytes(NSPLIT);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NSTAGES * SB);
    uint64_t* full = bars;                    // [NSTAGES] operands written by the 8 producer warps
    uint64_t* empty = bars + NSTAGES;         // [NSTAGES] products of the stage complete
    uint64_t* acc_done = bars + 2 * NSTAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* csum_s = reinterpret_cast<float*>(smem + NSTAGES * SB + 256);          // [PWARPS][UN] column sums of the warps

    if (tid == 0) {
        for (int s = 0; s < NSTAGES; ++s) { mbar_init(&full[s], PWARPS); mbar_init(&empty[s], 1); }
        mbar_init(acc_done, 1);
        abort_flag[0] = 0;
        abort_flag[1] = p.wait_budget;
        fence_barrier_init();
    }
    if (warp == PWARPS) { tmem_alloc(tmem_slot, UN); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t s32 = smem_u32(smem);

    const int64_t row_begin = (int64_t)blockIdx.x * p.rows_per_cta;
    int64_t row_end = row_begin + p.rows_per_cta;
    if (row_end > p.Nrows) row_end = p.Nrows;
    const int nst = row_end > row_begin ? (int)((row_end - row_begin + RS - 1) / RS) : 0;
    const int nmma = (p.Nw + 15) / 16 * 16;                  // UMMA N of this launch

    if (warp < PWARPS) {
        // ==================================== producers ====================================
        const bool a_on = 4 * lane < p.Mw;
        const bool b0_on = 4 * lane < p.Nw, b1_on = 128 + 4 * lane < p.Nw;
        const bool two = p.Nw > 128;
        float4 cs0 = zero4(), cs1 = zero4();
        int si = 0;
        uint32_t sph = 0;
        bool alive = true;
        for (int st = 0; st < nst; ++st) {
            // the stage's rows of this warp first (loads in flight while waiting for the slot)
            float4 va[4], vb0[4], vb1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t row = row_begin + (int64_t)st * RS + warp + 8 * i;
                const bool on = row < row_end;
                va[i] = (on && a_on) ? ldg4(reinterpret_cast<const float4*>(p.A + row * p.M + p.m0) + lane) : zero4();
                vb0[i] = (on && b0_on) ? ldg4(reinterpret_cast<const float4*>(p.B + row * p.N + p.n0) + lane) : zero4();
                vb1[i] = (on && b1_on) ? ldg4(reinterpret_cast<const float4*>(p.B + row * p.N + p.n0 + 128) + lane) : zero4();
            }
            if (!warp_wait(&empty[si], sph ^ 1u, abort_flag, lane)) { alive = false; break; }
            const uint32_t sa = s32 + (uint32_t)si * (uint32_t)SB;             // [A hi][A lo?][B hi][B lo?]
            const uint32_t sb = sa + NSPLIT * A_TILE;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = warp + 8 * i;                                      // K-row of the stage
                const uint32_t piece = ((((uint32_t)(lane & 15) >> 1) ^ (uint32_t)(k & 7)) << 4) + (uint32_t)(lane & 1) * 8u;
                const uint32_t rowa = (uint32_t)(k >> 3) * SBO_A + (uint32_t)(k & 7) * 128u + (uint32_t)(lane >> 4) * ATOM + piece;
                const uint32_t rowb = (uint32_t)(k >> 3) * SBO_B + (uint32_t)(k & 7) * 128u + (uint32_t)(lane >> 4) * ATOM + piece;
                put4<NSPLIT>(sa + rowa, A_TILE, va[i]);
                put4<NSPLIT>(sb + rowb, B_TILE, vb0[i]);
                if (two) put4<NSPLIT>(sb + rowb + 2 * ATOM, B_TILE, vb1[i]);
                add4(cs0, vb0[i]);
                add4(cs1, vb1[i]);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[si]);
            if (++si == NSTAGES) { si = 0; sph ^= 1u; }
        }
        // column sums of B: the warps' sums in warp order
        if (p.colsum_partial) {
            reinterpret_cast<float4*>(csum_s + warp * UN)[lane] = cs0;
            reinterpret_cast<float4*>(csum_s + warp * UN + 128)[lane] = cs1;
        }
        // ---- drain: accumulator rows = columns of A, accumulator columns = columns of B
        if (alive && warp_wait(acc_done, 0u, abort_flag, lane)) {
            tc_fence_after();
            const int q = warp & 3, half = warp >> 2;
            const int m = q * 32 + lane;
            float* out = p.partial + (int64_t)blockIdx.x * p.M * p.N + (int64_t)(p.m0 + m) * p.N + p.n0;
#pragma unroll 1
            for (int g = 0; g < 4; ++g) {
                const int col = half * 128 + g * 32;
                if (col >= nmma) break;
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)col, r);
                tmem_ld_wait();
                if (m < p.Mw) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        if (col + j < p.Nw)
                            *reinterpret_cast<float4*>(out + col + j) =
                                nst > 0 ? make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                                      __uint_as_float(r[j + 3]))
                                        : zero4();
                }
            }
            tc_fence_before();
        }
    } else if (lane == 0) {
        // ================================== product issuer ==================================
        const uint32_t idesc = instr_desc_mnmajor(FMT_BF16, UM, (uint32_t)nmma);
        const uint64_t da0 = smem_desc_mnmajor_b16(s32, ATOM, SBO_A);
        const uint64_t db0 = smem_desc_mnmajor_b16(s32 + NSPLIT * A_TILE, ATOM, SBO_B);
        int si = 0;
        uint32_t sph = 0;
        bool alive = true;
        for (int st = 0; st < nst; ++st) {
            if (!mbar_wait(&full[si], sph, abort_flag)) { alive = false; break; }
            tc_fence_after();
            const uint64_t soff = (uint64_t)(((uint32_t)si * (uint32_t)SB) >> 4);
#pragma unroll
            for (int ks = 0; ks < RS / 16; ++ks) {
                const uint64_t a_hi = da0 + soff + (uint64_t)((ks * 2 * SBO_A) >> 4);
                const uint64_t b_hi = db0 + soff + (uint64_t)((ks * 2 * SBO_B) >> 4);
                const uint32_t first = (st | ks) != 0;
                if (NSPLIT == 1) {
                    mma_f16(tmem_base, a_hi, b_hi, idesc, first);
                } else {
                    mma_f16(tmem_base, a_hi + (A_TILE >> 4), b_hi, idesc, first);
                    mma_f16(tmem_base, a_hi, b_hi + (B_TILE >> 4), idesc, 1u);
                    mma_f16(tmem_base, a_hi, b_hi, idesc, 1u);
                }
            }
            tc_commit(&empty[si]);
            if (++si == NSTAGES) { si = 0; sph ^= 1u; }
        }
        if (alive) tc_commit(acc_done);
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (p.colsum_partial && tid < p.Nw && !abort_flag[0]) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < PWARPS; ++w) s += csum_s[w * UN + tid];
        p.colsum_partial[(int64_t)blockIdx.x * p.N + p.n0 + tid] = s;
    }
    if (warp == PWARPS) tmem_dealloc(tmem_base, UN);
    if (tid == 0 && abort_flag[0] && p.async_err) {
        *p.async_err = 6;
        __threadfence_system();
    }
}

// rows per CTA: enough CTAs to fill the GPU twice over when the rows allow it, never a chain longer than
// MAX_ROWS_PER_CTA, and not so many CTAs that the partial results outgrow 256 MB
static int rows_per_cta(int64_t Nrows, int M, int N) {
    int64_t r = ceil_div(Nrows > 0 ? Nrows : 1, 2 * (int64_t)sm_count());
    r = ceil_div(r, RS) * RS;
    if (r < MIN_ROWS_PER_CTA) r = MIN_ROWS_PER_CTA;
    const int64_t cap_ctas = (256LL << 20) / ((int64_t)M * N * 4);
    if (cap_ctas > 0 && ceil_div(Nrows, r) > cap_ctas) r = ceil_div(ceil_div(Nrows, cap_ctas), RS) * RS;
    if (r > MAX_ROWS_PER_CTA) r = MAX_ROWS_PER_CTA;
    return (int)r;
}

constexpr size_t smem_bytes(int nsplit) { return NSTAGES * stage_bytes(nsplit) + 256 + PWARPS * UN * 4 + 1024; }

}  // namespace rc
}  // namespace tc
}  // namespace pb

using namespace pb;

extern "C" {

size_t pb200_rows_contract_workspace_bytes(int64_t Nrows, int M, int N) {
    if (Nrows < 0 || M <= 0 || N <= 0) return 0;
    const size_t ctas = (size_t)ceil_div(Nrows > 0 ? Nrows : 1, tc::rc::rows_per_cta(Nrows, M, N));
    return align_up(sizeof(float) * ctas * (size_t)M * N, 256) + align_up(sizeof(float) * ctas * (size_t)N, 256);
}

int pb200_rows_contract(int64_t Nrows, int M, int N, const float* A, const float* B, float* out, float* colsum, int precision,
                        void* workspace, size_t workspace_bytes, void* stream_) {
    using namespace tc::rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nrows >= 0 && M > 0 && N > 0 && M % 4 == 0 && N % 4 == 0 && Nrows < (1LL << 31), PB200_EINVAL,
               "rows_contract: bad sizes (the widths must be multiples of 4)");
    PB_REQUIRE(precision == PB200_PREC_FP32 || precision == PB200_PREC_BF16, PB200_EINVAL,
               "rows_contract: precision must be PB200_PREC_FP32 or PB200_PREC_BF16");
    PB_REQUIRE(out, PB200_EINVAL, "rows_contract: null pointer");
    if (Nrows == 0) {
        PB_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * (size_t)M * N, stream));
        if (colsum) PB_CUDA(cudaMemsetAsync(colsum, 0, sizeof(float) * (size_t)N, stream));
        return PB200_OK;
    }
    PB_REQUIRE(A && B, PB200_EINVAL, "rows_contract: null pointer");
    PB_REQUIRE((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0, PB200_EINVAL,
               "rows_contract: A and B must be 16-byte aligned");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_rows_contract_workspace_bytes(Nrows, M, N), PB200_EWORKSPACE,
               "rows_contract: workspace too small");
    int rc = tc::check_async_error("rows_contract");
    if (rc) return rc;
    const int rpc = rows_per_cta(Nrows, M, N);
    const int ctas = (int)ceil_div(Nrows, rpc);
    Params p;
    p.rows_per_cta = rpc;
    p.Nrows = Nrows; p.M = M; p.N = N; p.A = A; p.B = B;
    p.partial = (float*)workspace;
    float* cpart = (float*)((char*)workspace + align_up(sizeof(float) * (size_t)ctas * M * N, 256));
    p.async_err = tc::async_error_word();
    p.wait_budget = tc::wait_budget_kclocks();
    const int nsplit = precision == PB200_PREC_BF16 ? 1 : 2;
    const size_t smem = smem_bytes(nsplit);
    for (int m0 = 0; m0 < M; m0 += UM)
        for (int n0 = 0; n0 < N; n0 += UN) {
            p.m0 = m0; p.n0 = n0;
            p.Mw = M - m0 < UM ? M - m0 : UM;
            p.Nw = N - n0 < UN ? N - n0 : UN;
            p.colsum_partial = (colsum && m0 == 0) ? cpart : nullptr;
            if (nsplit == 2) {
                PB_CUDA(cudaFuncSetAttribute(rows_contract_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                PB_LAUNCH("rows_contract_tc", rows_contract_tc_kernel<2>, ctas, NTHREADS, smem, stream, p);
            } else {
                PB_CUDA(cudaFuncSetAttribute(rows_contract_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                PB_LAUNCH("rows_contract_tc", rows_contract_tc_kernel<1>, ctas, NTHREADS, smem, stream, p);
            }
        }
    rc = reduce_partials(p.partial, ctas, (int64_t)M * N, out, stream);
    if (rc) return rc;
    if (colsum) return reduce_partials(cpart, ctas, N, colsum, stream);
    return PB200_OK;
}

}  // extern "C"

// Thin wrappers over the sm_100a PTX this library uses: mbarriers, bulk (TMA-engine)
// copies, tcgen05 tensor-core instructions with TMEM accumulators.  Every wait is
// bounded: it gives up after a clock budget, raises the block's abort flag, and returns
// false so the caller can unwind, free its TMEM and report the failure.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pb {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Default wait budget in units of 1024 clocks: about one second at 2 GHz, far above any
// legitimate wait of these kernels.  A block keeps two ints in shared memory: abort_flag[0]
// is the flag, abort_flag[1] the budget (set once by thread 0 before the first wait).
constexpr int WAIT_BUDGET_KCLOCKS = 2000000;

// Bounded wait on one phase of an mbarrier.  Returns false (and raises *abort_flag) on
// time-out, or as soon as another thread of the block has raised the flag.
// A failed probe backs off with a short sleep so that a waiting role (the MMA issuer, the
// bulk-copy thread) does not take issue slots from the warps it is waiting for.
#ifndef PB_WAIT_SPIN
#define PB_WAIT_SPIN 0          // probes without a sleep in between before the back-off starts
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
        if (i >= PB_WAIT_SPIN) __nanosleep(i < PB_WAIT_SPIN + 8 ? 20 : 100);
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            if (abort_flag[0]) return false;
            if (((clock64() - t0) >> 10) > (long long)abort_flag[1]) { abort_flag[0] = 1; return false; }
        }
    }
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// make generic-proxy shared-memory writes visible to the async proxy (tensor core, bulk copy)
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// -------------------------------------------------------------------- bulk (TMA) copies
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.  Source and
// destination 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// ------------------------------------------------------------------------------ tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {   // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {                                 // whole warp
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {      // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// arrive on an mbarrier when every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns of TMEM -> 32 registers per thread (lane = row)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------- UMMA descriptors
// Shared-memory matrix descriptor of a K-major operand tile stored as rows of `row_bytes`
// (32, 64 or 128) with the matching swizzle; 8-row groups are contiguous (SBO = 8 rows).
constexpr uint64_t SWZ_128B = 2, SWZ_64B = 4, SWZ_32B = 6;
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t smem_addr, uint32_t row_bytes, uint64_t swizzle) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);              // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                    // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)((8u * row_bytes) >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                    // descriptor version of sm_100
    d |= swizzle << 61;
    return d;
}

// Shared-memory matrix descriptor of an MN-major operand tile of 32-bit elements (the one
// layout tf32 accepts MN-major: 128-byte swizzle with a 32-byte base).  A 512-byte atom holds
// 4 K-rows of 128 bytes (32 consecutive M/N elements); `lbo_bytes` steps to the next 32 M/N
// elements, `sbo_bytes` to the next 4 K-rows.  32-byte chunk j of K-row k sits at chunk
// j ^ (k & 3) of the row (address bits [5,7) ^= bits [7,9)); atoms are 512-byte aligned.
constexpr uint64_t SWZ_128B_BASE32B = 1;
__device__ __forceinline__ uint64_t smem_desc_mnmajor_b32(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= SWZ_128B_BASE32B << 61;
    return d;
}

// Instruction descriptor: fp32 accumulate, both operands K-major, M x N tile.
constexpr uint32_t FMT_F16 = 0, FMT_BF16 = 1, FMT_TF32 = 2;
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt_ab, uint32_t M, uint32_t N) {
    return (1u << 4) | (fmt_ab << 7) | (fmt_ab << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// the same with both operands MN-major (bits 15 and 16)
__host__ __device__ constexpr uint32_t instr_desc_mnmajor(uint32_t fmt_ab, uint32_t M, uint32_t N) {
    return instr_desc(fmt_ab, M, N) | (1u << 15) | (1u << 16);
}

// byte offset of 16-byte chunk `c` of row `r` inside a K-major tile with 64-byte rows and
// 64-byte swizzle (address bits [4,5] ^= bits [7,8])
__device__ __forceinline__ uint32_t swz64_offset(uint32_t r, uint32_t c) {
    return r * 64u + ((c ^ ((r >> 1) & 3u)) << 4);
}

// shared-window (32-bit address) accessors: one instruction each, immediate offsets fold in
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ int lds_i32(uint32_t a) {
    int v;
    asm volatile("ld.shared.s32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_f4(uint32_t a, const float4& v) {
    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__device__ __forceinline__ float to_tf32_rna(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}
__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

// two floats -> packed bf16x2 (round to nearest even), first value in the low half
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// hi = bf16(v), lo = bf16(v - hi) for two values at once
__device__ __forceinline__ void split_bf16x2(float a, float b, uint32_t& hi, uint32_t& lo) {
    hi = pack_bf16x2(a, b);
    // both remainders with one packed FMA: (a, b) - (hi_a, hi_b)
    const float2 h2 = make_float2(__uint_as_float(hi << 16), __uint_as_float(hi & 0xFFFF0000u));
    const float2 r = __ffma2_rn(h2, make_float2(-1.f, -1.f), make_float2(a, b));
    lo = pack_bf16x2(r.x, r.y);
}

// Shared-memory matrix descriptor of an MN-major operand tile of 16-bit elements with the
// 128-byte swizzle: a 1 KB atom holds 8 K-rows of 128 bytes (64 consecutive M/N elements);
// `lbo_bytes` steps to the next 64 M/N elements, `sbo_bytes` to the next 8 K-rows.  16-byte
// chunk c of K-row k sits at chunk c ^ (k & 7) of the row; atoms are 1 KB aligned.
__device__ __forceinline__ uint64_t smem_desc_mnmajor_b16(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= SWZ_128B << 61;
    return d;
}

}  // namespace ptx
}  // namespace pb

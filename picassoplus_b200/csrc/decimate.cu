// Quadric-error mesh decimation, one pass (the reference's `meshDecimationLauncher`,
// picasso/mesh/pi_modules/source/decimate_gpu.cu:618-747) and the cluster merge
// (`combineClustersLauncher`, decimate_gpu.cu:750-812), entirely on the device.
//
// The reference sorts edge indices with a comparator sort, loops over the samples of the batch
// on the host (unique / cost / sort per sample), copies the sorted candidates to the host and
// clusters vertices there in two sequential sweeps.  Here one pass is:
//   1. edge keys (lower vertex, higher vertex) -> stable LSD radix sort -> boundary flags
//      (an edge seen once) and the list of distinct candidates, for the whole batch at once;
//   2. vertex quadrics pulled through the vertex CSR in ascending (face, corner) order
//      (no float atomics: run-to-run deterministic), boundary quadrics in the same walk;
//   3. candidate costs, one radix sort by (sample, cost) -> every candidate's rank;
//   4. the first sequential sweep (an edge is taken when neither end is covered) is the greedy
//      matching in rank order.  It equals the fixed point of "take every edge whose rank is
//      the smallest among the live edges at both of its ends", computed in parallel rounds
//      (atomicMin per vertex); the sweep's early stop is a prefix count over ranks;
//   5. the second sweep attaches every still-uncovered vertex through its lowest-ranked
//      edge: after a complete first sweep no edge joins two uncovered vertices, so these
//      choices are independent; its early stop is again a prefix count;
//   6. cluster positions (members added in ascending vertex id), relabelled faces, degenerate
//      flags, vertex map and the per-sample output sizes.
// Results equal the sequential procedure's for any input; the host reads back three counters
// (a few stream synchronisations), never mesh data.
//
// This file is compiled with --fmad=false: every float operation is rounded on its own, so the
// costs (and therefore the clustering) can be reproduced exactly by a plain C restatement.
#include "common.cuh"

namespace pb {
namespace dec {

constexpr uint32_t NO_RANK = 0xffffffffu;

// ------------------------------------------------------------------ exclusive scan (int32)
// out[0..n] (n + 1 values): out[i] = sum of in[0..i); in place allowed.
constexpr int SC_THREADS = 256, SC_ITEMS = 8, SC_TILE = SC_THREADS * SC_ITEMS;

__global__ void scan_tiles_kernel(const int32_t* in, int64_t n, int32_t* out, int32_t* __restrict__ tile_sum) {
    __shared__ int32_t warp_tot[SC_THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * SC_TILE + (int64_t)threadIdx.x * SC_ITEMS;
    int32_t v[SC_ITEMS], run = 0;
#pragma unroll
    for (int j = 0; j < SC_ITEMS; ++j) {
        const int32_t x = (base + j < n) ? in[base + j] : 0;
        v[j] = run;
        run += x;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int32_t inc = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int32_t warp_off = 0;
    for (int w = 0; w < warp; ++w) warp_off += warp_tot[w];
    const int32_t excl = warp_off + inc - run;
#pragma unroll
    for (int j = 0; j < SC_ITEMS; ++j)
        if (base + j <= n) out[base + j] = excl + v[j];
    if (threadIdx.x == SC_THREADS - 1) tile_sum[blockIdx.x] = warp_off + inc;
}

// one block: exclusive scan of the tile totals, 1024 at a time with a carry
__global__ void scan_sums_kernel(int32_t* __restrict__ tile_sum, int ntiles) {
    __shared__ int32_t wt[32];
    __shared__ int32_t carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < ntiles; base += 1024) {
        const int i = base + threadIdx.x;
        const int32_t x = i < ntiles ? tile_sum[i] : 0;
        int32_t inc = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int32_t t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) wt[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            const int32_t w = wt[lane];
            int32_t winc = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int32_t t = __shfl_up_sync(0xffffffffu, winc, o);
                if (lane >= o) winc += t;
            }
            wt[lane] = winc - w;
        }
        __syncthreads();
        const int32_t excl = carry + wt[warp] + inc - x;
        if (i < ntiles) tile_sum[i] = excl;
        __syncthreads();
        if (threadIdx.x == 1023) carry = excl + x;
        __syncthreads();
    }
}

__global__ void scan_add_kernel(int32_t* __restrict__ out, int64_t n, const int32_t* __restrict__ tile_off) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= n) out[i] += tile_off[i / SC_TILE];
}

static size_t scan_tiles_for(int64_t n) { return (size_t)ceil_div(n + 1, SC_TILE); }

static int exclusive_scan(const int32_t* in, int64_t n, int32_t* out, int32_t* tile_sum, cudaStream_t stream) {
    const int ntiles = (int)scan_tiles_for(n);
    PB_LAUNCH("dec_scan_tiles", scan_tiles_kernel, ntiles, SC_THREADS, 0, stream, in, n, out, tile_sum);
    if (ntiles > 1) {
        PB_LAUNCH("dec_scan_sums", scan_sums_kernel, 1, 1024, 0, stream, tile_sum, ntiles);
        PB_LAUNCH("dec_scan_add", scan_add_kernel, (unsigned)ceil_div(n + 1, 256), 256, 0, stream, out, n,
                  (const int32_t*)tile_sum);
    }
    return PB200_OK;
}

// ------------------------------------------------ stable LSD radix sort, 8 bits per pass
// 64-bit keys with a 32-bit payload.  A block owns a tile of 2048 consecutive elements, a warp
// 256 consecutive ones in 8 rounds of 32: the rank of an element among equal digits follows
// the element order, which makes every pass stable.
constexpr int RS_THREADS = 256, RS_ROUNDS = 8, RS_TILE = RS_THREADS * RS_ROUNDS, RS_WARPS = RS_THREADS / 32;

__global__ void rs_hist_kernel(const uint64_t* __restrict__ keys, int64_t n, int shift, int nblocks,
                               int32_t* __restrict__ hist) {
    __shared__ int32_t h[256];
    h[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * RS_TILE;
#pragma unroll
    for (int j = 0; j < RS_ROUNDS; ++j) {
        const int64_t i = base + j * RS_THREADS + threadIdx.x;
        if (i < n) atomicAdd(&h[(int)((keys[i] >> shift) & 255u)], 1);
    }
    __syncthreads();
    hist[(int64_t)threadIdx.x * nblocks + blockIdx.x] = h[threadIdx.x];
}

__global__ void rs_scatter_kernel(const uint64_t* __restrict__ kin, const uint32_t* __restrict__ vin,
                                  uint64_t* __restrict__ kout, uint32_t* __restrict__ vout, int64_t n, int shift,
                                  int nblocks, const int32_t* __restrict__ hist_scan) {
    __shared__ int32_t wc[RS_WARPS][256];
    for (int i = threadIdx.x; i < RS_WARPS * 256; i += RS_THREADS) (&wc[0][0])[i] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t seg = (int64_t)blockIdx.x * RS_TILE + (int64_t)warp * (RS_ROUNDS * 32);
    uint64_t k[RS_ROUNDS];
    uint32_t v[RS_ROUNDS];
    int32_t lr[RS_ROUNDS];
#pragma unroll
    for (int j = 0; j < RS_ROUNDS; ++j) {
        const int64_t i = seg + j * 32 + lane;
        const bool valid = i < n;
        k[j] = valid ? kin[i] : 0;
        v[j] = valid ? vin[i] : 0;
        const int d = valid ? (int)((k[j] >> shift) & 255u) : 256 + lane;     // elements past the end: groups of one
        const unsigned mask = __match_any_sync(0xffffffffu, d);
        const int leader = __ffs(mask) - 1;
        int32_t old = 0;
        if (valid && lane == leader) { old = wc[warp][d]; wc[warp][d] = old + __popc(mask); }
        old = __shfl_sync(0xffffffffu, old, leader);
        lr[j] = old + __popc(mask & ((1u << lane) - 1u));
        __syncwarp();
    }
    __syncthreads();
    {
        const int d = threadIdx.x;
        int32_t run = hist_scan[(int64_t)d * nblocks + blockIdx.x];
#pragma unroll
        for (int w = 0; w < RS_WARPS; ++w) { const int32_t t = wc[w][d]; wc[w][d] = run; run += t; }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < RS_ROUNDS; ++j) {
        const int64_t i = seg + j * 32 + lane;
        if (i < n) {
            const int32_t pos = wc[warp][(int)((k[j] >> shift) & 255u)] + lr[j];
            kout[pos] = k[j];
            vout[pos] = v[j];
        }
    }
}

// sorts (k, v) by the low `bits` bits of k; on return k / v point at the sorted arrays
static int radix_sort(uint64_t*& k, uint64_t*& kalt, uint32_t*& v, uint32_t*& valt, int64_t n, int bits,
                      int32_t* hist, int32_t* tile_sum, cudaStream_t stream) {
    if (n <= 1) return PB200_OK;
    const int nblocks = (int)ceil_div(n, RS_TILE);
    for (int shift = 0; shift < bits; shift += 8) {
        PB_LAUNCH("dec_sort_hist", rs_hist_kernel, nblocks, RS_THREADS, 0, stream, (const uint64_t*)k, n, shift, nblocks, hist);
        int rc = exclusive_scan(hist, (int64_t)256 * nblocks, hist, tile_sum, stream);
        if (rc != PB200_OK) return rc;
        PB_LAUNCH("dec_sort_scatter", rs_scatter_kernel, nblocks, RS_THREADS, 0, stream, (const uint64_t*)k,
                  (const uint32_t*)v, kalt, valt, n, shift, nblocks, (const int32_t*)hist);
        uint64_t* tk = k; k = kalt; kalt = tk;
        uint32_t* tv = v; v = valt; valt = tv;
    }
    return PB200_OK;
}

static int bit_length(int64_t x) { int b = 0; while (x > 0) { ++b; x >>= 1; } return b; }

// ------------------------------------------------------------------------ small helpers
// sample that owns vertex (or face) id x: first s with x < cum[s]; B when none
__device__ __forceinline__ int sample_of(int x, const int32_t* __restrict__ cum, int B) {
    int lo = 0, hi = B;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (x < cum[mid]) hi = mid; else lo = mid + 1; }
    return lo;
}

// appends the elements whose `pred` holds to list[*counter...]; called by whole warps
__device__ __forceinline__ void warp_append(bool pred, uint32_t value, uint32_t* __restrict__ list, int32_t* counter) {
    const unsigned m = __ballot_sync(0xffffffffu, pred);
    if (m == 0) return;
    const int lane = threadIdx.x & 31, leader = __ffs(m) - 1;
    int32_t base = 0;
    if (lane == leader) base = atomicAdd(counter, __popc(m));
    base = __shfl_sync(0xffffffffu, base, leader);
    if (pred) list[base + __popc(m & ((1u << lane) - 1u))] = value;
}

// face edge slots as the reference numbers them (decimate_gpu.cu:262-308):
// slot 0 joins corners (0,1), slot 1 corners (0,2), slot 2 corners (1,2)
__device__ __forceinline__ int slot_a(int k) { return k == 2 ? 1 : 0; }
__device__ __forceinline__ int slot_b(int k) { return k == 0 ? 1 : 2; }

// ------------------------------------------------------------------------------ edges
__global__ void edge_keys_kernel(int64_t Ne, int64_t Nv, int vbits, const int32_t* __restrict__ face,
                                 uint64_t* __restrict__ key, uint32_t* __restrict__ val, int32_t* __restrict__ status) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= Ne) return;
    const int64_t f = e / 3;
    const int k = (int)(e - 3 * f);
    int a = face[3 * f + slot_a(k)], b = face[3 * f + slot_b(k)];
    if (a < 0 || b < 0 || a >= Nv || b >= Nv) { *status = PB200_EINDEX; a = b = (int)Nv; }
    const uint64_t lo = (uint64_t)(a <= b ? a : b), hi = (uint64_t)(a <= b ? b : a);
    key[e] = (lo << vbits) | hi;
    val[e] = (uint32_t)e;
}

// over the sorted edges: boundary flag of the edge instance, first-of-run flag
__global__ void edge_flags_kernel(int64_t Ne, int64_t Nv, int vbits, const uint64_t* __restrict__ skey,
                                  const uint32_t* __restrict__ sval, uint8_t* __restrict__ bnd, int32_t* __restrict__ uflag) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Ne) return;
    const uint64_t k = skey[i];
    const bool valid = (int64_t)(k >> vbits) < Nv;
    const bool same_prev = i > 0 && skey[i - 1] == k;
    const bool same_next = i + 1 < Ne && skey[i + 1] == k;
    bnd[sval[i]] = (valid && !same_prev && !same_next) ? 1 : 0;
    uflag[i] = (valid && !same_prev) ? 1 : 0;
}

__global__ void unique_write_kernel(int64_t Ne, int vbits, const uint64_t* __restrict__ skey,
                                    const int32_t* __restrict__ uflag_scan, int32_t* __restrict__ ulo,
                                    int32_t* __restrict__ uhi) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Ne) return;
    if (uflag_scan[i + 1] == uflag_scan[i]) return;
    const uint64_t k = skey[i];
    const int u = uflag_scan[i];
    ulo[u] = (int32_t)(k >> vbits);
    uhi[u] = (int32_t)(k & ((1ull << vbits) - 1ull));
}

// ---------------------------------------------------------------------------- quadrics
__device__ __forceinline__ void plane_quadric(const float n0, const float n1, const float n2, const float d, float* Q) {
    Q[0] = n0 * n0; Q[1] = n0 * n1; Q[2] = n0 * n2;
    Q[3] = n1 * n1; Q[4] = n1 * n2; Q[5] = n2 * n2;
    Q[6] = n0 * d;  Q[7] = n1 * d;  Q[8] = n2 * d;
    Q[9] = d * d;
}

// One thread per vertex: the face quadrics of its corners in ascending (face, corner) order
// (decimate_gpu.cu:225-256), then the boundary quadrics of the corners' edges in the same
// order, lower edge slot first (decimate_gpu.cu:311-374).
__global__ void vertex_quadric_kernel(int64_t Nv, int D, int useArea, float wgtBnd, const int32_t* __restrict__ rowptr,
                                      const int32_t* __restrict__ entries, const int32_t* __restrict__ face,
                                      const float* __restrict__ plane, const float* __restrict__ vertex,
                                      const uint8_t* __restrict__ bnd, float* __restrict__ Qout) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= Nv) return;
    float acc[10];
#pragma unroll
    for (int t = 0; t < 10; ++t) acc[t] = 0.f;
    const int beg = rowptr[v], end = rowptr[v + 1];
    for (int p = beg; p < end; ++p) {
        const int64_t f = entries[p] >> 2;
        const float* pl = plane + 5 * f;
        float Q[10];
        plane_quadric(pl[0], pl[1], pl[2], pl[3], Q);
        const float area = pl[4] * 100.0f;
        const float w = useArea ? area / 3 : 1.0f;
#pragma unroll
        for (int t = 0; t < 10; ++t) acc[t] += Q[t] * w;
    }
    if (wgtBnd > 0)
        for (int p = beg; p < end; ++p) {
            const int64_t f = entries[p] >> 2;
            const int c = entries[p] & 3;
            for (int s = 0; s < 2; ++s) {
                const int k = c == 0 ? s : (c == 1 ? 2 * s : 1 + s);
                if (!bnd[3 * f + k]) continue;
                const int a = face[3 * f + slot_a(k)], b = face[3 * f + slot_b(k)];
                const int vi = a <= b ? a : b, vj = a <= b ? b : a;
                const float* pl = plane + 5 * f;
                const float* pi = vertex + (int64_t)vi * D;
                const float* pj = vertex + (int64_t)vj * D;
                const float dx0 = pj[0] - pi[0], dx1 = pj[1] - pi[1], dx2 = pj[2] - pi[2];
                float b0 = pl[1] * dx2 - pl[2] * dx1;
                float b1 = pl[2] * dx0 - pl[0] * dx2;
                float b2 = pl[0] * dx1 - pl[1] * dx0;
                float len = sqrtf(b0 * b0 + b1 * b1 + b2 * b2);
                len = len > 1e-20f ? len : 1e-20f;
                b0 /= len; b1 /= len; b2 /= len;
                const float d = -(b0 * pi[0] + b1 * pi[1] + b2 * pi[2]);
                float wb = (dx0 * dx0 + dx1 * dx1 + dx2 * dx2) * 100.0f;
                if (useArea) wb *= wgtBnd; else wb = wgtBnd;
                float Q[10];
                plane_quadric(b0, b1, b2, d, Q);
#pragma unroll
                for (int t = 0; t < 10; ++t) acc[t] += Q[t] * wb;
            }
        }
#pragma unroll
    for (int t = 0; t < 10; ++t) Qout[10 * v + t] = acc[t];
}

// quadric error x^T A x + 2 b.x + c with the reference's association (decimate_gpu.cu:189-197)
__device__ __forceinline__ float quadric_error(const float* x, const float (*A)[3], const float* b, float c) {
    return ((x[0] * A[0][0] + x[1] * A[1][0] + x[2] * A[2][0]) * x[0]
          + (x[0] * A[0][1] + x[1] * A[1][1] + x[2] * A[2][1]) * x[1]
          + (x[0] * A[0][2] + x[1] * A[1][2] + x[2] * A[2][2]) * x[2])
          + (x[0] * b[0] + x[1] * b[1] + x[2] * b[2]) * 2
          + c;
}

// Gauss-Jordan reduction of [A | b | I] with partial pivoting and the reference's column
// tolerance (decimate_gpu.cu:80-187): minimiser -A^-1 b and the reciprocal condition estimate.
__device__ float reduce_system(const float (*A)[3], const float* b, float* xyz) {
    float M[3][7];
    float normA = 0.f;
    for (int r = 0; r < 3; ++r) {
        float s = 0.f;
        for (int c = 0; c < 3; ++c) { M[r][c] = A[r][c]; M[r][4 + c] = r == c ? 1.f : 0.f; s += fabsf(A[r][c]); }
        M[r][3] = b[r];
        if (normA < s) normA = s;
    }
    const float tol = 2.220446049250313e-16f * 7 * normA;
    int i = 0, j = 0;
    while (i < 3 && j < 7) {
        float p = fabsf(M[i][j]);
        int k = i;
        for (int r = i + 1; r < 3; ++r) {
            const float q = fabsf(M[r][j]);
            if (p < q) { p = q; k = r; }
        }
        if (p <= tol) {
            for (int r = i; r < 3; ++r) M[r][j] = 0.f;
            ++j;
            continue;
        }
        for (int c = j; c < 7; ++c) { const float t = M[i][c]; M[i][c] = M[k][c]; M[k][c] = t; }
        const float piv = M[i][j];
        for (int c = j; c < 7; ++c) M[i][c] = M[i][c] / piv;
        for (int r = 0; r < 3; ++r) {
            if (r == i) continue;
            const float m = M[r][j];
            for (int c = j; c < 7; ++c) M[r][c] -= m * M[i][c];
        }
        ++i; ++j;
    }
    xyz[0] = -M[0][3]; xyz[1] = -M[1][3]; xyz[2] = -M[2][3];
    float normInv = 0.f;
    for (int r = 0; r < 3; ++r) {
        const float s = fabsf(M[r][4]) + fabsf(M[r][5]) + fabsf(M[r][6]);
        if (normInv < s) normInv = s;
    }
    return 1 / (normA * normInv);
}

// sortable image of a cost: ascending unsigned order = ascending cost, -0 = +0, every NaN last
__device__ __forceinline__ uint32_t cost_key(float c) {
    if (c != c) return 0xffffffffu;
    if (c == 0.f) c = 0.f;
    const uint32_t u = __float_as_uint(c);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// one thread per candidate (decimate_gpu.cu:378-416); sort key = (sample, cost), payload = candidate
__global__ void edge_cost_kernel(int64_t nu, int64_t Nv, int D, int B, const int32_t* __restrict__ nvIn,
                                 const int32_t* __restrict__ ulo, const int32_t* __restrict__ uhi,
                                 const float* __restrict__ vertex, const float* __restrict__ Qv,
                                 uint64_t* __restrict__ key, uint32_t* __restrict__ val, float* __restrict__ costOut) {
    const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= nu) return;
    const int vi = ulo[u], vj = uhi[u];
    float q[10];
#pragma unroll
    for (int t = 0; t < 10; ++t) q[t] = Qv[10 * (int64_t)vi + t] + Qv[10 * (int64_t)vj + t];
    const float A[3][3] = {{q[0], q[1], q[2]}, {q[1], q[3], q[4]}, {q[2], q[4], q[5]}};
    const float b[3] = {q[6], q[7], q[8]};
    float x[3], cost;
    const float rc = reduce_system(A, b, x);
    if (rc > 1e-6f) cost = quadric_error(x, A, b, q[9]);
    else {
        const float ei = quadric_error(vertex + (int64_t)vi * D, A, b, q[9]);
        const float ej = quadric_error(vertex + (int64_t)vj * D, A, b, q[9]);
        cost = ei < ej ? ei : ej;
    }
    key[u] = ((uint64_t)sample_of(vi, nvIn, B) << 32) | cost_key(cost);
    val[u] = (uint32_t)u;
    if (costOut) costOut[u] = cost;
}

// first candidate of every sample (candidates are in ascending lower-vertex order)
__global__ void segment_kernel(int B, int64_t nu, const int32_t* __restrict__ nvIn, const int32_t* __restrict__ ulo,
                               int32_t* __restrict__ segstart) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s > B) return;
    const int bound = s == 0 ? 0 : nvIn[s - 1];
    int64_t lo = 0, hi = nu;
    while (lo < hi) { const int64_t mid = (lo + hi) >> 1; if (ulo[mid] < bound) lo = mid + 1; else hi = mid; }
    segstart[s] = (int32_t)lo;
}

__global__ void rank_kernel(int64_t nu, const uint32_t* __restrict__ sorted_u, uint32_t* __restrict__ rank) {
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r < nu) rank[sorted_u[r]] = (uint32_t)r;
}

// ---------------------------------------------------------------------------- matching
// live list of the first sweep: candidates of samples that still have vertices to remove
__global__ void match_init_kernel(int64_t nu, int B, const int32_t* __restrict__ nvIn, const int32_t* __restrict__ want,
                                  const int32_t* __restrict__ ulo, const int32_t* __restrict__ uhi,
                                  uint32_t* __restrict__ list, int32_t* __restrict__ count) {
    for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x; i0 < nu; i0 += (int64_t)gridDim.x * blockDim.x) {
        const int64_t u = i0 + threadIdx.x;
        bool take = false;
        if (u < nu) {
            const int lo = ulo[u], hi = uhi[u];
            const int s = sample_of(lo, nvIn, B);
            take = lo != hi && s < B && want[s] > 0;
        }
        warp_append(take, (uint32_t)u, list, count);
    }
}

// round, first half: every live edge posts its rank at both ends
__global__ void match_post_kernel(const uint32_t* __restrict__ list, const int32_t* __restrict__ count,
                                  int32_t* __restrict__ next_count, const int32_t* __restrict__ ulo,
                                  const int32_t* __restrict__ uhi, const uint32_t* __restrict__ rank,
                                  const uint8_t* __restrict__ covered, uint32_t* __restrict__ vmin) {
    const int n = *count;
    if (blockIdx.x == 0 && threadIdx.x == 0) *next_count = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const uint32_t u = list[i];
        const int lo = ulo[u], hi = uhi[u];
        if (covered[lo] | covered[hi]) continue;
        const uint32_t r = rank[u];
        atomicMin(&vmin[lo], r);
        atomicMin(&vmin[hi], r);
    }
}

// round, second half: an edge that holds the minimum at both ends is taken; edges with two
// free ends stay live and clear the slots of the other minimum array for the next round
__global__ void match_take_kernel(const uint32_t* __restrict__ list, const int32_t* __restrict__ count,
                                  uint32_t* __restrict__ next_list, int32_t* __restrict__ next_count,
                                  const int32_t* __restrict__ ulo, const int32_t* __restrict__ uhi,
                                  const uint32_t* __restrict__ rank, uint8_t* covered,
                                  const uint32_t* __restrict__ vmin, uint32_t* __restrict__ vmin_next,
                                  int32_t* __restrict__ mflag) {
    const int n = *count;
    for (int i0 = blockIdx.x * blockDim.x; i0 < n; i0 += gridDim.x * blockDim.x) {
        const int i = i0 + threadIdx.x;
        bool live = false;
        uint32_t u = 0;
        if (i < n) {
            u = list[i];
            const int lo = ulo[u], hi = uhi[u];
            const uint32_t r = rank[u];
            if (vmin[lo] == r && vmin[hi] == r) {
                mflag[r] = 1;
                covered[lo] = 1;
                covered[hi] = 1;
            } else if (!(covered[lo] | covered[hi])) {
                live = true;
                vmin_next[lo] = NO_RANK;
                vmin_next[hi] = NO_RANK;
            }
        }
        warp_append(live, u, next_list, next_count);
    }
}

// the same rounds for a short live list, by one block until the list is empty; every round
// takes at least the lowest-ranked live edge, so `count + 1` rounds bound the loop
constexpr int TAIL_THREADS = 1024;
constexpr int TAIL_LIMIT = 8192;
__global__ void __launch_bounds__(TAIL_THREADS)
match_tail_kernel(uint32_t* listA, uint32_t* listB, int32_t* countA, const int32_t* __restrict__ ulo,
                  const int32_t* __restrict__ uhi, const uint32_t* __restrict__ rank, uint8_t* covered,
                  uint32_t* vminA, uint32_t* vminB, int32_t* __restrict__ mflag, int32_t* __restrict__ rounds_out) {
    __shared__ int32_t next_n;
    uint32_t* list = listA;
    uint32_t* next = listB;
    uint32_t* vmin = vminA;
    uint32_t* vmin_next = vminB;
    int n = *countA;
    const int limit = n + 1;
    int rounds = 0;
    while (n > 0 && rounds < limit) {
        if (threadIdx.x == 0) next_n = 0;
        for (int i = threadIdx.x; i < n; i += TAIL_THREADS) {
            const uint32_t u = list[i];
            const int lo = ulo[u], hi = uhi[u];
            if (covered[lo] | covered[hi]) continue;
            const uint32_t r = rank[u];
            atomicMin(&vmin[lo], r);
            atomicMin(&vmin[hi], r);
        }
        __syncthreads();
        for (int i0 = 0; i0 < n; i0 += TAIL_THREADS) {
            const int i = i0 + threadIdx.x;
            bool live = false;
            uint32_t u = 0;
            if (i < n) {
                u = list[i];
                const int lo = ulo[u], hi = uhi[u];
                const uint32_t r = rank[u];
                if (vmin[lo] == r && vmin[hi] == r) {
                    mflag[r] = 1;
                    covered[lo] = 1;
                    covered[hi] = 1;
                } else if (!(covered[lo] | covered[hi])) {
                    live = true;
                    vmin_next[lo] = NO_RANK;
                    vmin_next[hi] = NO_RANK;
                }
            }
            warp_append(live, u, next, &next_n);
        }
        __syncthreads();
        n = next_n;
        __syncthreads();
        uint32_t* t = list; list = next; next = t;
        uint32_t* tv = vmin; vmin = vmin_next; vmin_next = tv;
        ++rounds;
    }
    if (threadIdx.x == 0) { *countA = n; *rounds_out = rounds; }
}

// matched edges per sample (prefix counts over ranks)
__global__ void segment_count_kernel(int B, const int32_t* __restrict__ segstart, const int32_t* __restrict__ scan,
                                     int32_t* __restrict__ per_sample) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < B) per_sample[s] = scan[segstart[s + 1]] - scan[segstart[s]];
}

// first sweep applied: the first want[s] matched edges of every sample in rank order
// (decimate_gpu.cu:568-584): the lower vertex is contracted into the higher one
__global__ void apply_matched_kernel(int64_t nu, int B, const int32_t* __restrict__ want, const int32_t* __restrict__ segstart,
                                     const uint64_t* __restrict__ skey, const uint32_t* __restrict__ sorted_u,
                                     const int32_t* __restrict__ mflag, const int32_t* __restrict__ mscan,
                                     const int32_t* __restrict__ ulo, const int32_t* __restrict__ uhi,
                                     int32_t* __restrict__ vtReplace) {
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= nu || !mflag[r]) return;
    const int s = (int)(skey[r] >> 32);
    if (s >= B) return;
    if (mscan[r] - mscan[segstart[s]] >= want[s]) return;
    const uint32_t u = sorted_u[r];
    const int lo = ulo[u], hi = uhi[u];
    vtReplace[lo] = -hi;
    atomicAdd(&vtReplace[hi], 1);
}

// second sweep (decimate_gpu.cu:586-612), only where the first one ran out of edges before it
// reached want[s]: an uncovered vertex joins through its lowest-ranked edge
__global__ void attach_post_kernel(int64_t nu, int B, const int32_t* __restrict__ nvIn, const int32_t* __restrict__ want,
                                   const int32_t* __restrict__ matched, const int32_t* __restrict__ ulo,
                                   const int32_t* __restrict__ uhi, const uint32_t* __restrict__ rank,
                                   const uint8_t* __restrict__ covered, uint32_t* __restrict__ vmin) {
    const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= nu) return;
    const int lo = ulo[u], hi = uhi[u];
    if (lo == hi) return;
    const int s = sample_of(lo, nvIn, B);
    if (s >= B || matched[s] >= want[s]) return;
    const int cl = covered[lo], ch = covered[hi];
    if (cl == ch) return;
    atomicMin(&vmin[cl ? hi : lo], rank[u]);
}

__global__ void attach_flag_kernel(int64_t nu, int B, const int32_t* __restrict__ nvIn, const int32_t* __restrict__ want,
                                   const int32_t* __restrict__ matched, const int32_t* __restrict__ ulo,
                                   const int32_t* __restrict__ uhi, const uint32_t* __restrict__ rank,
                                   const uint8_t* __restrict__ covered, const uint32_t* __restrict__ vmin,
                                   int32_t* __restrict__ aflag) {
    const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= nu) return;
    const int lo = ulo[u], hi = uhi[u];
    if (lo == hi) return;
    const int s = sample_of(lo, nvIn, B);
    if (s >= B || matched[s] >= want[s]) return;
    const int cl = covered[lo], ch = covered[hi];
    if (cl == ch) return;
    const uint32_t r = rank[u];
    if (vmin[cl ? hi : lo] == r) aflag[r] = 1;
}

__global__ void apply_attach_kernel(int64_t nu, int B, const int32_t* __restrict__ want, const int32_t* __restrict__ matched,
                                    const int32_t* __restrict__ segstart, const uint64_t* __restrict__ skey,
                                    const uint32_t* __restrict__ sorted_u, const int32_t* __restrict__ aflag,
                                    const int32_t* __restrict__ ascan, const int32_t* __restrict__ ulo,
                                    const int32_t* __restrict__ uhi, const uint8_t* __restrict__ covered,
                                    int32_t* vtReplace) {
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= nu || !aflag[r]) return;
    const int s = (int)(skey[r] >> 32);
    if (s >= B) return;
    if (ascan[r] - ascan[segstart[s]] >= want[s] - matched[s]) return;
    const uint32_t u = sorted_u[r];
    const int lo = ulo[u], hi = uhi[u];
    const int seed = covered[lo] ? lo : hi, joiner = covered[lo] ? hi : lo;
    const int rep = vtReplace[seed];
    const int root = rep < 0 ? -rep : seed;
    vtReplace[joiner] = -root;
    atomicAdd(&vtReplace[root], 1);
}

// -------------------------------------------------------------------- contraction, faces
__global__ void cluster_key_kernel(int64_t Nv, const int32_t* __restrict__ vtReplace, int32_t* __restrict__ key) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v < Nv) key[v] = vtReplace[v] < 0 ? -vtReplace[v] : -1;
}

// decimate_gpu.cu:403-441: a representative moves to the mean of its cluster, a vertex on its
// own keeps its row, a contracted vertex's row is zero
__global__ void contract_kernel(int64_t Nv, int D, const int32_t* __restrict__ vtReplace, const int32_t* __restrict__ rowptr,
                                const int32_t* __restrict__ members, const float* __restrict__ vertexIn,
                                float* __restrict__ vertexOut) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Nv * D) return;
    const int64_t v = i / D;
    const int t = (int)(i - v * D);
    const int rep = vtReplace[v];
    float out = 0.f;
    if (rep > 0) {
        float acc = 0.f;
        for (int p = rowptr[v]; p < rowptr[v + 1]; ++p) acc += vertexIn[(int64_t)members[p] * D + t];
        out = (acc + vertexIn[i]) / (rep + 1);
    } else if (rep == 0) {
        out = vertexIn[i];
    }
    vertexOut[i] = out;
}

// decimate_gpu.cu:444-507
__global__ void face_relabel_kernel(int64_t Nf, int B, const int32_t* __restrict__ mfIn, const int32_t* __restrict__ vtReplace,
                                    const int32_t* __restrict__ faceIn, int32_t* __restrict__ faceOut,
                                    uint8_t* __restrict__ isDegenerate, int32_t* __restrict__ kept, int32_t* __restrict__ mfOut) {
    for (int64_t f0 = (int64_t)blockIdx.x * blockDim.x; f0 < Nf; f0 += (int64_t)gridDim.x * blockDim.x) {
        const int64_t f = f0 + threadIdx.x;
        int s = -1 - (int)(threadIdx.x & 31);                   // lanes without a kept face: groups of one
        if (f < Nf) {
            int v[3];
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                v[c] = faceIn[3 * f + c];
                const int rep = vtReplace[v[c]];
                if (rep < 0) v[c] = -rep;
                faceOut[3 * f + c] = v[c];
            }
            const bool deg = v[0] == v[1] || v[0] == v[2] || v[1] == v[2];
            isDegenerate[f] = deg ? 1 : 0;
            if (!deg) {
                kept[v[0]] = 1; kept[v[1]] = 1; kept[v[2]] = 1;
                s = sample_of((int)f, mfIn, B);
                if (s > B - 1) s = B - 1;
            }
        }
        const unsigned m = __match_any_sync(0xffffffffu, s);
        if (s >= 0 && (int)(threadIdx.x & 31) == __ffs(m) - 1) atomicAdd(&mfOut[s], __popc(m));
    }
}

// decimate_gpu.cu:509-533: kept vertices are numbered in order, the others map to -1
__global__ void vertex_map_kernel(int64_t Nv, const int32_t* __restrict__ kept, const int32_t* __restrict__ kscan,
                                  int32_t* __restrict__ vtMap) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v < Nv) vtMap[v] = kept[v] ? kscan[v] : -1;
}

__global__ void sample_sizes_kernel(int B, const int32_t* __restrict__ nvIn, const int32_t* __restrict__ kscan,
                                    int32_t* __restrict__ nvOut) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < B) nvOut[s] = kscan[nvIn[s]] - kscan[s == 0 ? 0 : nvIn[s - 1]];
}

__global__ void face_update_kernel(int64_t Nf, const int32_t* __restrict__ vtMap, const uint8_t* __restrict__ isDegenerate,
                                   int32_t* __restrict__ faceOut) {
    const int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= Nf || isDegenerate[f]) return;
#pragma unroll
    for (int c = 0; c < 3; ++c) faceOut[3 * f + c] = vtMap[faceOut[3 * f + c]];
}

// ------------------------------------------------------------------------ cluster merge
// decimate_gpu.cu:750-812.  repB_work[vo] of a vertex B kept becomes its id in A; a vertex of A
// whose representative was contracted in B follows that contraction.
__global__ void merge_back_kernel(int64_t nvA, int64_t nvB, const int32_t* __restrict__ mapA, int32_t* __restrict__ repB_work) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= nvA) return;
    const int vo = mapA[v];
    if (vo >= 0 && vo < nvB && repB_work[vo] >= 0) repB_work[vo] = (int32_t)v;
}
__global__ void merge_follow_kernel(int64_t nvA, int64_t nvB, const int32_t* __restrict__ repA, const int32_t* __restrict__ mapA,
                                    const int32_t* __restrict__ repB_work, int32_t* repOut, int32_t* __restrict__ status) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= nvA) return;
    int64_t vi = v;
    if (repA[v] < 0) vi = -(int64_t)repA[v];
    if (vi >= nvA) { *status = PB200_EINDEX; return; }
    const int vo = mapA[vi];
    if (vo < 0) return;
    if (vo >= nvB) { *status = PB200_EINDEX; return; }
    const int rb = repB_work[vo];
    if (rb >= 0) return;
    const int64_t root_b = -(int64_t)rb;
    if (root_b >= nvB) { *status = PB200_EINDEX; return; }
    const int root_a = repB_work[root_b];
    if (root_a < 0 || root_a >= nvA) { *status = PB200_EINDEX; return; }
    repOut[v] = -root_a;
    atomicAdd(&repOut[root_a], 1);
}
__global__ void merge_map_kernel(int64_t nvA, int64_t nvB, const int32_t* __restrict__ mapA, const int32_t* __restrict__ mapB,
                                 int32_t* __restrict__ mapOut) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= nvA) return;
    const int vo = mapA[v];
    mapOut[v] = (vo >= 0 && vo < nvB) ? mapB[vo] : -1;
}

// ---------------------------------------------------------------------------- workspace
struct Carve {
    char* p;
    size_t used;
    explicit Carve(void* base) : p((char*)base), used(0) {}
    template <typename T> T* take(size_t n) {
        T* r = p ? (T*)(p + used) : nullptr;
        used += align_up(sizeof(T) * (n > 0 ? n : 1), 256);
        return r;
    }
};

struct Work {
    uint64_t *keyA, *keyB;
    uint32_t *valA, *valB, *rank, *listA, *listB, *vminA, *vminB;
    int32_t *hist, *tile_sum, *flag, *scan, *ulo, *uhi, *segstart, *matched, *counters, *rowptr, *entries, *key,
            *crowptr, *members, *kept, *kscan, *status;
    uint8_t *bnd, *covered;
    float* Q;
    void *csr_ws, *ccsr_ws;
    size_t csr_ws_bytes, ccsr_ws_bytes, total;
};

static Work carve(void* base, int64_t B, int64_t Nv, int64_t Nf) {
    Work w;
    Carve c(base);
    const size_t Ne = (size_t)(3 * Nf);
    const size_t nblocks = (size_t)ceil_div((int64_t)Ne, RS_TILE) + 1;
    w.keyA = c.take<uint64_t>(Ne);  w.keyB = c.take<uint64_t>(Ne);
    w.valA = c.take<uint32_t>(Ne);  w.valB = c.take<uint32_t>(Ne);
    w.rank = c.take<uint32_t>(Ne);  w.listA = c.take<uint32_t>(Ne);  w.listB = c.take<uint32_t>(Ne);
    w.vminA = c.take<uint32_t>((size_t)Nv);  w.vminB = c.take<uint32_t>((size_t)Nv);
    w.hist = c.take<int32_t>(256 * nblocks + 1);
    size_t longest = 256 * nblocks + 1;
    if (Ne + 1 > longest) longest = Ne + 1;
    if ((size_t)Nv + 1 > longest) longest = (size_t)Nv + 1;
    w.tile_sum = c.take<int32_t>(scan_tiles_for((int64_t)longest) + 1);
    w.flag = c.take<int32_t>(Ne + 1);  w.scan = c.take<int32_t>(Ne + 1);
    w.ulo = c.take<int32_t>(Ne);  w.uhi = c.take<int32_t>(Ne);
    w.segstart = c.take<int32_t>((size_t)B + 2);  w.matched = c.take<int32_t>((size_t)B + 1);
    w.counters = c.take<int32_t>(8);
    w.rowptr = c.take<int32_t>((size_t)Nv + 1);  w.entries = c.take<int32_t>(Ne);
    w.key = c.take<int32_t>((size_t)Nv);
    w.crowptr = c.take<int32_t>((size_t)Nv + 1);  w.members = c.take<int32_t>((size_t)Nv);
    w.kept = c.take<int32_t>((size_t)Nv + 1);  w.kscan = c.take<int32_t>((size_t)Nv + 1);
    w.status = c.take<int32_t>(4);
    w.bnd = c.take<uint8_t>(Ne);  w.covered = c.take<uint8_t>((size_t)Nv);
    w.Q = c.take<float>(10 * (size_t)Nv);
    w.csr_ws_bytes = pb200_vertex_csr_workspace_bytes(Nf, Nv);
    w.csr_ws = c.take<char>(w.csr_ws_bytes);
    w.ccsr_ws_bytes = pb200_cluster_csr_workspace_bytes(Nv, Nv);
    w.ccsr_ws = c.take<char>(w.ccsr_ws_bytes);
    w.total = c.used + 256;
    return w;
}

}  // namespace dec
}  // namespace pb

using namespace pb;
using namespace pb::dec;

extern "C" {

size_t pb200_mesh_simplify_workspace_bytes(int64_t B, int64_t Nv, int64_t Nf) {
    if (B < 0 || Nv < 0 || Nf < 0) return 0;
    return carve(nullptr, B, Nv, Nf).total;
}

int pb200_mesh_simplify(int useArea, float wgtBnd, int64_t B, int64_t D, int64_t Nv, int64_t Nf,
                        const int32_t* nvIn, const int32_t* mfIn, const int32_t* nv2Remove, const float* vertexIn,
                        const int32_t* faceIn, const float* planeIn, int32_t* nvOut, int32_t* mfOut, float* vertexOut,
                        int32_t* faceOut, int32_t* vtReplace, int32_t* vtMap, uint8_t* isDegenerate, float* edgeCost,
                        int64_t* info, void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(B >= 1 && B < (1 << 20) && D >= 3 && D <= 4096 && Nv >= 0 && Nf >= 0 && Nf < (1LL << 29) && Nv < (1LL << 30),
               PB200_EINVAL, "mesh_simplify: bad sizes");
    PB_REQUIRE(Nv > 0 || Nf == 0, PB200_EINVAL, "mesh_simplify: faces without vertices");
    PB_REQUIRE(nvIn && mfIn && nv2Remove && nvOut && mfOut, PB200_EINVAL, "mesh_simplify: null pointer");
    PB_REQUIRE(Nv == 0 || (vertexIn && vertexOut && vtReplace && vtMap), PB200_EINVAL, "mesh_simplify: null pointer");
    PB_REQUIRE(Nf == 0 || (faceIn && planeIn && faceOut && isDegenerate), PB200_EINVAL, "mesh_simplify: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_mesh_simplify_workspace_bytes(B, Nv, Nf), PB200_EWORKSPACE,
               "mesh_simplify: workspace too small");
    if (info) info[0] = info[1] = info[2] = info[3] = 0;

    // the per-sample running totals decide the segmentation: check them on the host (B values each)
    {
        int32_t* h = (int32_t*)malloc(sizeof(int32_t) * 2 * (size_t)B);
        PB_REQUIRE(h, PB200_EINVAL, "mesh_simplify: out of host memory");
        cudaError_t e = cudaMemcpyAsync(h, nvIn, sizeof(int32_t) * B, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(h + B, mfIn, sizeof(int32_t) * B, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        bool ok = e == cudaSuccess;
        for (int64_t s = 0; ok && s < B; ++s) {
            const int32_t pv = s ? h[s - 1] : 0, pf = s ? h[B + s - 1] : 0;
            ok = h[s] >= pv && h[B + s] >= pf;
        }
        ok = ok && h[B - 1] == Nv && h[2 * B - 1] == Nf;
        free(h);
        if (e != cudaSuccess) return cuda_fail(e, "mesh_simplify: reading the sample sizes");
        PB_REQUIRE(ok, PB200_EINVAL, "mesh_simplify: nvIn / mfIn must be non-decreasing running totals ending at Nv / Nf");
    }

    Work w = carve(workspace, B, Nv, Nf);
    const int64_t Ne = 3 * Nf;
    PB_CUDA(cudaMemsetAsync(w.status, 0, sizeof(int32_t) * 4, stream));
    PB_CUDA(cudaMemsetAsync(w.counters, 0, sizeof(int32_t) * 8, stream));
    PB_CUDA(cudaMemsetAsync(mfOut, 0, sizeof(int32_t) * B, stream));
    if (Nv > 0) {
        PB_CUDA(cudaMemsetAsync(vtReplace, 0, sizeof(int32_t) * Nv, stream));
        PB_CUDA(cudaMemsetAsync(w.covered, 0, (size_t)Nv, stream));
        PB_CUDA(cudaMemsetAsync(w.kept, 0, sizeof(int32_t) * (Nv + 1), stream));
        PB_CUDA(cudaMemsetAsync(w.vminA, 0xff, sizeof(uint32_t) * Nv, stream));
        PB_CUDA(cudaMemsetAsync(w.vminB, 0xff, sizeof(uint32_t) * Nv, stream));
    }

    int64_t nu = 0;
    uint64_t* skey = w.keyA;       // (sample, cost) keys in rank order, once sorted
    uint32_t* sorted_u = w.valA;   // candidate of every rank
    if (Ne > 0 && Nv > 0) {
        // ---- 1. edges
        const int vbits = bit_length(Nv);
        PB_LAUNCH("dec_edge_keys", edge_keys_kernel, (unsigned)ceil_div(Ne, 256), 256, 0, stream, Ne, Nv, vbits, faceIn,
                  w.keyA, w.valA, w.status);
        uint64_t *k = w.keyA, *kalt = w.keyB;
        uint32_t *v = w.valA, *valt = w.valB;
        int rc = radix_sort(k, kalt, v, valt, Ne, 2 * vbits, w.hist, w.tile_sum, stream);
        if (rc != PB200_OK) return rc;
        PB_LAUNCH("dec_edge_flags", edge_flags_kernel, (unsigned)ceil_div(Ne, 256), 256, 0, stream, Ne, Nv, vbits,
                  (const uint64_t*)k, (const uint32_t*)v, w.bnd, w.flag);
        rc = exclusive_scan(w.flag, Ne, w.scan, w.tile_sum, stream);
        if (rc != PB200_OK) return rc;
        PB_LAUNCH("dec_unique_write", unique_write_kernel, (unsigned)ceil_div(Ne, 256), 256, 0, stream, Ne, vbits,
                  (const uint64_t*)k, (const int32_t*)w.scan, w.ulo, w.uhi);
        int32_t h[2] = {0, 0};
        PB_CUDA(cudaMemcpyAsync(&h[0], w.scan + Ne, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
        PB_CUDA(cudaMemcpyAsync(&h[1], w.status, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
        PB_CUDA(cudaStreamSynchronize(stream));
        PB_REQUIRE(h[1] == 0, PB200_EINDEX, "mesh_simplify: face holds a vertex id outside [0, Nv)");
        nu = h[0];

        // ---- 2. quadrics
        rc = pb200_build_vertex_csr(Nf, Nv, Nv, faceIn, nullptr, w.rowptr, w.entries, w.status + 1, w.csr_ws, w.csr_ws_bytes,
                                    stream_);
        if (rc != PB200_OK) return rc;
        PB_LAUNCH("dec_vertex_quadric", vertex_quadric_kernel, (unsigned)ceil_div(Nv, 128), 128, 0, stream, Nv, (int)D,
                  useArea ? 1 : 0, wgtBnd, (const int32_t*)w.rowptr, (const int32_t*)w.entries, faceIn, planeIn, vertexIn,
                  (const uint8_t*)w.bnd, w.Q);
    }
    if (nu > 0) {
        // ---- 3. costs and ranks
        PB_LAUNCH("dec_edge_cost", edge_cost_kernel, (unsigned)ceil_div(nu, 128), 128, 0, stream, nu, Nv, (int)D, (int)B, nvIn,
                  (const int32_t*)w.ulo, (const int32_t*)w.uhi, vertexIn, (const float*)w.Q, w.keyA, w.valA, edgeCost);
        uint64_t *k = w.keyA, *kalt = w.keyB;
        uint32_t *v = w.valA, *valt = w.valB;
        int rc = radix_sort(k, kalt, v, valt, nu, 32 + bit_length(B), w.hist, w.tile_sum, stream);
        if (rc != PB200_OK) return rc;
        skey = k; sorted_u = v;
        PB_LAUNCH("dec_rank", rank_kernel, (unsigned)ceil_div(nu, 256), 256, 0, stream, nu, (const uint32_t*)sorted_u, w.rank);
        PB_LAUNCH("dec_segments", segment_kernel, (unsigned)ceil_div(B + 1, 128), 128, 0, stream, (int)B, nu, nvIn,
                  (const int32_t*)w.ulo, w.segstart);

        // ---- 4. first sweep as parallel rounds
        PB_CUDA(cudaMemsetAsync(w.flag, 0, sizeof(int32_t) * (nu + 1), stream));
        int32_t* count[2] = {w.counters, w.counters + 1};
        uint32_t* list[2] = {w.listA, w.listB};
        uint32_t* vmin[2] = {w.vminA, w.vminB};
        const int grid = 4 * sm_count();
        PB_LAUNCH("dec_match_init", match_init_kernel, grid, 256, 0, stream, nu, (int)B, nvIn, nv2Remove,
                  (const int32_t*)w.ulo, (const int32_t*)w.uhi, list[0], count[0]);
        int cur = 0;
        int32_t live = 0;
        int64_t rounds = 0;
        PB_CUDA(cudaMemcpyAsync(&live, count[0], sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
        PB_CUDA(cudaStreamSynchronize(stream));
        while (live > TAIL_LIMIT) {
            for (int r = 0; r < 4; ++r) {
                PB_LAUNCH("dec_match_post", match_post_kernel, grid, 256, 0, stream, (const uint32_t*)list[cur],
                          (const int32_t*)count[cur], count[cur ^ 1], (const int32_t*)w.ulo, (const int32_t*)w.uhi,
                          (const uint32_t*)w.rank, (const uint8_t*)w.covered, vmin[cur]);
                PB_LAUNCH("dec_match_take", match_take_kernel, grid, 256, 0, stream, (const uint32_t*)list[cur],
                          (const int32_t*)count[cur], list[cur ^ 1], count[cur ^ 1], (const int32_t*)w.ulo,
                          (const int32_t*)w.uhi, (const uint32_t*)w.rank, w.covered, (const uint32_t*)vmin[cur],
                          vmin[cur ^ 1], w.flag);
                cur ^= 1;
                ++rounds;
            }
            PB_CUDA(cudaMemcpyAsync(&live, count[cur], sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
            PB_CUDA(cudaStreamSynchronize(stream));
        }
        if (info) { info[1] = rounds; info[2] = live; }
        if (live > 0) {
            PB_LAUNCH("dec_match_tail", match_tail_kernel, 1, TAIL_THREADS, 0, stream, list[cur], list[cur ^ 1], count[cur],
                      (const int32_t*)w.ulo, (const int32_t*)w.uhi, (const uint32_t*)w.rank, w.covered, vmin[cur],
                      vmin[cur ^ 1], w.flag, w.counters + 2);
        }
        int rc2 = exclusive_scan(w.flag, nu, w.scan, w.tile_sum, stream);
        if (rc2 != PB200_OK) return rc2;
        PB_LAUNCH("dec_segment_count", segment_count_kernel, (unsigned)ceil_div(B, 128), 128, 0, stream, (int)B,
                  (const int32_t*)w.segstart, (const int32_t*)w.scan, w.matched);
        PB_LAUNCH("dec_apply_matched", apply_matched_kernel, (unsigned)ceil_div(nu, 256), 256, 0, stream, nu, (int)B, nv2Remove,
                  (const int32_t*)w.segstart, (const uint64_t*)skey, (const uint32_t*)sorted_u, (const int32_t*)w.flag,
                  (const int32_t*)w.scan, (const int32_t*)w.ulo, (const int32_t*)w.uhi, vtReplace);

        // ---- 5. second sweep
        PB_CUDA(cudaMemsetAsync(w.vminA, 0xff, sizeof(uint32_t) * Nv, stream));
        PB_CUDA(cudaMemsetAsync(w.flag, 0, sizeof(int32_t) * (nu + 1), stream));
        PB_LAUNCH("dec_attach_post", attach_post_kernel, (unsigned)ceil_div(nu, 256), 256, 0, stream, nu, (int)B, nvIn, nv2Remove,
                  (const int32_t*)w.matched, (const int32_t*)w.ulo, (const int32_t*)w.uhi, (const uint32_t*)w.rank,
                  (const uint8_t*)w.covered, w.vminA);
        PB_LAUNCH("dec_attach_flag", attach_flag_kernel, (unsigned)ceil_div(nu, 256), 256, 0, stream, nu, (int)B, nvIn, nv2Remove,
                  (const int32_t*)w.matched, (const int32_t*)w.ulo, (const int32_t*)w.uhi, (const uint32_t*)w.rank,
                  (const uint8_t*)w.covered, (const uint32_t*)w.vminA, w.flag);
        rc2 = exclusive_scan(w.flag, nu, w.scan, w.tile_sum, stream);
        if (rc2 != PB200_OK) return rc2;
        PB_LAUNCH("dec_apply_attach", apply_attach_kernel, (unsigned)ceil_div(nu, 256), 256, 0, stream, nu, (int)B, nv2Remove,
                  (const int32_t*)w.matched, (const int32_t*)w.segstart, (const uint64_t*)skey, (const uint32_t*)sorted_u,
                  (const int32_t*)w.flag, (const int32_t*)w.scan, (const int32_t*)w.ulo, (const int32_t*)w.uhi,
                  (const uint8_t*)w.covered, vtReplace);
    }
    if (info) info[0] = nu;

    // ---- 6. contraction, faces, vertex map
    if (Nv > 0) {
        PB_LAUNCH("dec_cluster_key", cluster_key_kernel, (unsigned)ceil_div(Nv, 256), 256, 0, stream, Nv,
                  (const int32_t*)vtReplace, w.key);
        int rc = pb200_build_key_csr(Nv, Nv, w.key, 1, w.crowptr, w.members, w.status + 2, w.ccsr_ws, w.ccsr_ws_bytes, stream_);
        if (rc != PB200_OK) return rc;
        PB_LAUNCH("dec_contract", contract_kernel, (unsigned)ceil_div(Nv * D, 256), 256, 0, stream, Nv, (int)D,
                  (const int32_t*)vtReplace, (const int32_t*)w.crowptr, (const int32_t*)w.members, vertexIn, vertexOut);
    }
    if (Nf > 0)
        PB_LAUNCH("dec_face_relabel", face_relabel_kernel, 4 * sm_count(), 256, 0, stream, Nf, (int)B, mfIn,
                  (const int32_t*)vtReplace, faceIn, faceOut, isDegenerate, w.kept, mfOut);
    {
        int rc = exclusive_scan(w.kept, Nv, w.kscan, w.tile_sum, stream);
        if (rc != PB200_OK) return rc;
        if (Nv > 0)
            PB_LAUNCH("dec_vertex_map", vertex_map_kernel, (unsigned)ceil_div(Nv, 256), 256, 0, stream, Nv,
                      (const int32_t*)w.kept, (const int32_t*)w.kscan, vtMap);
        PB_LAUNCH("dec_sample_sizes", sample_sizes_kernel, (unsigned)ceil_div(B, 128), 128, 0, stream, (int)B, nvIn,
                  (const int32_t*)w.kscan, nvOut);
    }
    if (Nf > 0)
        PB_LAUNCH("dec_face_update", face_update_kernel, (unsigned)ceil_div(Nf, 256), 256, 0, stream, Nf,
                  (const int32_t*)vtMap, (const uint8_t*)isDegenerate, faceOut);
    return PB200_OK;
}

int pb200_combine_clusters(int64_t nvA, int64_t nvB, const int32_t* repA, const int32_t* mapA, const int32_t* repB,
                           const int32_t* mapB, int32_t* repOut, int32_t* mapOut, int32_t* status, void* workspace,
                           size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(nvA >= 0 && nvB >= 0 && nvA < (1LL << 31) - 1 && nvB < (1LL << 31) - 1, PB200_EINVAL,
               "combine_clusters: bad sizes");
    PB_REQUIRE(status && (nvA == 0 || (repA && mapA && repOut && mapOut)) && (nvB == 0 || (repB && mapB)), PB200_EINVAL,
               "combine_clusters: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= sizeof(int32_t) * (size_t)(nvB + 1), PB200_EWORKSPACE,
               "combine_clusters: workspace too small");
    PB_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    if (nvA == 0) return PB200_OK;
    int32_t* rb = (int32_t*)workspace;
    if (nvB > 0) PB_CUDA(cudaMemcpyAsync(rb, repB, sizeof(int32_t) * nvB, cudaMemcpyDeviceToDevice, stream));
    PB_CUDA(cudaMemcpyAsync(repOut, repA, sizeof(int32_t) * nvA, cudaMemcpyDeviceToDevice, stream));
    const unsigned grid = (unsigned)ceil_div(nvA, 256);
    PB_LAUNCH("dec_merge_back", merge_back_kernel, grid, 256, 0, stream, nvA, nvB, mapA, rb);
    PB_LAUNCH("dec_merge_follow", merge_follow_kernel, grid, 256, 0, stream, nvA, nvB, repA, mapA, (const int32_t*)rb, repOut,
              status);
    PB_LAUNCH("dec_merge_map", merge_map_kernel, grid, 256, 0, stream, nvA, nvB, mapA, mapB, mapOut);
    return PB200_OK;
}

}  // extern "C"

// Adjacency: per-vertex incident-face counts, the vertex -> (face, corner) CSR that every
// scatter-shaped kernel pulls through, triangle geometry, and row expansion by sample
// counts.  All integer work; results are bit-exact and independent of scheduling.
#include "common.cuh"
#include "sph_core.cuh"

namespace pb {

// ---------------------------------------------------------------- counting / validation
// One thread per face corner.  Out-of-range ids are reported through `status` and the
// corner is skipped, so no kernel downstream ever dereferences a bad index.
__global__ void corner_count_kernel(int64_t ncorner, int64_t NvIn, int64_t NvOut,
                                    const int32_t* __restrict__ face, const int32_t* __restrict__ vtMap,
                                    int32_t* __restrict__ cnt, int32_t* __restrict__ status) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ncorner) return;
    int vi = face[i];
    if (vi < 0 || vi >= NvIn) { if (status) *status = PB200_EINDEX; return; }
    int vo = vtMap ? vtMap[vi] : vi;
    if (vo >= NvOut || vo < -1) { if (status) *status = PB200_EINDEX; return; }
    if (vo >= 0) atomicAdd(&cnt[vo], 1);
}

// ------------------------------------------------------------------------ exclusive scan
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

__global__ void scan_tiles_kernel(const int32_t* __restrict__ in, int64_t n, int32_t* __restrict__ out,
                                  int32_t* __restrict__ tile_sum) {
    __shared__ int32_t warp_tot[SCAN_THREADS / 32];
    int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    int32_t v[SCAN_ITEMS];
    int32_t run = 0;
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS; ++j) {
        int32_t x = (base + j < n) ? in[base + j] : 0;
        v[j] = run;
        run += x;
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int32_t inc = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int32_t warp_off = 0;
    for (int w = 0; w < warp; ++w) warp_off += warp_tot[w];
    int32_t excl = warp_off + inc - run;
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS; ++j)
        if (base + j < n) out[base + j] = excl + v[j];
    if (threadIdx.x == SCAN_THREADS - 1) tile_sum[blockIdx.x] = warp_off + inc;
}

__global__ void scan_tile_sums_kernel(int32_t* __restrict__ tile_sum, int ntiles, int32_t* __restrict__ total_out) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int32_t run = 0;
    for (int t = 0; t < ntiles; ++t) { int32_t x = tile_sum[t]; tile_sum[t] = run; run += x; }
    *total_out = run;
}

__global__ void scan_finish_kernel(int32_t* __restrict__ rowptr, int64_t n, const int32_t* __restrict__ tile_off,
                                   int32_t* __restrict__ cursor) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int32_t v = rowptr[i] + tile_off[i / SCAN_TILE];
    rowptr[i] = v;
    cursor[i] = v;
}

// -------------------------------------------------------------------------------- fill
__global__ void corner_fill_kernel(int64_t ncorner, int64_t NvIn, int64_t NvOut,
                                   const int32_t* __restrict__ face, const int32_t* __restrict__ vtMap,
                                   int32_t* __restrict__ cursor, int32_t* __restrict__ entries) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ncorner) return;
    int vi = face[i];
    if (vi < 0 || vi >= NvIn) return;
    int vo = vtMap ? vtMap[vi] : vi;
    if (vo >= NvOut || vo < 0) return;
    int32_t pos = atomicAdd(&cursor[vo], 1);
    int64_t f = i / 3;
    entries[pos] = (int32_t)((f << 2) | (i - 3 * f));
}

// --------------------------------------------------------------------- vertex clusters
// Decimation encodes clusters as (picasso/mesh/pi_modules/decimate.py:23-28): vtReplace[v] < 0 names
// the representative -vtReplace[v] a contracted vertex merged into; the representative holds the
// cluster size minus one (0 for a singleton); vtMap[representative] is the coarse vertex id, -1 for
// contracted or dropped vertices.  key[v] = coarse id of v's cluster, or -1.
__device__ __forceinline__ int cluster_key(int64_t v, int64_t NvIn, int64_t NvOut, const int32_t* __restrict__ vtReplace,
                                           const int32_t* __restrict__ vtMap, bool* bad) {
    int rep = vtReplace[v];
    int64_t m = rep < 0 ? -(int64_t)rep : v;
    if (m >= NvIn) { *bad = true; return -1; }
    int vo = vtMap[m];
    if (vo >= NvOut || vo < -1) { *bad = true; return -1; }
    return vo;
}

__global__ void cluster_count_kernel(int64_t NvIn, int64_t NvOut, const int32_t* __restrict__ vtReplace,
                                     const int32_t* __restrict__ vtMap, int32_t* __restrict__ key,
                                     int32_t* __restrict__ cnt, int32_t* __restrict__ status) {
    int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= NvIn) return;
    bool bad = false;
    int vo = cluster_key(v, NvIn, NvOut, vtReplace, vtMap, &bad);
    if (bad) *status = PB200_EINDEX;
    key[v] = vo;
    if (vo >= 0) atomicAdd(&cnt[vo], 1);
}

// generic grouping: item i belongs to row key[i * stride] (-1 = no row)
__global__ void key_count_kernel(int64_t N, int64_t NvOut, const int32_t* __restrict__ key, int stride,
                                 int32_t* __restrict__ cnt, int32_t* __restrict__ status) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int k = key[i * stride];
    if (k >= NvOut || k < -1) { *status = PB200_EINDEX; return; }
    if (k >= 0) atomicAdd(&cnt[k], 1);
}

__global__ void key_fill_kernel(int64_t N, int64_t NvOut, const int32_t* __restrict__ key, int stride,
                                int32_t* __restrict__ cursor, int32_t* __restrict__ members) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int k = key[i * stride];
    if (k >= 0 && k < NvOut) members[atomicAdd(&cursor[k], 1)] = (int32_t)i;
}

__global__ void cluster_fill_kernel(int64_t NvIn, const int32_t* __restrict__ key, int32_t* __restrict__ cursor,
                                    int32_t* __restrict__ members) {
    int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= NvIn) return;
    int vo = key[v];
    if (vo >= 0) members[atomicAdd(&cursor[vo], 1)] = (int32_t)v;
}

// Rows come out of the atomic fill in arbitrary order; sorting each row ascending makes
// the CSR (and every reduction that walks it) independent of scheduling.
constexpr int SHORT_ROW = 32;

__global__ void sort_short_rows_kernel(int64_t nrows, const int32_t* __restrict__ rowptr,
                                       int32_t* __restrict__ entries, int32_t* __restrict__ long_rows,
                                       int32_t* __restrict__ n_long) {
    int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= nrows) return;
    int beg = rowptr[v], end = rowptr[v + 1];
    int deg = end - beg;
    if (deg <= 1) return;
    if (deg > SHORT_ROW) { long_rows[atomicAdd(n_long, 1)] = (int32_t)v; return; }
    int32_t a[SHORT_ROW];
    for (int i = 0; i < deg; ++i) a[i] = entries[beg + i];
    for (int i = 1; i < deg; ++i) {
        int32_t x = a[i];
        int j = i - 1;
        while (j >= 0 && a[j] > x) { a[j + 1] = a[j]; --j; }
        a[j + 1] = x;
    }
    for (int i = 0; i < deg; ++i) entries[beg + i] = a[i];
}

// One warp per long row: every element finds its rank by counting smaller elements
// (all entries of a row are distinct), writes itself to that slot of `tmp`, then the
// row is copied back.
__global__ void sort_long_rows_kernel(const int32_t* __restrict__ rowptr, int32_t* __restrict__ entries,
                                      const int32_t* __restrict__ long_rows, const int32_t* __restrict__ n_long,
                                      int32_t* __restrict__ tmp) {
    int lane = threadIdx.x & 31;
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int nwarps = (gridDim.x * blockDim.x) >> 5;
    int total = *n_long;
    for (int r = warp; r < total; r += nwarps) {
        int v = long_rows[r];
        int beg = rowptr[v], end = rowptr[v + 1];
        for (int i = beg + lane; i < end; i += 32) {
            int32_t x = entries[i];
            int rank = 0;
            for (int j = beg; j < end; ++j) rank += (entries[j] < x);
            tmp[beg + rank] = x;
        }
        __syncwarp();
        for (int i = beg + lane; i < end; i += 32) entries[i] = tmp[i];
        __syncwarp();
    }
}

// ----------------------------------------------------------------------------- geometry
__global__ void triangle_geometry_kernel(int64_t Nf, int64_t Nv, int vstride, const float* __restrict__ vertex,
                                         const int32_t* __restrict__ face, float* __restrict__ geom) {
    int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= Nf) return;
    int i0 = face[3 * f], i1 = face[3 * f + 1], i2 = face[3 * f + 2];
    float* g = geom + f * 5;
    if (i0 < 0 || i1 < 0 || i2 < 0 || i0 >= Nv || i1 >= Nv || i2 >= Nv) {
        g[0] = g[1] = g[2] = g[3] = g[4] = 0.f;
        return;
    }
    const float* a = vertex + (int64_t)i0 * vstride;
    const float* b = vertex + (int64_t)i1 * vstride;
    const float* c = vertex + (int64_t)i2 * vstride;
    float ax = a[0], ay = a[1], az = a[2];
    float ux = b[0] - ax, uy = b[1] - ay, uz = b[2] - az;
    float vx = c[0] - ax, vy = c[1] - ay, vz = c[2] - az;
    float nx = __fsub_rn(__fmul_rn(uy, vz), __fmul_rn(uz, vy));
    float ny = __fsub_rn(__fmul_rn(uz, vx), __fmul_rn(ux, vz));
    float nz = __fsub_rn(__fmul_rn(ux, vy), __fmul_rn(uy, vx));
    float l2 = sqrtf(__fadd_rn(__fadd_rn(__fmul_rn(nx, nx), __fmul_rn(ny, ny)), __fmul_rn(nz, nz)));
    float den = l2 + 1e-10f;
    nx = nx / den; ny = ny / den; nz = nz / den;
    g[0] = nx; g[1] = ny; g[2] = nz;
    g[3] = -__fadd_rn(__fadd_rn(__fmul_rn(nx, ax), __fmul_rn(ny, ay)), __fmul_rn(nz, az));
    g[4] = l2 / 2.f;
}

// ------------------------------------------------------------- fused per-level preparation
// One pass over the faces of a mesh level: triangle geometry (normal, plane intercept, area), the
// optionally re-oriented normal (flipped when it points away from the origin as viewpoint,
// reference: picasso/networks/scene_seg.py:117-124), its spherical-harmonic coefficients, and the
// per-vertex corner counts that seed the vertex CSR (= the reference's nfCount).  The vertex rows of
// a face are read once for all of it; the K coefficients are staged through shared memory so the
// global store is coalesced.
constexpr int PREP_BLOCK = 128;

__global__ void __launch_bounds__(PREP_BLOCK)
level_prepare_kernel(int64_t Nf, int64_t NvIn, int64_t NvOut, int vstride, const float* __restrict__ vertex,
                     const int32_t* __restrict__ face, const int32_t* __restrict__ vtMap, int L, int orient, SphConst cst,
                     float* __restrict__ geom, float* __restrict__ normal_out, float* __restrict__ coeff,
                     int32_t* __restrict__ cnt, int32_t* __restrict__ status) {
    extern __shared__ float stage[];            // [PREP_BLOCK][K+1]
    const int K = (L + 1) * (L + 1), KP = K + 1;
    const int64_t base = (int64_t)blockIdx.x * PREP_BLOCK;
    const int64_t f = base + threadIdx.x;
    if (f < Nf) {
        const int i0 = face[3 * f], i1 = face[3 * f + 1], i2 = face[3 * f + 2];
        float nx = 0.f, ny = 0.f, nz = 0.f, dd = 0.f, area = 0.f;
        const bool ok = !(i0 < 0 || i1 < 0 || i2 < 0 || i0 >= NvIn || i1 >= NvIn || i2 >= NvIn);
        if (ok) {
            const float* a = vertex + (int64_t)i0 * vstride;
            const float* b = vertex + (int64_t)i1 * vstride;
            const float* c = vertex + (int64_t)i2 * vstride;
            const float ax = a[0], ay = a[1], az = a[2];
            const float bx = b[0], by = b[1], bz = b[2], cx = c[0], cy = c[1], cz = c[2];
            const float ux = bx - ax, uy = by - ay, uz = bz - az;
            const float vx = cx - ax, vy = cy - ay, vz = cz - az;
            nx = __fsub_rn(__fmul_rn(uy, vz), __fmul_rn(uz, vy));
            ny = __fsub_rn(__fmul_rn(uz, vx), __fmul_rn(ux, vz));
            nz = __fsub_rn(__fmul_rn(ux, vy), __fmul_rn(uy, vx));
            const float l2 = sqrtf(__fadd_rn(__fadd_rn(__fmul_rn(nx, nx), __fmul_rn(ny, ny)), __fmul_rn(nz, nz)));
            const float den = l2 + 1e-10f;
            nx = nx / den; ny = ny / den; nz = nz / den;
            dd = -__fadd_rn(__fadd_rn(__fmul_rn(nx, ax), __fmul_rn(ny, ay)), __fmul_rn(nz, az));
            area = l2 / 2.f;
            if (geom) { float* g = geom + f * 5; g[0] = nx; g[1] = ny; g[2] = nz; g[3] = dd; g[4] = area; }
            if (orient) {
                // sign(sum(-center * normal)) with every value above -1 set to +1: only a strictly
                // negative dot product flips the normal
                const float mx = __fadd_rn(__fadd_rn(ax, bx), cx) / 3.f, my = __fadd_rn(__fadd_rn(ay, by), cy) / 3.f,
                            mz = __fadd_rn(__fadd_rn(az, bz), cz) / 3.f;
                const float dot = __fadd_rn(__fadd_rn(__fmul_rn(-mx, nx), __fmul_rn(-my, ny)), __fmul_rn(-mz, nz));
                if (dot < 0.f) { nx = -nx; ny = -ny; nz = -nz; }
            }
        } else {
            if (status) *status = PB200_EINDEX;
            if (geom) { float* g = geom + f * 5; g[0] = g[1] = g[2] = g[3] = g[4] = 0.f; }
        }
        if (normal_out) { normal_out[3 * f] = nx; normal_out[3 * f + 1] = ny; normal_out[3 * f + 2] = nz; }
        sph_eval(nx, ny, nz, L, cst.c, stage + threadIdx.x * KP);
        if (cnt && ok) {
            const int vi[3] = {i0, i1, i2};
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int vo = vtMap ? vtMap[vi[j]] : vi[j];
                if (vo >= NvOut || vo < -1) { if (status) *status = PB200_EINDEX; }
                else if (vo >= 0) atomicAdd(&cnt[vo], 1);
            }
        }
    }
    __syncthreads();
    const int64_t nfb = Nf - base < PREP_BLOCK ? Nf - base : PREP_BLOCK;
    float* dst = coeff + base * K;
    for (int64_t j = threadIdx.x; j < nfb * K; j += PREP_BLOCK) {
        const int p = (int)(j / K), k = (int)(j - (int64_t)p * K);
        dst[j] = stage[p * KP + k];
    }
}

__global__ void copy_counts_kernel(int64_t n, const int32_t* __restrict__ src, int32_t* __restrict__ dst) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[i];
}

// ------------------------------------------------------------------------ row expansion
// out[f] = mean of the rows of face f's samples, added in ascending order (0 for a face without samples)
template <int VEC>
__global__ void face_mean_rows_kernel(int64_t Nf, int64_t NiK, int CVn, const float* __restrict__ rows,
                                      const int32_t* __restrict__ cum, float* __restrict__ out) {
    int64_t total = Nf * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t f = i / CVn;
        int c = (int)(i - f * CVn);
        int k0 = f > 0 ? __ldg(cum + f - 1) : 0, k1 = __ldg(cum + f);
        if (k0 < 0) k0 = 0;
        if (k1 > NiK) k1 = (int)NiK;
        const float inv = k1 > k0 ? 1.f / (float)(k1 - k0) : 0.f;
        if (VEC == 4) {
            float4 acc = zero4();
            for (int k = k0; k < k1; ++k) add4(acc, __ldg(reinterpret_cast<const float4*>(rows) + (int64_t)k * CVn + c));
            reinterpret_cast<float4*>(out)[i] = scale4(acc, inv);
        } else {
            float acc = 0.f;
            for (int k = k0; k < k1; ++k) acc += __ldg(rows + (int64_t)k * CVn + c);
            out[i] = acc * inv;
        }
    }
}


// The samples of face f are rows cum[f-1] .. cum[f]-1 (cum = inclusive running count).
// forward: one item per (face, channel group); the face's row is read once and written to
// each of its samples (rows k0..k1-1, contiguous in the output)
template <int VEC>
__global__ void expand_rows_fwd_kernel(int64_t Nf, int64_t NiK, int CVn, const float* __restrict__ in,
                                       const int32_t* __restrict__ cum, float* __restrict__ out) {
    int64_t total = Nf * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t f = i / CVn;
        int c = (int)(i - f * CVn);
        int k0 = f > 0 ? __ldg(cum + f - 1) : 0, k1 = __ldg(cum + f);
        if (k0 < 0) k0 = 0;
        if (k1 > NiK) k1 = (int)NiK;
        if (VEC == 4) {
            float4 v = __ldg(reinterpret_cast<const float4*>(in) + i);
            for (int k = k0; k < k1; ++k) __stcs(reinterpret_cast<float4*>(out) + (int64_t)k * CVn + c, v);
        } else {
            float v = in[i];
            for (int k = k0; k < k1; ++k) out[(int64_t)k * CVn + c] = v;
        }
    }
}

template <int VEC>
__global__ void expand_rows_bwd_kernel(int64_t Nf, int64_t NiK, int CVn, const float* __restrict__ gout,
                                       const int32_t* __restrict__ cum, float* __restrict__ gin) {
    int64_t total = Nf * CVn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t f = i / CVn;
        int c = (int)(i - f * CVn);
        int k0 = f > 0 ? cum[f - 1] : 0, k1 = cum[f];
        if (k0 < 0) k0 = 0;
        if (k1 > NiK) k1 = (int)NiK;
        if (VEC == 4) {
            float4 acc = zero4();
            for (int k = k0; k < k1; ++k)
                add4(acc, __ldcs(reinterpret_cast<const float4*>(gout) + (int64_t)k * CVn + c));
            reinterpret_cast<float4*>(gin)[i] = acc;
        } else {
            float acc = 0.f;
            for (int k = k0; k < k1; ++k) acc += gout[(int64_t)k * CVn + c];
            gin[i] = acc;
        }
    }
}

// numInterior must be a non-decreasing running count inside [0, NiK] that ends at NiK
__global__ void check_running_count_kernel(int64_t Nf, int64_t NiK, const int32_t* __restrict__ cum,
                                           int32_t* __restrict__ status) {
    bool bad = false;
    for (int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; f < Nf; f += (int64_t)gridDim.x * blockDim.x) {
        const int k1 = cum[f], k0 = f > 0 ? cum[f - 1] : 0;
        if (k0 < 0 || k1 < k0 || k1 > NiK || (f == Nf - 1 && k1 != NiK)) bad = true;
    }
    if (bad) *status = PB200_EINDEX;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// second half of the vertex-CSR build: exclusive scan of the corner counts in cursor[0..NvOut]
// (last slot 0) -> rowptr, atomic-cursor fill, per-row sort
static int finish_vertex_csr(int64_t Nf, int64_t NvIn, int64_t NvOut, const int32_t* face, const int32_t* vtMap,
                             int32_t* rowptr, int32_t* entries, int32_t* cursor, int32_t* tile_sum, int32_t* long_rows,
                             int32_t* tmp, int32_t* n_long, cudaStream_t stream) {
    const int ntiles = (int)ceil_div(NvOut + 1, SCAN_TILE);
    PB_LAUNCH("scan_tiles", scan_tiles_kernel, ntiles, SCAN_THREADS, 0, stream,
              (const int32_t*)cursor, NvOut + 1, rowptr, tile_sum);
    PB_LAUNCH("scan_tile_sums", scan_tile_sums_kernel, 1, 32, 0, stream, tile_sum, ntiles, tile_sum + ntiles);
    PB_LAUNCH("scan_finish", scan_finish_kernel, (unsigned)ceil_div(NvOut + 1, 256), 256, 0, stream,
              rowptr, NvOut + 1, (const int32_t*)tile_sum, cursor);
    if (Nf > 0 && NvOut > 0) {
        PB_LAUNCH("corner_fill", corner_fill_kernel, (unsigned)ceil_div(3 * Nf, 256), 256, 0, stream,
                  3 * Nf, NvIn, NvOut, face, vtMap, cursor, entries);
        PB_LAUNCH("sort_short_rows", sort_short_rows_kernel, (unsigned)ceil_div(NvOut, 128), 128, 0, stream,
                  NvOut, (const int32_t*)rowptr, entries, long_rows, n_long);
        PB_LAUNCH("sort_long_rows", sort_long_rows_kernel, 2 * sm_count(), 256, 0, stream,
                  (const int32_t*)rowptr, entries, (const int32_t*)long_rows, (const int32_t*)n_long, tmp);
    }
    return PB200_OK;
}

}  // namespace pb

using namespace pb;

extern "C" {

int pb200_count_vertex_adjface(int64_t Nf, int64_t NvIn, int64_t NvOut, const int32_t* face,
                               const int32_t* vtMap, int32_t* nfCount, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NvIn >= 0 && NvOut >= 0 && Nf < (1LL << 29), PB200_EINVAL, "count_vertex_adjface: bad sizes");
    if (NvOut == 0) return PB200_OK;
    PB_REQUIRE(nfCount && (Nf == 0 || face), PB200_EINVAL, "count_vertex_adjface: null pointer");
    PB_CUDA(cudaMemsetAsync(nfCount, 0, sizeof(int32_t) * NvOut, stream));
    if (Nf == 0) return PB200_OK;
    PB_LAUNCH("corner_count", corner_count_kernel, (unsigned)ceil_div(3 * Nf, 256), 256, 0, stream,
              3 * Nf, NvIn, NvOut, face, vtMap, nfCount, (int32_t*)nullptr);
    return PB200_OK;
}

size_t pb200_vertex_csr_workspace_bytes(int64_t Nf, int64_t NvOut) {
    if (Nf < 0 || NvOut < 0) return 0;
    size_t cursor = align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    size_t tiles = align_up(sizeof(int32_t) * (size_t)(ceil_div(NvOut + 1, SCAN_TILE) + 1), 256);
    size_t longs = align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    size_t tmp = align_up(sizeof(int32_t) * (size_t)(3 * Nf + 1), 256);
    return cursor + tiles + longs + tmp + 256;
}

int pb200_build_vertex_csr(int64_t Nf, int64_t NvIn, int64_t NvOut, const int32_t* face,
                           const int32_t* vtMap, int32_t* rowptr, int32_t* entries, int32_t* status,
                           void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NvIn >= 0 && NvOut >= 0 && Nf < (1LL << 29) && NvOut < (1LL << 31) - 1, PB200_EINVAL,
               "build_vertex_csr: bad sizes");
    PB_REQUIRE(rowptr && status && (Nf == 0 || (face && entries)), PB200_EINVAL, "build_vertex_csr: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_vertex_csr_workspace_bytes(Nf, NvOut), PB200_EWORKSPACE,
               "build_vertex_csr: workspace too small");
    char* w = (char*)workspace;
    int32_t* cursor = (int32_t*)w;  w += align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    int ntiles = (int)ceil_div(NvOut + 1, SCAN_TILE);
    int32_t* tile_sum = (int32_t*)w; w += align_up(sizeof(int32_t) * (size_t)(ntiles + 1), 256);
    int32_t* long_rows = (int32_t*)w; w += align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    int32_t* tmp = (int32_t*)w;      w += align_up(sizeof(int32_t) * (size_t)(3 * Nf + 1), 256);
    int32_t* n_long = (int32_t*)w;

    PB_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    PB_CUDA(cudaMemsetAsync(cursor, 0, sizeof(int32_t) * (NvOut + 1), stream));
    PB_CUDA(cudaMemsetAsync(n_long, 0, sizeof(int32_t), stream));
    if (Nf > 0)
        PB_LAUNCH("corner_count", corner_count_kernel, (unsigned)ceil_div(3 * Nf, 256), 256, 0, stream,
                  3 * Nf, NvIn, NvOut, face, vtMap, cursor, status);
    return pb::finish_vertex_csr(Nf, NvIn, NvOut, face, vtMap, rowptr, entries, cursor, tile_sum, long_rows, tmp, n_long,
                                 stream);
}

int pb200_level_prepare(int64_t Nf, int64_t NvIn, int64_t NvOut, int vstride, const float* vertex, const int32_t* face,
                        const int32_t* vtMap, int L, int orient, float* geometry, float* normals, float* coeff,
                        int32_t* nfCount, int32_t* rowptr, int32_t* entries, int32_t* status,
                        void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NvIn >= 0 && NvOut >= 0 && Nf < (1LL << 29) && NvOut < (1LL << 31) - 1 && vstride >= 3,
               PB200_EINVAL, "level_prepare: bad sizes");
    PB_REQUIRE(L >= 0 && L <= 5, PB200_EINVAL, "level_prepare: degree L=%d not supported (0..5)", L);
    PB_REQUIRE(rowptr && status && nfCount && (Nf == 0 || (face && entries && vertex && coeff)), PB200_EINVAL,
               "level_prepare: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_vertex_csr_workspace_bytes(Nf, NvOut), PB200_EWORKSPACE,
               "level_prepare: workspace too small");
    char* w = (char*)workspace;
    int32_t* cursor = (int32_t*)w;  w += align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    int ntiles = (int)ceil_div(NvOut + 1, SCAN_TILE);
    int32_t* tile_sum = (int32_t*)w; w += align_up(sizeof(int32_t) * (size_t)(ntiles + 1), 256);
    int32_t* long_rows = (int32_t*)w; w += align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    int32_t* tmp = (int32_t*)w;      w += align_up(sizeof(int32_t) * (size_t)(3 * Nf + 1), 256);
    int32_t* n_long = (int32_t*)w;
    PB_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    PB_CUDA(cudaMemsetAsync(cursor, 0, sizeof(int32_t) * (NvOut + 1), stream));
    PB_CUDA(cudaMemsetAsync(n_long, 0, sizeof(int32_t), stream));
    if (Nf > 0) {
        static const SphConst cst = make_sph_const();
        const int K = (L + 1) * (L + 1);
        PB_LAUNCH("level_prepare", level_prepare_kernel, (unsigned)ceil_div(Nf, PREP_BLOCK), PREP_BLOCK,
                  sizeof(float) * PREP_BLOCK * (K + 1), stream, Nf, NvIn, NvOut, vstride, vertex, face, vtMap, L, orient, cst,
                  geometry, normals, coeff, cursor, status);
    }
    if (NvOut > 0)      // the corner counts are the reference's nfCount; the scan below overwrites the cursor
        PB_LAUNCH("copy_counts", copy_counts_kernel, (unsigned)ceil_div(NvOut, 256), 256, 0, stream, NvOut,
                  (const int32_t*)cursor, nfCount);
    return pb::finish_vertex_csr(Nf, NvIn, NvOut, face, vtMap, rowptr, entries, cursor, tile_sum, long_rows, tmp, n_long,
                                 stream);
}

size_t pb200_cluster_csr_workspace_bytes(int64_t NvIn, int64_t NvOut) {
    if (NvIn < 0 || NvOut < 0) return 0;
    size_t cursor = align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    size_t tiles = align_up(sizeof(int32_t) * (size_t)(ceil_div(NvOut + 1, SCAN_TILE) + 1), 256);
    size_t longs = align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    size_t tmp = align_up(sizeof(int32_t) * (size_t)(NvIn + 1), 256);
    return cursor + tiles + longs + tmp + 256;
}

int pb200_build_cluster_csr(int64_t NvIn, int64_t NvOut, const int32_t* vtReplace, const int32_t* vtMap,
                            int32_t* key, int32_t* rowptr, int32_t* members, int32_t* status,
                            void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(NvIn >= 0 && NvOut >= 0 && NvIn < (1LL << 31) - 1 && NvOut < (1LL << 31) - 1, PB200_EINVAL,
               "build_cluster_csr: bad sizes");
    PB_REQUIRE(rowptr && status && (NvIn == 0 || (vtReplace && vtMap && key && members)), PB200_EINVAL,
               "build_cluster_csr: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_cluster_csr_workspace_bytes(NvIn, NvOut), PB200_EWORKSPACE,
               "build_cluster_csr: workspace too small");
    char* w = (char*)workspace;
    int32_t* cursor = (int32_t*)w;  w += align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    int ntiles = (int)ceil_div(NvOut + 1, SCAN_TILE);
    int32_t* tile_sum = (int32_t*)w; w += align_up(sizeof(int32_t) * (size_t)(ntiles + 1), 256);
    int32_t* long_rows = (int32_t*)w; w += align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    int32_t* tmp = (int32_t*)w;      w += align_up(sizeof(int32_t) * (size_t)(NvIn + 1), 256);
    int32_t* n_long = (int32_t*)w;
    PB_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    PB_CUDA(cudaMemsetAsync(cursor, 0, sizeof(int32_t) * (NvOut + 1), stream));
    PB_CUDA(cudaMemsetAsync(n_long, 0, sizeof(int32_t), stream));
    if (NvIn > 0)
        PB_LAUNCH("cluster_count", cluster_count_kernel, (unsigned)ceil_div(NvIn, 256), 256, 0, stream,
                  NvIn, NvOut, vtReplace, vtMap, key, cursor, status);
    PB_LAUNCH("scan_tiles", scan_tiles_kernel, ntiles, SCAN_THREADS, 0, stream,
              (const int32_t*)cursor, NvOut + 1, rowptr, tile_sum);
    PB_LAUNCH("scan_tile_sums", scan_tile_sums_kernel, 1, 32, 0, stream, tile_sum, ntiles, tile_sum + ntiles);
    PB_LAUNCH("scan_finish", scan_finish_kernel, (unsigned)ceil_div(NvOut + 1, 256), 256, 0, stream,
              rowptr, NvOut + 1, (const int32_t*)tile_sum, cursor);
    if (NvIn > 0 && NvOut > 0) {
        PB_LAUNCH("cluster_fill", cluster_fill_kernel, (unsigned)ceil_div(NvIn, 256), 256, 0, stream,
                  NvIn, (const int32_t*)key, cursor, members);
        PB_LAUNCH("sort_short_rows", sort_short_rows_kernel, (unsigned)ceil_div(NvOut, 128), 128, 0, stream,
                  NvOut, (const int32_t*)rowptr, members, long_rows, n_long);
        PB_LAUNCH("sort_long_rows", sort_long_rows_kernel, 2 * sm_count(), 256, 0, stream,
                  (const int32_t*)rowptr, members, (const int32_t*)long_rows, (const int32_t*)n_long, tmp);
    }
    return PB200_OK;
}

int pb200_build_key_csr(int64_t N, int64_t NvOut, const int32_t* key, int key_stride, int32_t* rowptr,
                        int32_t* members, int32_t* status, void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(N >= 0 && NvOut >= 0 && N < (1LL << 31) - 1 && NvOut < (1LL << 31) - 1 && key_stride >= 1, PB200_EINVAL,
               "build_key_csr: bad sizes");
    PB_REQUIRE(rowptr && status && (N == 0 || (key && members)), PB200_EINVAL, "build_key_csr: null pointer");
    PB_REQUIRE(workspace && workspace_bytes >= pb200_cluster_csr_workspace_bytes(N, NvOut), PB200_EWORKSPACE,
               "build_key_csr: workspace too small");
    char* w = (char*)workspace;
    int32_t* cursor = (int32_t*)w;  w += align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    int ntiles = (int)ceil_div(NvOut + 1, SCAN_TILE);
    int32_t* tile_sum = (int32_t*)w; w += align_up(sizeof(int32_t) * (size_t)(ntiles + 1), 256);
    int32_t* long_rows = (int32_t*)w; w += align_up(sizeof(int32_t) * (size_t)(NvOut + 1), 256);
    int32_t* tmp = (int32_t*)w;      w += align_up(sizeof(int32_t) * (size_t)(N + 1), 256);
    int32_t* n_long = (int32_t*)w;
    PB_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    PB_CUDA(cudaMemsetAsync(cursor, 0, sizeof(int32_t) * (NvOut + 1), stream));
    PB_CUDA(cudaMemsetAsync(n_long, 0, sizeof(int32_t), stream));
    if (N > 0)
        PB_LAUNCH("key_count", key_count_kernel, (unsigned)ceil_div(N, 256), 256, 0, stream, N, NvOut, key, key_stride,
                  cursor, status);
    PB_LAUNCH("scan_tiles", scan_tiles_kernel, ntiles, SCAN_THREADS, 0, stream,
              (const int32_t*)cursor, NvOut + 1, rowptr, tile_sum);
    PB_LAUNCH("scan_tile_sums", scan_tile_sums_kernel, 1, 32, 0, stream, tile_sum, ntiles, tile_sum + ntiles);
    PB_LAUNCH("scan_finish", scan_finish_kernel, (unsigned)ceil_div(NvOut + 1, 256), 256, 0, stream,
              rowptr, NvOut + 1, (const int32_t*)tile_sum, cursor);
    if (N > 0 && NvOut > 0) {
        PB_LAUNCH("key_fill", key_fill_kernel, (unsigned)ceil_div(N, 256), 256, 0, stream, N, NvOut, key, key_stride,
                  cursor, members);
        PB_LAUNCH("sort_short_rows", sort_short_rows_kernel, (unsigned)ceil_div(NvOut, 128), 128, 0, stream,
                  NvOut, (const int32_t*)rowptr, members, long_rows, n_long);
        PB_LAUNCH("sort_long_rows", sort_long_rows_kernel, 2 * sm_count(), 256, 0, stream,
                  (const int32_t*)rowptr, members, (const int32_t*)long_rows, (const int32_t*)n_long, tmp);
    }
    return PB200_OK;
}

int pb200_triangle_geometry(int64_t Nf, int64_t Nv, int vstride, const float* vertex, const int32_t* face,
                            float* geometry, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && Nv >= 0 && vstride >= 3, PB200_EINVAL, "triangle_geometry: bad sizes");
    if (Nf == 0) return PB200_OK;
    PB_REQUIRE(vertex && face && geometry, PB200_EINVAL, "triangle_geometry: null pointer");
    PB_LAUNCH("triangle_geometry", triangle_geometry_kernel, (unsigned)ceil_div(Nf, 256), 256, 0, stream,
              Nf, Nv, vstride, vertex, face, geometry);
    return PB200_OK;
}

int pb200_check_num_interior(int64_t Nf, int64_t NiK, const int32_t* numInterior, int32_t* status, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NiK >= 0 && NiK < (1LL << 31), PB200_EINVAL, "check_num_interior: bad sizes");
    PB_REQUIRE(status && (Nf == 0 || numInterior), PB200_EINVAL, "check_num_interior: null pointer");
    PB_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    if (Nf == 0) return PB200_OK;
    PB_LAUNCH("check_running_count", check_running_count_kernel, persistent_blocks(Nf, 256, 8), 256, 0, stream,
              Nf, NiK, numInterior, status);
    return PB200_OK;
}

int pb200_face_mean_rows(int64_t Nf, int64_t NiK, int C, const float* rows, const int32_t* cum, float* out, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NiK >= 0 && C > 0, PB200_EINVAL, "face_mean_rows: bad sizes");
    if (Nf == 0) return PB200_OK;
    PB_REQUIRE(cum && out && (NiK == 0 || rows), PB200_EINVAL, "face_mean_rows: null pointer");
    bool vec = (C % 4 == 0) && aligned16(rows) && aligned16(out);
    int CVn = vec ? C / 4 : C;
    int grid = persistent_blocks(Nf * CVn, 256, 16);
    if (vec) PB_LAUNCH("face_mean_rows", face_mean_rows_kernel<4>, grid, 256, 0, stream, Nf, NiK, CVn, rows, cum, out);
    else     PB_LAUNCH("face_mean_rows", face_mean_rows_kernel<1>, grid, 256, 0, stream, Nf, NiK, CVn, rows, cum, out);
    return PB200_OK;
}

int pb200_expand_rows_forward(int64_t Nf, int64_t NiK, int C, const float* in, const int32_t* cum, float* out,
                              void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NiK >= 0 && C > 0, PB200_EINVAL, "expand_rows_forward: bad sizes");
    if (NiK == 0) return PB200_OK;
    PB_REQUIRE(in && cum && out, PB200_EINVAL, "expand_rows_forward: null pointer");
    bool vec = (C % 4 == 0) && aligned16(in) && aligned16(out);
    int CVn = vec ? C / 4 : C;
    int grid = persistent_blocks(Nf * CVn, 256, 16);
    if (vec) PB_LAUNCH("expand_rows_fwd", expand_rows_fwd_kernel<4>, grid, 256, 0, stream, Nf, NiK, CVn, in, cum, out);
    else     PB_LAUNCH("expand_rows_fwd", expand_rows_fwd_kernel<1>, grid, 256, 0, stream, Nf, NiK, CVn, in, cum, out);
    return PB200_OK;
}

int pb200_expand_rows_backward(int64_t Nf, int64_t NiK, int C, const float* gout, const int32_t* cum, float* gin,
                               void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    PB_REQUIRE(Nf >= 0 && NiK >= 0 && C > 0, PB200_EINVAL, "expand_rows_backward: bad sizes");
    if (Nf == 0) return PB200_OK;
    PB_REQUIRE(cum && gin && (NiK == 0 || gout), PB200_EINVAL, "expand_rows_backward: null pointer");
    bool vec = (C % 4 == 0) && aligned16(gout) && aligned16(gin);
    int CVn = vec ? C / 4 : C;
    int grid = persistent_blocks(Nf * CVn, 256, 16);
    if (vec) PB_LAUNCH("expand_rows_bwd", expand_rows_bwd_kernel<4>, grid, 256, 0, stream, Nf, NiK, CVn, gout, cum, gin);
    else     PB_LAUNCH("expand_rows_bwd", expand_rows_bwd_kernel<1>, grid, 256, 0, stream, Nf, NiK, CVn, gout, cum, gin);
    return PB200_OK;
}

}  // extern "C"

/* TEST INFRASTRUCTURE ONLY -- never linked into or called by the product library.
 *
 * Sequential CPU restatement of one pass of the reference's quadric-error mesh decimation
 * (picasso/mesh/pi_modules/source/decimate_gpu.cu:618-747, `meshDecimationLauncher`) and of its
 * cluster merge (`combineClustersLauncher`, decimate_gpu.cu:750-812).  It follows the reference
 * step by step -- including the sequential two-sweep vertex clustering of `clusterVertices`
 * (decimate_gpu.cu:561-614), which the GPU implementation replaces by a parallel formulation --
 * so that comparing the two is a real test.
 *
 * Where the reference leaves an order open (float atomicAdd), this restatement fixes one and
 * says so; every float operation is rounded on its own (compile with -ffp-contract=off), so a
 * GPU kernel that performs the same operations in the same order without fused multiply-adds
 * agrees with it bit for bit.
 *
 *   quadric of a vertex   = sum over its face corners, ascending (face, corner), of the face
 *                           quadric times the area weight; then, in the same corner order,
 *                           the boundary quadrics of the corner's two face edges (lower edge
 *                           slot first) -- decimate_gpu.cu:225-256, 311-374
 *   edge order            = ascending (lower vertex, higher vertex); duplicates collapse to
 *                           one candidate; an edge seen once is a boundary edge
 *   candidate order       = ascending cost per sample, ties in edge order (the reference sorts
 *                           with a stable radix sort, decimate_gpu.cu:689); -0 counts as +0
 *                           and every NaN as the largest value
 *   cluster position      = (sum of the contracted vertices' rows, ascending vertex id, then the
 *                           representative's own row) / cluster size -- decimate_gpu.cu:403-441
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define RCOND_EPS 1e-6f
#define EPS_F 2.220446049250313e-16f
#define AREA_MAGNITUDE 100.0f

static void quadric_of_plane(const float n[3], float d, float Q[10]) {
    Q[0] = n[0] * n[0]; Q[1] = n[0] * n[1]; Q[2] = n[0] * n[2];
    Q[3] = n[1] * n[1]; Q[4] = n[1] * n[2]; Q[5] = n[2] * n[2];
    Q[6] = n[0] * d;    Q[7] = n[1] * d;    Q[8] = n[2] * d;
    Q[9] = d * d;
}

static float dot3(const float a[3], const float b[3]) { return a[0] * b[0] + a[1] * b[1] + a[2] * b[2]; }

/* reduced row echelon form of [A | b | I] with partial pivoting (decimate_gpu.cu:80-187):
 * returns the reciprocal condition number estimate, xyz = -A^-1 b */
static float solve_rref(const float A[3][3], const float b[3], float xyz[3]) {
    float M[3][7];
    for (int r = 0; r < 3; ++r) {
        for (int c = 0; c < 3; ++c) { M[r][c] = A[r][c]; M[r][c + 4] = (r == c) ? 1.f : 0.f; }
        M[r][3] = b[r];
    }
    float normA = 0.f;
    for (int r = 0; r < 3; ++r) {
        float s = 0.f;
        for (int c = 0; c < 3; ++c) s += fabsf(M[r][c]);
        if (normA < s) normA = s;
    }
    const float tol = EPS_F * 7 * normA;
    int i = 0, j = 0;
    while (i < 3 && j < 7) {
        float p = fabsf(M[i][j]);
        int k = i;
        for (int r = i + 1; r < 3; ++r)
            if (p < fabsf(M[r][j])) { p = fabsf(M[r][j]); k = r; }
        if (p <= tol) {
            for (int r = i; r < 3; ++r) M[r][j] = 0.f;
            ++j;
        } else {
            for (int c = j; c < 7; ++c) { float t = M[i][c]; M[i][c] = M[k][c]; M[k][c] = t; }
            const float piv = M[i][j];
            for (int c = j; c < 7; ++c) M[i][c] = M[i][c] / piv;
            for (int r = 0; r < 3; ++r) {
                if (r == i) continue;
                const float v = M[r][j];
                for (int c = j; c < 7; ++c) M[r][c] -= v * M[i][c];
            }
            ++i; ++j;
        }
    }
    xyz[0] = -M[0][3]; xyz[1] = -M[1][3]; xyz[2] = -M[2][3];
    float normInv = 0.f;
    for (int r = 0; r < 3; ++r) {
        float s = 0.f;
        for (int c = 0; c < 3; ++c) s += fabsf(M[r][c + 4]);
        if (normInv < s) normInv = s;
    }
    return 1 / (normA * normInv);
}

static float quadric_error(const float x[3], const float A[3][3], const float b[3], float c) {
    return ((x[0] * A[0][0] + x[1] * A[1][0] + x[2] * A[2][0]) * x[0]
          + (x[0] * A[0][1] + x[1] * A[1][1] + x[2] * A[2][1]) * x[1]
          + (x[0] * A[0][2] + x[1] * A[1][2] + x[2] * A[2][2]) * x[2])
          + (x[0] * b[0] + x[1] * b[1] + x[2] * b[2]) * 2
          + c;
}

/* sortable image of a cost: ascending unsigned order == ascending float order, -0 == +0, NaN last */
static uint32_t cost_key(float c) {
    uint32_t u;
    if (c != c) return 0xffffffffu;
    if (c == 0.f) c = 0.f;
    memcpy(&u, &c, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

typedef struct { int lo, hi, e; } edge_t;
static int cmp_edge(const void* a, const void* b) {
    const edge_t* x = (const edge_t*)a; const edge_t* y = (const edge_t*)b;
    if (x->lo != y->lo) return x->lo < y->lo ? -1 : 1;
    if (x->hi != y->hi) return x->hi < y->hi ? -1 : 1;
    return x->e < y->e ? -1 : (x->e > y->e);
}
typedef struct { uint32_t key; int pos; } cand_t;
static int cmp_cand(const void* a, const void* b) {
    const cand_t* x = (const cand_t*)a; const cand_t* y = (const cand_t*)b;
    if (x->key != y->key) return x->key < y->key ? -1 : 1;
    return x->pos < y->pos ? -1 : (x->pos > y->pos);
}

/* face edge slots as in decimate_gpu.cu:262-308: slot 0 = (v1,v2), 1 = (v1,v3), 2 = (v2,v3) */
static const int SLOT_A[3] = {0, 0, 1}, SLOT_B[3] = {1, 2, 2};
/* the two edge slots that touch corner c, lower slot first */
static const int CORNER_SLOTS[3][2] = {{0, 1}, {0, 2}, {1, 2}};

/* nvIn / mfIn are the running (inclusive) totals per sample, as the reference passes them */
int oracle_mesh_simplify(int useArea, float wgtBnd, int B, int D, int Nv, int Nf,
                         const int* nvIn, const int* mfIn, const int* nv2Remove,
                         const float* vertexIn, const int* faceIn, const float* planeIn,
                         int* nvOut, int* mfOut, float* vertexOut, int* faceOut,
                         int* vtReplace, int* vtMap, uint8_t* isDegenerate, float* edgeCostOut /* 3*Nf or NULL */) {
    const int Ne = 3 * Nf;
    float* Q = (float*)calloc((size_t)Nv * 10 + 1, sizeof(float));
    edge_t* ed = (edge_t*)malloc(sizeof(edge_t) * (size_t)(Ne + 1));
    uint8_t* bnd = (uint8_t*)calloc((size_t)Ne + 1, 1);
    int* ulo = (int*)malloc(sizeof(int) * (size_t)(Ne + 1));
    int* uhi = (int*)malloc(sizeof(int) * (size_t)(Ne + 1));
    cand_t* cand = (cand_t*)malloc(sizeof(cand_t) * (size_t)(Ne + 1));
    char* covered = (char*)calloc((size_t)Nv + 1, 1);
    int* kept = (int*)calloc((size_t)Nv + 1, sizeof(int));
    if (!Q || !ed || !bnd || !ulo || !uhi || !cand || !covered || !kept) return -1;

    /* face quadrics, decimate_gpu.cu:225-256 */
    for (int f = 0; f < Nf; ++f) {
        float Qf[10];
        quadric_of_plane(planeIn + 5 * f, planeIn[5 * f + 3], Qf);
        const float area = planeIn[5 * f + 4] * AREA_MAGNITUDE;
        const float w = useArea ? area / 3 : 1.0f;
        for (int c = 0; c < 3; ++c) {
            const int v = faceIn[3 * f + c];
            for (int t = 0; t < 10; ++t) Q[10 * v + t] += Qf[t] * w;
        }
    }
    /* edges, decimate_gpu.cu:259-308 */
    for (int f = 0; f < Nf; ++f)
        for (int k = 0; k < 3; ++k) {
            const int a = faceIn[3 * f + SLOT_A[k]], b = faceIn[3 * f + SLOT_B[k]];
            ed[3 * f + k].lo = a <= b ? a : b;
            ed[3 * f + k].hi = a <= b ? b : a;
            ed[3 * f + k].e = 3 * f + k;
        }
    qsort(ed, (size_t)Ne, sizeof(edge_t), cmp_edge);
    int nu = 0;
    for (int i = 0; i < Ne; ++i) {
        const int same_prev = i > 0 && ed[i - 1].lo == ed[i].lo && ed[i - 1].hi == ed[i].hi;
        const int same_next = i + 1 < Ne && ed[i + 1].lo == ed[i].lo && ed[i + 1].hi == ed[i].hi;
        if (!same_prev && !same_next) bnd[ed[i].e] = 1;
        if (!same_prev) { ulo[nu] = ed[i].lo; uhi[nu] = ed[i].hi; ++nu; }
    }
    /* boundary quadrics, decimate_gpu.cu:311-374 */
    if (wgtBnd > 0)
        for (int f = 0; f < Nf; ++f)
            for (int c = 0; c < 3; ++c)
                for (int s = 0; s < 2; ++s) {
                    const int k = CORNER_SLOTS[c][s];
                    if (!bnd[3 * f + k]) continue;
                    const int a = faceIn[3 * f + SLOT_A[k]], b = faceIn[3 * f + SLOT_B[k]];
                    const int vi = a <= b ? a : b, vj = a <= b ? b : a;
                    const float* n = planeIn + 5 * f;
                    const float* pi = vertexIn + (size_t)vi * D;
                    const float* pj = vertexIn + (size_t)vj * D;
                    const float dx[3] = {pj[0] - pi[0], pj[1] - pi[1], pj[2] - pi[2]};
                    float bn[3];
                    bn[0] = n[1] * dx[2] - n[2] * dx[1];
                    bn[1] = n[2] * dx[0] - n[0] * dx[2];
                    bn[2] = n[0] * dx[1] - n[1] * dx[0];
                    float len = sqrtf(bn[0] * bn[0] + bn[1] * bn[1] + bn[2] * bn[2]);
                    len = len > 1e-20f ? len : 1e-20f;
                    bn[0] /= len; bn[1] /= len; bn[2] /= len;
                    const float d = -dot3(bn, pi);
                    float wb = dot3(dx, dx) * AREA_MAGNITUDE;
                    if (useArea) wb *= wgtBnd; else wb = wgtBnd;
                    float Qe[10];
                    quadric_of_plane(bn, d, Qe);
                    const int v = faceIn[3 * f + c];
                    for (int t = 0; t < 10; ++t) Q[10 * v + t] += Qe[t] * wb;
                }
    /* candidate costs, decimate_gpu.cu:378-416 */
    for (int u = 0; u < nu; ++u) {
        const int vi = ulo[u], vj = uhi[u];
        float q[10];
        for (int t = 0; t < 10; ++t) q[t] = Q[10 * vi + t] + Q[10 * vj + t];
        const float A[3][3] = {{q[0], q[1], q[2]}, {q[1], q[3], q[4]}, {q[2], q[4], q[5]}};
        const float b[3] = {q[6], q[7], q[8]};
        float x[3], cost;
        const float rc = solve_rref(A, b, x);
        if (rc > RCOND_EPS) cost = quadric_error(x, A, b, q[9]);
        else {
            const float ei = quadric_error(vertexIn + (size_t)vi * D, A, b, q[9]);
            const float ej = quadric_error(vertexIn + (size_t)vj * D, A, b, q[9]);
            cost = ei < ej ? ei : ej;
        }
        cand[u].key = cost_key(cost);
        cand[u].pos = u;
        if (edgeCostOut) edgeCostOut[u] = cost;
    }
    /* per sample: order by cost, then the two sequential sweeps of decimate_gpu.cu:561-614 */
    memset(vtReplace, 0, sizeof(int) * (size_t)Nv);
    int ubeg = 0;
    for (int s = 0; s < B; ++s) {
        const int vend = nvIn[s];
        int uend = ubeg;
        while (uend < nu && ulo[uend] < vend) ++uend;
        qsort(cand + ubeg, (size_t)(uend - ubeg), sizeof(cand_t), cmp_cand);
        const int want = nv2Remove[s];
        int removed = 0;
        for (int i = ubeg; i < uend && removed < want; ++i) {
            const int vi = ulo[cand[i].pos], vj = uhi[cand[i].pos];
            if (vi == vj) continue;                       /* degenerate input face: no candidate */
            if (!covered[vi] && !covered[vj]) {
                vtReplace[vi] = -vj;
                vtReplace[vj] += 1;
                covered[vi] = covered[vj] = 1;
                ++removed;
            }
        }
        for (int i = ubeg; i < uend && removed < want; ++i) {
            int a = ulo[cand[i].pos], b = uhi[cand[i].pos];
            if (a == b) continue;
            if (covered[a] && covered[b]) continue;
            if (covered[b] == 1) { const int t = a; a = b; b = t; }
            if (vtReplace[a] < 0) a = -vtReplace[a];
            vtReplace[b] = -a;
            vtReplace[a] += 1;
            covered[b] = 2;
            ++removed;
        }
        ubeg = uend;
    }
    /* contraction, decimate_gpu.cu:403-441 */
    memset(vertexOut, 0, sizeof(float) * (size_t)Nv * D);
    for (int v = 0; v < Nv; ++v)
        if (vtReplace[v] < 0) {
            const int r = -vtReplace[v];
            for (int t = 0; t < D; ++t) vertexOut[(size_t)r * D + t] += vertexIn[(size_t)v * D + t];
        }
    for (int v = 0; v < Nv; ++v) {
        if (vtReplace[v] > 0)
            for (int t = 0; t < D; ++t)
                vertexOut[(size_t)v * D + t] = (vertexOut[(size_t)v * D + t] + vertexIn[(size_t)v * D + t]) / (vtReplace[v] + 1);
        if (vtReplace[v] == 0)
            for (int t = 0; t < D; ++t) vertexOut[(size_t)v * D + t] = vertexIn[(size_t)v * D + t];
    }
    /* faces, decimate_gpu.cu:444-507 */
    for (int s = 0; s < B; ++s) mfOut[s] = 0;
    for (int f = 0; f < Nf; ++f) {
        int s = 0;
        while (s < B - 1 && f >= mfIn[s]) ++s;
        int v[3];
        for (int c = 0; c < 3; ++c) {
            v[c] = faceIn[3 * f + c];
            if (vtReplace[v[c]] < 0) v[c] = -vtReplace[v[c]];
            faceOut[3 * f + c] = v[c];
        }
        if (v[0] == v[1] || v[0] == v[2] || v[1] == v[2]) isDegenerate[f] = 1;
        else { isDegenerate[f] = 0; mfOut[s] += 1; kept[v[0]] = kept[v[1]] = kept[v[2]] = 1; }
    }
    /* vertex map and output sizes, decimate_gpu.cu:509-533, 727-733 */
    int run = 0, prev = 0;
    for (int s = 0, v = 0; s < B; ++s) {
        for (; v < nvIn[s]; ++v) { run += kept[v]; vtMap[v] = kept[v] ? run - 1 : -1; }
        nvOut[s] = run - prev;
        prev = run;
    }
    for (int f = 0; f < Nf; ++f)
        if (!isDegenerate[f])
            for (int c = 0; c < 3; ++c) faceOut[3 * f + c] = vtMap[faceOut[3 * f + c]];
    free(Q); free(ed); free(bnd); free(ulo); free(uhi); free(cand); free(covered); free(kept);
    return nu;
}

/* decimate_gpu.cu:750-812: clusters of a mesh A (rep, map) merged with those of its decimated
 * version B into clusters of A over the vertices B kept */
void oracle_combine_clusters(int nvA, int nvB, const int* repA, const int* mapA, const int* repB, const int* mapB,
                             int* repOut, int* mapOut) {
    int* rb = (int*)malloc(sizeof(int) * (size_t)(nvB + 1));
    memcpy(rb, repB, sizeof(int) * (size_t)nvB);
    memcpy(repOut, repA, sizeof(int) * (size_t)nvA);
    for (int v = 0; v < nvA; ++v) {
        const int vo = mapA[v];
        if (vo >= 0 && rb[vo] >= 0) rb[vo] = v;
    }
    for (int v = 0; v < nvA; ++v) {
        int vi = v;
        if (repA[vi] < 0) vi = -repA[vi];
        int vo = mapA[vi];
        if (vo >= 0 && rb[vo] < 0) {
            vo = -rb[vo];
            repOut[v] = -rb[vo];
            repOut[rb[vo]] += 1;
        }
    }
    for (int v = 0; v < nvA; ++v) mapOut[v] = mapA[v] >= 0 ? mapB[mapA[v]] : -1;
    free(rb);
}

/* Plain-C restatement of the reference's mesh-convolution kernels, one sequential loop
 * nest per CUDA kernel, executed in ascending thread order (the reference's atomics make
 * its own summation order arbitrary; ascending order is one legal schedule of it).
 *
 * TEST INFRASTRUCTURE ONLY: the product library never links or calls this file.  It is a
 * second, independent restatement used to cross-check oracle/mesh_oracle.py and the CUDA
 * kernels on small inputs.  Parity of both restatements is pinned against outputs of the
 * reference's own CUDA operators (tests/golden/).
 *
 * `ACC` is the accumulator type: float reproduces the reference's arithmetic, double
 * (-DORACLE_ACC_DOUBLE) gives the arbiter used when two fp32 results disagree.
 * Citations are paths relative to the reference root.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef ORACLE_ACC_DOUBLE
typedef double ACC;
#define NAME(x) x##_f64acc
#else
typedef float ACC;
#define NAME(x) x
#endif

/* picasso/mesh/pi_modules/source/mesh_conv3d_gpu.cu:176-195 */
void NAME(oracle_v2f_forward)(int Nf, int C, int r, const int32_t* face, const float* in,
                              const float* filter, float* out) {
    int Cr = C * r;
    for (int f = 0; f < Nf; ++f)
        for (int co = 0; co < Cr; ++co) {
            ACC feat = 0;
            for (int k = 0; k < 3; ++k)
                feat += (ACC)filter[co + k * Cr] * (ACC)in[(int64_t)face[3 * f + k] * C + co / r];
            out[(int64_t)f * Cr + co] = (float)feat;
        }
}

/* mesh_conv3d_gpu.cu:201-260 (input and filter gradients; outputs must be zeroed) */
void NAME(oracle_v2f_backward)(int Nf, int Nv, int C, int r, const int32_t* face, const float* in,
                               const float* filter, const float* gout, float* gin, float* gfilt,
                               ACC* scratch /* Nv*C + 3*C*r */) {
    int Cr = C * r;
    ACC* ain = scratch;
    ACC* af = scratch + (int64_t)Nv * C;
    memset(scratch, 0, sizeof(ACC) * ((int64_t)Nv * C + 3 * Cr));
    for (int f = 0; f < Nf; ++f)
        for (int co = 0; co < Cr; ++co) {
            ACC g = gout[(int64_t)f * Cr + co];
            for (int k = 0; k < 3; ++k) {
                int64_t v = face[3 * f + k];
                ain[v * C + co / r] += g * (ACC)filter[co + k * Cr];
                af[k * Cr + co] += g * (ACC)in[v * C + co / r];
            }
        }
    for (int64_t i = 0; i < (int64_t)Nv * C; ++i) gin[i] = (float)ain[i];
    for (int i = 0; i < 3 * Cr; ++i) gfilt[i] = (float)af[i];
}

/* mesh_conv3d_gpu.cu:299-329 (output must be zeroed; the division is applied per term) */
void NAME(oracle_f2v_forward)(int Nf, int NvOut, int C, int r, int K, const int32_t* vtMap,
                              const int32_t* nfCount, const int32_t* face, const float* coeff,
                              const float* in, const float* filter, float* out,
                              ACC* scratch /* NvOut*C*r */) {
    int Cr = C * r;
    memset(scratch, 0, sizeof(ACC) * (int64_t)NvOut * Cr);
    for (int f = 0; f < Nf; ++f)
        for (int co = 0; co < Cr; ++co) {
            ACC w = 0;
            for (int k = 0; k < K; ++k) w += (ACC)coeff[(int64_t)f * K + k] * (ACC)filter[k * Cr + co];
            ACC feat = w * (ACC)in[(int64_t)f * C + co / r];
            for (int j = 0; j < 3; ++j) {
                int vo = vtMap[face[3 * f + j]];
                if (vo >= 0) scratch[(int64_t)vo * Cr + co] += feat / (ACC)nfCount[vo];
            }
        }
    for (int64_t i = 0; i < (int64_t)NvOut * Cr; ++i) out[i] = (float)scratch[i];
}

/* mesh_conv3d_gpu.cu:338-426 */
void NAME(oracle_f2v_backward)(int Nf, int C, int r, int K, const int32_t* vtMap,
                               const int32_t* nfCount, const int32_t* face, const float* coeff,
                               const float* in, const float* filter, const float* gout,
                               float* gin, float* gfilt, ACC* scratch /* Nf*C + K*C*r */) {
    int Cr = C * r;
    ACC* ain = scratch;
    ACC* af = scratch + (int64_t)Nf * C;
    memset(scratch, 0, sizeof(ACC) * ((int64_t)Nf * C + (int64_t)K * Cr));
    for (int f = 0; f < Nf; ++f)
        for (int co = 0; co < Cr; ++co) {
            ACC w = 0;
            for (int k = 0; k < K; ++k) w += (ACC)coeff[(int64_t)f * K + k] * (ACC)filter[k * Cr + co];
            ACC x = in[(int64_t)f * C + co / r];
            for (int j = 0; j < 3; ++j) {
                int vo = vtMap[face[3 * f + j]];
                if (vo < 0) continue;
                ACC g = (ACC)gout[(int64_t)vo * Cr + co];
                ACC nf = (ACC)nfCount[vo];
                ain[(int64_t)f * C + co / r] += g * w / nf;
                for (int k = 0; k < K; ++k)
                    af[k * Cr + co] += g * ((ACC)coeff[(int64_t)f * K + k] * x) / nf;
            }
        }
    for (int64_t i = 0; i < (int64_t)Nf * C; ++i) gin[i] = (float)ain[i];
    for (int i = 0; i < K * Cr; ++i) gfilt[i] = (float)af[i];
}

/* mesh_conv3d_gpu.cu:6-37 (output must be zeroed) */
void NAME(oracle_f2f_forward)(int Nf, int F, int Cin, int Cout, const int32_t* cum, const float* bary,
                              const float* in, const float* filter, float* out) {
    for (int f = 0; f < Nf; ++f) {
        int k0 = f > 0 ? cum[f - 1] : 0, k1 = cum[f];
        int T = k1 - k0;
        for (int co = 0; co < Cout; ++co) {
            ACC acc = 0;
            for (int ci = 0; ci < Cin; ++ci) {
                const float* w = filter + ((int64_t)co * Cin + ci) * F;
                for (int k = k0; k < k1; ++k) {
                    ACC weight = 0;
                    for (int d = 0; d < F; ++d) weight += (ACC)bary[(int64_t)k * F + d] * (ACC)w[d];
                    acc += (ACC)in[(int64_t)k * Cin + ci] * weight / (ACC)T;
                }
            }
            out[(int64_t)f * Cout + co] = (float)acc;
        }
    }
}

/* mesh_conv3d_gpu.cu:45-135 */
void NAME(oracle_f2f_backward)(int Nf, int NiK, int F, int Cin, int Cout, const int32_t* cum,
                               const float* bary, const float* in, const float* filter,
                               const float* gout, float* gin, float* gfilt,
                               ACC* scratch /* NiK*Cin + Cout*Cin*F */) {
    ACC* ain = scratch;
    ACC* af = scratch + (int64_t)NiK * Cin;
    memset(scratch, 0, sizeof(ACC) * ((int64_t)NiK * Cin + (int64_t)Cout * Cin * F));
    for (int f = 0; f < Nf; ++f) {
        int k0 = f > 0 ? cum[f - 1] : 0, k1 = cum[f];
        int T = k1 - k0;
        for (int co = 0; co < Cout; ++co) {
            ACC g = gout[(int64_t)f * Cout + co];
            for (int ci = 0; ci < Cin; ++ci) {
                int64_t ch = ((int64_t)co * Cin + ci) * F;
                for (int k = k0; k < k1; ++k) {
                    ACC weight = 0;
                    for (int d = 0; d < F; ++d) weight += (ACC)bary[(int64_t)k * F + d] * (ACC)filter[ch + d];
                    ain[(int64_t)k * Cin + ci] += g * weight / (ACC)T;
                    ACC t = g * (ACC)in[(int64_t)k * Cin + ci] / (ACC)T;
                    for (int d = 0; d < F; ++d) af[ch + d] += t * (ACC)bary[(int64_t)k * F + d];
                }
            }
        }
    }
    for (int64_t i = 0; i < (int64_t)NiK * Cin; ++i) gin[i] = (float)ain[i];
    for (int64_t i = 0; i < (int64_t)Cout * Cin * F; ++i) gfilt[i] = (float)af[i];
}

#ifndef ORACLE_ACC_DOUBLE
/* picasso/mesh/pi_modules/source/decimate_gpu.cu:813-831 (output must be zeroed) */
void oracle_count_vertex_adjface(int Nf, const int32_t* face, const int32_t* vtMap, int32_t* nfCount) {
    for (int f = 0; f < Nf; ++f)
        for (int k = 0; k < 3; ++k) {
            int vo = vtMap[face[3 * f + k]];
            if (vo >= 0) nfCount[vo] += 1;
        }
}

/* picasso/mesh/layers.py:341-356 followed by picasso/math_utils.py:10-62, in fp32 with
 * the 36 normalisation constants `c` supplied by the caller (they are evaluated in fp32
 * by the reference, see mesh_oracle.py:_sph_constants). */
void oracle_sph_harm_coeff(int N, int L, const float* xyz, const float* c, float* out) {
    int K = (L + 1) * (L + 1);
    const float PI_F = (float)3.14159265358979323846;
    for (int i = 0; i < N; ++i) {
        float x = xyz[3 * i], y = xyz[3 * i + 1], z = xyz[3 * i + 2];
        float l2 = sqrtf(x * x + y * y + z * z) + 1e-10f;
        x /= l2; y /= l2; z /= l2;
        float phi = atan2f(y, x);
        float theta = atan2f(z, sqrtf(x * x + y * y));
        if (phi < 0) phi += 2 * PI_F;
        theta = PI_F / 2 - theta;
        float st = sinf(theta), ct = cosf(theta);
        float st2 = st * st, st3 = st2 * st, st4 = powf(st, 4.f), st5 = powf(st, 5.f);
        float ct2 = ct * ct, ct3 = ct2 * ct, ct4 = powf(ct, 4.f), ct5 = powf(ct, 5.f);
        float o[36];
        o[0] = c[0];
        o[1] = c[1] * st * cosf(phi);  o[2] = c[2] * ct;  o[3] = c[3] * st * sinf(phi);
        o[4] = c[4] * st2 * cosf(2 * phi);  o[5] = c[5] * st * ct * cosf(phi);
        o[6] = c[6] * (3 * ct2 - 1);
        o[7] = c[7] * st2 * sinf(2 * phi);  o[8] = c[8] * st * ct * sinf(phi);
        o[9] = c[9] * st3 * cosf(3 * phi);  o[10] = c[10] * st2 * ct * cosf(2 * phi);
        o[11] = c[11] * st * (5 * ct2 - 1) * cosf(phi);  o[12] = c[12] * (5 * ct3 - 3 * ct);
        o[13] = c[13] * st3 * sinf(3 * phi);  o[14] = c[14] * st2 * ct * sinf(2 * phi);
        o[15] = c[15] * st * (5 * ct2 - 1) * sinf(phi);
        o[16] = c[16] * st4 * cosf(4 * phi);  o[17] = c[17] * st3 * ct * cosf(3 * phi);
        o[18] = c[18] * st2 * (7 * ct2 - 1) * cosf(2 * phi);
        o[19] = c[19] * st * (7 * ct3 - 3 * ct) * cosf(phi);
        o[20] = c[20] * (35 * ct4 - 30 * ct2 + 3);
        o[21] = c[21] * st4 * sinf(4 * phi);  o[22] = c[22] * st3 * ct * sinf(3 * phi);
        o[23] = c[23] * st2 * (7 * ct2 - 1) * sinf(2 * phi);
        o[24] = c[24] * st * (7 * ct3 - 3 * ct) * sinf(phi);
        o[25] = c[25] * st5 * cosf(5 * phi);  o[26] = c[26] * st4 * ct * cosf(4 * phi);
        o[27] = c[27] * st3 * (9 * ct2 - 1) * cosf(3 * phi);
        o[28] = c[28] * st2 * (3 * ct3 - ct) * cosf(2 * phi);
        o[29] = c[29] * st * (21 * ct4 - 14 * ct2 + 1) * cosf(phi);
        o[30] = c[30] * (63 * ct5 - 70 * ct3 + 15 * ct);
        o[31] = c[31] * st5 * sinf(5 * phi);  o[32] = c[32] * st4 * ct * sinf(4 * phi);
        o[33] = c[33] * st3 * (9 * ct2 - 1) * sinf(3 * phi);
        o[34] = c[34] * st2 * (3 * ct3 - ct) * sinf(2 * phi);
        o[35] = c[35] * st * (21 * ct4 - 14 * ct2 + 1) * sinf(phi);
        for (int k = 0; k < K; ++k) out[(int64_t)i * K + k] = o[k];
    }
}

/* picasso/mesh/pi_modules/decimate.py:70-85 */
void oracle_triangle_geometry(int Nf, int vstride, const float* vertex, const int32_t* face, float* geom) {
    for (int f = 0; f < Nf; ++f) {
        const float* a = vertex + (int64_t)face[3 * f] * vstride;
        const float* b = vertex + (int64_t)face[3 * f + 1] * vstride;
        const float* c = vertex + (int64_t)face[3 * f + 2] * vstride;
        float u[3] = {b[0] - a[0], b[1] - a[1], b[2] - a[2]};
        float v[3] = {c[0] - a[0], c[1] - a[1], c[2] - a[2]};
        float n[3] = {u[1] * v[2] - u[2] * v[1], u[2] * v[0] - u[0] * v[2], u[0] * v[1] - u[1] * v[0]};
        float l2 = sqrtf(n[0] * n[0] + n[1] * n[1] + n[2] * n[2]);
        float* g = geom + (int64_t)f * 5;
        for (int i = 0; i < 3; ++i) g[i] = n[i] / (l2 + 1e-10f);
        g[3] = -(g[0] * a[0] + g[1] * a[1] + g[2] * a[2]);
        g[4] = l2 / 2;
    }
}
#endif

/* ---- mesh pool / unpool.  mapid = -vtReplace[v] for a contracted vertex, else v; the cluster's
 * coarse id is vtMap[mapid] (picasso/mesh/pi_modules/source/mesh_pool3d_gpu.cu:49-58). */
#ifndef ORACLE_ACC_DOUBLE
static int cluster_of(int v, const int32_t* vtReplace, const int32_t* vtMap) {
    int mapid = vtReplace[v] < 0 ? -vtReplace[v] : v;
    return vtMap[mapid];
}

/* mesh_pool3d_gpu.cu:20-88 (init, forward, index); the argmax is the smallest member id */
void oracle_max_pool_forward(int nvIn, int nvOut, int C, const int32_t* vtReplace, const int32_t* vtMap,
                             const float* in, float* out, int32_t* maxIndex) {
    memset(out, 0, sizeof(float) * (size_t)nvOut * C);
    memset(maxIndex, 0, sizeof(int32_t) * (size_t)nvOut * C);
    for (int v = 0; v < nvIn; ++v)
        if (vtMap[v] >= 0)
            for (int c = 0; c < C; ++c) out[(int64_t)vtMap[v] * C + c] = in[(int64_t)v * C + c];
    for (int v = 0; v < nvIn; ++v) {
        int vo = cluster_of(v, vtReplace, vtMap);
        if (vo < 0) continue;
        for (int c = 0; c < C; ++c) out[(int64_t)vo * C + c] = fmaxf(out[(int64_t)vo * C + c], in[(int64_t)v * C + c]);
    }
    for (int v = nvIn - 1; v >= 0; --v) {          /* descending: the smallest id is written last */
        int vo = cluster_of(v, vtReplace, vtMap);
        if (vo < 0) continue;
        for (int c = 0; c < C; ++c)
            if (fabsf(in[(int64_t)v * C + c] - out[(int64_t)vo * C + c]) < 1e-16F) maxIndex[(int64_t)vo * C + c] = v;
    }
}

/* mesh_pool3d_gpu.cu:93-105 */
void oracle_max_pool_backward(int nvIn, int nvOut, int C, const int32_t* maxIndex, const float* gout, float* gin) {
    memset(gin, 0, sizeof(float) * (size_t)nvIn * C);
    for (int vo = 0; vo < nvOut; ++vo)
        for (int c = 0; c < C; ++c) gin[(int64_t)maxIndex[(int64_t)vo * C + c] * C + c] = gout[(int64_t)vo * C + c];
}

/* mesh_pool3d_gpu.cu:112-132 */
void oracle_avg_pool_forward(int nvIn, int nvOut, int C, const int32_t* vtReplace, const int32_t* vtMap,
                             const float* in, float* out) {
    memset(out, 0, sizeof(float) * (size_t)nvOut * C);
    for (int v = 0; v < nvIn; ++v) {
        int mapid = vtReplace[v] < 0 ? -vtReplace[v] : v;
        int vo = vtMap[mapid];
        if (vo < 0) continue;
        int count = vtReplace[mapid] + 1;
        for (int c = 0; c < C; ++c) out[(int64_t)vo * C + c] += in[(int64_t)v * C + c] / count;
    }
}

/* mesh_pool3d_gpu.cu:138-158 */
void oracle_avg_pool_backward(int nvIn, int C, const int32_t* vtReplace, const int32_t* vtMap, const float* gout,
                              float* gin) {
    memset(gin, 0, sizeof(float) * (size_t)nvIn * C);
    for (int v = 0; v < nvIn; ++v) {
        int mapid = vtReplace[v] < 0 ? -vtReplace[v] : v;
        int vo = vtMap[mapid];
        if (vo < 0) continue;
        int count = vtReplace[mapid] + 1;
        for (int c = 0; c < C; ++c) gin[(int64_t)v * C + c] = gout[(int64_t)vo * C + c] / count;
    }
}

/* mesh_unpool3d_gpu.cu:5-26 */
void oracle_unpool_forward(int nvFine, int C, const int32_t* vtReplace, const int32_t* vtMap, const float* in,
                           float* out) {
    memset(out, 0, sizeof(float) * (size_t)nvFine * C);
    for (int v = 0; v < nvFine; ++v) {
        int vi = cluster_of(v, vtReplace, vtMap);
        if (vi < 0) continue;
        for (int c = 0; c < C; ++c) out[(int64_t)v * C + c] = in[(int64_t)vi * C + c];
    }
}

/* mesh_unpool3d_gpu.cu:29-46 */
void oracle_unpool_backward(int nvFine, int nvCoarse, int C, const int32_t* vtReplace, const int32_t* vtMap,
                            const float* gout, float* gin) {
    memset(gin, 0, sizeof(float) * (size_t)nvCoarse * C);
    for (int v = 0; v < nvFine; ++v) {
        int vi = cluster_of(v, vtReplace, vtMap);
        if (vi < 0) continue;
        for (int c = 0; c < C; ++c) gin[(int64_t)vi * C + c] += gout[(int64_t)v * C + c];
    }
}

/* ---- point-cloud depthwise convolution, hard (coeff == NULL, T = 1) or fuzzy bin assignment;
 * picasso/point/pi_modules/source/pcloud_conv3d_gpu.cu:8-27,94-118 (forward), 30-48,121-147 (input
 * gradient), 51-88,150-193 (filter gradient); pairs in ascending order */
static float pcloud_weight(int p, int co, int Cr, int T, const int32_t* bin, const float* coeff, const float* filter) {
    if (!coeff) return filter[(int64_t)bin[p] * Cr + co];
    float w = 0;
    for (int t = 0; t < T; ++t) w += coeff[p * T + t] * filter[(int64_t)bin[p * T + t] * Cr + co];
    return w;
}

void oracle_pcloud_forward(int Mp, int Nout, int C, int r, int T, const int32_t* nnCount, const int32_t* nnIndex,
                           const int32_t* bin, const float* coeff, const float* in, const float* filter, float* out) {
    int Cr = C * r;
    memset(out, 0, sizeof(float) * (size_t)Mp * Cr);
    for (int p = 0; p < Nout; ++p) {
        int o = nnIndex[2 * p], i = nnIndex[2 * p + 1];
        for (int co = 0; co < Cr; ++co)
            out[(int64_t)o * Cr + co] += in[(int64_t)i * C + co / r] * pcloud_weight(p, co, Cr, T, bin, coeff, filter) / nnCount[o];
    }
}

void oracle_pcloud_backward(int Np, int Nout, int F, int C, int r, int T, const int32_t* nnCount, const int32_t* nnIndex,
                            const int32_t* bin, const float* coeff, const float* in, const float* filter,
                            const float* gout, float* gin, float* gfilter) {
    int Cr = C * r;
    memset(gin, 0, sizeof(float) * (size_t)Np * C);
    memset(gfilter, 0, sizeof(float) * (size_t)F * Cr);
    for (int p = 0; p < Nout; ++p) {
        int o = nnIndex[2 * p], i = nnIndex[2 * p + 1];
        for (int co = 0; co < Cr; ++co) {
            float g = gout[(int64_t)o * Cr + co];
            gin[(int64_t)i * C + co / r] += g * pcloud_weight(p, co, Cr, T, bin, coeff, filter) / nnCount[o];
            float d = g * in[(int64_t)i * C + co / r] / nnCount[o];
            if (!coeff) gfilter[(int64_t)bin[p] * Cr + co] += d;
            else for (int t = 0; t < T; ++t) gfilter[(int64_t)bin[p * T + t] * Cr + co] += coeff[p * T + t] * d;
        }
    }
}
#endif

// Core of the spherical-harmonic basis shared by the stand-alone kernel and the fused
// per-level preparation: constants evaluated as the reference evaluates them, and the
// per-point evaluation (projection to the unit sphere, angles, (L+1)^2 components).
#pragma once
#include <math.h>

namespace pb {

struct SphConst { float c[36]; };

// The reference evaluates each normalisation constant in fp32 from the fp32 value of pi
// (a python scalar combined with tensor(pi)); the same operations, in the same order,
// in IEEE fp32 on the host give the same bits.
static SphConst make_sph_const() {
    SphConst s;
    const float PI_F = (float)M_PI;
    auto q = [&](float num) { return sqrtf(num / PI_F); };             // sqrt(num/pi)
    auto qh = [&](float num) { return sqrtf(num / 2.f / PI_F); };      // sqrt(num/2/pi)
    float* c = s.c;
    c[0] = 0.5f * q(1.f);
    c[1] = 0.5f * qh(3.f);  c[2] = 0.5f * q(3.f);  c[3] = c[1];
    c[4] = 0.25f * qh(15.f); c[5] = 0.5f * qh(15.f); c[6] = 0.25f * q(5.f); c[7] = c[4]; c[8] = c[5];
    c[9] = 0.125f * q(35.f); c[10] = 0.25f * qh(105.f); c[11] = 0.125f * q(21.f); c[12] = 0.25f * q(7.f);
    c[13] = c[9]; c[14] = c[10]; c[15] = c[11];
    c[16] = (3.f / 16.f) * qh(35.f); c[17] = (3.f / 8.f) * q(35.f); c[18] = (3.f / 8.f) * qh(5.f);
    c[19] = (3.f / 8.f) * q(5.f); c[20] = (3.f / 16.f) * q(1.f);
    c[21] = c[16]; c[22] = c[17]; c[23] = c[18]; c[24] = c[19];
    c[25] = (3.f / 32.f) * q(77.f); c[26] = (3.f / 16.f) * qh(385.f); c[27] = (1.f / 32.f) * q(385.f);
    c[28] = (1.f / 8.f) * qh(1155.f); c[29] = (1.f / 16.f) * qh(165.f); c[30] = (1.f / 16.f) * q(11.f);
    c[31] = c[25]; c[32] = c[26]; c[33] = c[27]; c[34] = c[28]; c[35] = c[29];
    return s;
}

// o[0 .. (L+1)^2) = components of the direction (x, y, z); reference: picasso/mesh/layers.py:341-356
// (projection with +1e-10, azimuth in [0, 2pi), polar angle from +z) and picasso/math_utils.py:10-62.
__device__ __forceinline__ void sph_eval(float x, float y, float z, int L, const float* __restrict__ c, float* o) {
    const float PI_F = 3.14159265358979323846f;
    float l2 = sqrtf(__fadd_rn(__fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y)), __fmul_rn(z, z))) + 1e-10f;
    x = x / l2; y = y / l2; z = z / l2;
    float phi = atan2f(y, x);
    float theta = atan2f(z, sqrtf(__fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y))));
    if (phi < 0.f) phi += 2.f * PI_F;
    theta = PI_F / 2.f - theta;
    float st, ct;
    sincosf(theta, &st, &ct);
    o[0] = c[0];
    if (L >= 1) {
        float s1, c1;
        sincosf(phi, &s1, &c1);
        o[1] = c[1] * st * c1; o[2] = c[2] * ct; o[3] = c[3] * st * s1;
        if (L >= 2) {
            float s2, c2;
            sincosf(2.f * phi, &s2, &c2);
            float st2 = st * st, ct2 = ct * ct;
            o[4] = c[4] * st2 * c2; o[5] = c[5] * st * ct * c1; o[6] = c[6] * (3.f * ct2 - 1.f);
            o[7] = c[7] * st2 * s2; o[8] = c[8] * st * ct * s1;
            if (L >= 3) {
                float s3, c3;
                sincosf(3.f * phi, &s3, &c3);
                float st3 = st2 * st, ct3 = ct2 * ct;
                o[9] = c[9] * st3 * c3; o[10] = c[10] * st2 * ct * c2;
                o[11] = c[11] * st * (5.f * ct2 - 1.f) * c1; o[12] = c[12] * (5.f * ct3 - 3.f * ct);
                o[13] = c[13] * st3 * s3; o[14] = c[14] * st2 * ct * s2;
                o[15] = c[15] * st * (5.f * ct2 - 1.f) * s1;
                if (L >= 4) {
                    float s4, c4;
                    sincosf(4.f * phi, &s4, &c4);
                    float st4 = st2 * st2, ct4 = ct2 * ct2;
                    o[16] = c[16] * st4 * c4; o[17] = c[17] * st3 * ct * c3;
                    o[18] = c[18] * st2 * (7.f * ct2 - 1.f) * c2;
                    o[19] = c[19] * st * (7.f * ct3 - 3.f * ct) * c1;
                    o[20] = c[20] * (35.f * ct4 - 30.f * ct2 + 3.f);
                    o[21] = c[21] * st4 * s4; o[22] = c[22] * st3 * ct * s3;
                    o[23] = c[23] * st2 * (7.f * ct2 - 1.f) * s2;
                    o[24] = c[24] * st * (7.f * ct3 - 3.f * ct) * s1;
                    if (L >= 5) {
                        float s5, c5;
                        sincosf(5.f * phi, &s5, &c5);
                        float st5 = st4 * st, ct5 = ct4 * ct;
                        o[25] = c[25] * st5 * c5; o[26] = c[26] * st4 * ct * c4;
                        o[27] = c[27] * st3 * (9.f * ct2 - 1.f) * c3;
                        o[28] = c[28] * st2 * (3.f * ct3 - ct) * c2;
                        o[29] = c[29] * st * (21.f * ct4 - 14.f * ct2 + 1.f) * c1;
                        o[30] = c[30] * (63.f * ct5 - 70.f * ct3 + 15.f * ct);
                        o[31] = c[31] * st5 * s5; o[32] = c[32] * st4 * ct * s4;
                        o[33] = c[33] * st3 * (9.f * ct2 - 1.f) * s3;
                        o[34] = c[34] * st2 * (3.f * ct3 - ct) * s2;
                        o[35] = c[35] * st * (21.f * ct4 - 14.f * ct2 + 1.f) * s1;
                    }
                }
            }
        }
    }
}

}  // namespace pb

// Gradient of the per-edge quantities with respect to the edge vector, shared by the adjoint kernels.
#pragma once

#include "fmb_common.cuh"

namespace fmb {

// gradient of the 16 harmonics (component normalised, on the unit vector u) and of the length with respect to the
// edge vector: fastmace/kernels/triton/edge_sh.py:82-126 plus dr * u.
__device__ __forceinline__ void edge_vector_gradient(const float* g, float dr, float x, float y, float z, float len,
                                                     float (&q)[3]) {
    const float S3 = 1.7320508075688772f, S5 = 2.23606797749979f, S56 = 0.9128709291752769f, S38 = 0.6123724356957945f;
    const float C1 = 1.7320508075688772f, C2 = 2.23606797749979f, C3 = 2.6457513110645907f;
    const float g1x = g[1] * C1, g1y = g[2] * C1, g1z = g[3] * C1;
    const float g20 = g[4] * C2, g21 = g[5] * C2, g22 = g[6] * C2, g23 = g[7] * C2, g24 = g[8] * C2;
    const float g30 = g[9] * C3, g31 = g[10] * C3, g32 = g[11] * C3, g33 = g[12] * C3, g34 = g[13] * C3,
                g35 = g[14] * C3, g36 = g[15] * C3;
    const float s20 = S3 * x * z;
    const float s24 = S3 / 2.0f * (z * z - x * x);
    const float y2 = y * y;
    const float x2z2 = x * x + z * z;
    const float a = 4.0f * y2 - x2z2;
    const float b = 2.0f * y2 - 3.0f * x2z2;
    const float gs20 = g20 + S56 * (g30 * z - g36 * x) + S5 * g31 * y;
    const float gs24 = g24 + S56 * (g30 * x + g36 * z) + S5 * g35 * y;
    const float ga = S38 * (g32 * x + g34 * z);
    const float gb = 0.5f * y * g33;
    const float gy2 = g22 + 4.0f * ga + 2.0f * gb;
    const float gx2z2 = -0.5f * g22 - ga - 3.0f * gb;
    const float gx = g1x + S3 * z * gs20 + S3 * y * g21 - S3 * x * gs24 + 2.0f * x * gx2z2 +
                     S56 * (g30 * s24 - g36 * s20) + S38 * a * g32;
    const float gy = g1y + S3 * x * g21 + S3 * z * g23 + 2.0f * y * gy2 + S5 * (g31 * s20 + g35 * s24) + 0.5f * b * g33;
    const float gz = g1z + S3 * x * gs20 + S3 * y * g23 + S3 * z * gs24 + 2.0f * z * gx2z2 +
                     S56 * (g30 * s20 + g36 * s24) + S38 * a * g34;
    const float d = fmaxf(len, 1e-12f);
    const float dot = len > 1e-12f ? x * gx + y * gy + z * gz : 0.0f;
    q[0] = (gx - x * dot) / d + dr * x;
    q[1] = (gy - y * dot) / d + dr * y;
    q[2] = (gz - z * dot) / d + dr * z;
}

}  // namespace fmb

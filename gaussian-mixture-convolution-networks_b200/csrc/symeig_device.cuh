// Closed-form eigen-decomposition of one symmetric 2x2 / 3x3 matrix (device function shared by the symeig operator and
// the ellipsoid bounding boxes of the linear BVH).
#pragma once

#include <cuda_runtime.h>

namespace gmc {

// Closed-form eigen-decomposition of symmetric 2x2 / 3x3 matrices, one matrix per thread. Eigenvalues ascending,
// eigenvectors in the columns of the output matrix (torch.linalg.eigh convention).
// 2x2: lambda = T/2 -+ sqrt(|T^2/4 - det|), vectors from the numerically larger of (b, lambda - a) / (lambda - d, b).
// 3x3: trigonometric solution of the characteristic polynomial; the vector of an eigenvalue is the longest column of
// the product of (A - other eigenvalue I) over the two other eigenvalues, the third is the cross product.
// Same formulas and branch rules as the reference's src/gmc/cpp/extensions/math/symeig_detail.h:17-138 (including its
// shortcut "off-diagonal exactly zero -> identity eigenvectors" in 2D).
__device__ __forceinline__ void longest_column_normalised(const float* m, float* v) {
    float best = 0.f;
    int idx = 0;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        const float len = m[c] * m[c] + m[3 + c] * m[3 + c] + m[6 + c] * m[6 + c];
        if (len > best) { best = len; idx = c; }
    }
    const float inv = 1.f / sqrtf(best);
    v[0] = m[idx] * inv; v[1] = m[3 + idx] * inv; v[2] = m[6 + idx] * inv;
}

// A: row-major D x D (symmetric). val: D eigenvalues ascending. vec: row-major D x D with the eigenvectors in its columns.
template <int D>
__device__ __forceinline__ void symeig_device(const float* A, float* val, float* vec) {
    if constexpr (D == 2) {
        const float a = A[0], b = A[2], d = A[3];
        const float T = a + d, det = a * d - A[1] * A[2];
        const float f1 = T * 0.5f, f2 = sqrtf(fabsf(T * T * 0.25f - det));
        const float l0 = f1 - f2, l1 = f1 + f2;
        val[0] = l0; val[1] = l1;
        if (b == 0.f) { vec[0] = 1.f; vec[1] = 0.f; vec[2] = 0.f; vec[3] = 1.f; return; }
        float e0x, e0y, e1x, e1y;
        if (a < d) { e0x = b; e0y = l0 - a; e1x = b; e1y = l1 - a; }
        else { e0x = l0 - d; e0y = b; e1x = l1 - d; e1y = b; }
        const float n0 = 1.f / sqrtf(e0x * e0x + e0y * e0y), n1 = 1.f / sqrtf(e1x * e1x + e1y * e1y);
        vec[0] = e0x * n0; vec[1] = e1x * n1; vec[2] = e0y * n0; vec[3] = e1y * n1;
    } else {
        float m[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) m[k] = A[k];
        float eig0, eig1, eig2;   // eig2 <= eig1 <= eig0
        const float p1 = m[1] * m[1] + m[2] * m[2] + m[5] * m[5];
        if (p1 <= 0.0000001f) { eig0 = m[0]; eig1 = m[4]; eig2 = m[8]; }
        else {
            const float q = (m[0] + m[4] + m[8]) / 3.f;
            const float p2 = (m[0] - q) * (m[0] - q) + (m[4] - q) * (m[4] - q) + (m[8] - q) * (m[8] - q) + 2.f * p1;
            const float p = sqrtf(p2 / 6.f);
            float B[9];
#pragma unroll
            for (int k = 0; k < 9; ++k) B[k] = (m[k] - ((k % 4 == 0) ? q : 0.f)) / p;
            const float r = 0.5f * (B[0] * (B[4] * B[8] - B[5] * B[7]) - B[1] * (B[3] * B[8] - B[5] * B[6]) + B[2] * (B[3] * B[7] - B[4] * B[6]));
            const float pi = 3.14159265358979323846f;
            float phi;
            if (r <= -1.f) phi = pi / 3.f;
            else if (r >= 1.f) phi = 0.f;
            else phi = acosf(r) / 3.f;
            eig0 = q + 2.f * p * cosf(phi);
            eig2 = q + 2.f * p * cosf(phi + 2.f * pi / 3.f);
            eig1 = 3.f * q - eig0 - eig2;
        }
        auto shifted_product = [&](float s, float t, float* out) {   // (A - s I)(A - t I)
            float X[9], Y[9];
#pragma unroll
            for (int k = 0; k < 9; ++k) { X[k] = m[k] - ((k % 4 == 0) ? s : 0.f); Y[k] = m[k] - ((k % 4 == 0) ? t : 0.f); }
#pragma unroll
            for (int r2 = 0; r2 < 3; ++r2)
#pragma unroll
                for (int c = 0; c < 3; ++c) out[r2 * 3 + c] = X[r2 * 3] * Y[c] + X[r2 * 3 + 1] * Y[3 + c] + X[r2 * 3 + 2] * Y[6 + c];
        };
        float P[9], v0[3], v1[3], v2[3];
        shifted_product(eig1, eig2, P);
        longest_column_normalised(P, v0);
        shifted_product(eig0, eig2, P);
        longest_column_normalised(P, v1);
        v2[0] = v0[1] * v1[2] - v0[2] * v1[1];
        v2[1] = v0[2] * v1[0] - v0[0] * v1[2];
        v2[2] = v0[0] * v1[1] - v0[1] * v1[0];
        val[0] = eig2; val[1] = eig1; val[2] = eig0;
#pragma unroll
        for (int r2 = 0; r2 < 3; ++r2) { vec[r2 * 3 + 0] = v2[r2]; vec[r2 * 3 + 1] = v1[r2]; vec[r2 * 3 + 2] = v0[r2]; }
    }
}

}  // namespace gmc

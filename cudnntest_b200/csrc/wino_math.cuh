// The three Winograd transforms as fully unrolled register arithmetic, for F(4x4,3x3) (A = 6) and
// F(2x2,3x3) (A = 4).  Matrices of F(4x4,3x3) are the reference's:
//   B^T  comparison/wrapedConv_NCHW.cuh:836-855     G  :881-898     A^T  :1084-1101
// with G applied as multiplications by constants, not divisions.  F(2x2,3x3) uses the Lavin-Gray form.
#pragma once

namespace wino {

// Value types of the input transform: one float, or two floats (two channels) that go through the packed FP32
// instructions of sm_100 (add / fma .f32x2: one issue slot for both channels, each rounded like the scalar operation).
struct vf1 {
    float v;
};
struct vf2 {
    float2 v;
};
__device__ __forceinline__ vf1 vadd(vf1 a, vf1 b) { return {a.v + b.v}; }
__device__ __forceinline__ vf1 vsub(vf1 a, vf1 b) { return {a.v - b.v}; }
__device__ __forceinline__ vf1 vfma(float c, vf1 x, vf1 y) { return {fmaf(c, x.v, y.v)}; }            // c*x + y
__device__ __forceinline__ vf2 vadd(vf2 a, vf2 b) { return {__fadd2_rn(a.v, b.v)}; }
__device__ __forceinline__ vf2 vsub(vf2 a, vf2 b) { return {__ffma2_rn(make_float2(-1.f, -1.f), b.v, a.v)}; }   // exact: a - b, one rounding
__device__ __forceinline__ vf2 vfma(float c, vf2 x, vf2 y) { return {__ffma2_rn(make_float2(c, c), x.v, y.v)}; }

// 1-D input transform t = B^T d (rows of B^T: comparison/wrapedConv_NCHW.cuh:836-855), 14 operations for F(4x4,3x3)
template <int A, typename V>
__device__ __forceinline__ void bt_1d(const V (&d)[A], V (&t)[A]) {
    if constexpr (A == 6) {
        const V a = vadd(d[1], d[2]), b = vadd(d[3], d[4]);
        const V c = vsub(d[1], d[2]), e = vsub(d[4], d[3]);
        const V f = vsub(d[3], d[1]), g = vsub(d[4], d[2]);
        t[0] = vfma(4.f, d[0], vfma(-5.f, d[2], d[4]));
        t[1] = vfma(-4.f, a, b);
        t[2] = vfma(4.f, c, e);
        t[3] = vfma(2.f, f, g);
        t[4] = vfma(-2.f, f, g);
        t[5] = vfma(4.f, d[1], vfma(-5.f, d[3], d[5]));
    } else {
        t[0] = vsub(d[0], d[2]);
        t[1] = vadd(d[1], d[2]);
        t[2] = vsub(d[2], d[1]);
        t[3] = vsub(d[1], d[3]);
    }
}

// V = B^T d B for one A x A patch held in registers (row major d[r][s]); result v[i][j]
template <int A, typename V>
__device__ __forceinline__ void input_tile_transform(const V (&d)[A][A], V (&v)[A][A]) {
    V tmp[A][A];  // tmp[r][j] = sum_s d[r][s] B[s][j]
#pragma unroll
    for (int r = 0; r < A; ++r) bt_1d<A, V>(d[r], tmp[r]);
#pragma unroll
    for (int j = 0; j < A; ++j) {
        V col[A], out[A];
#pragma unroll
        for (int r = 0; r < A; ++r) col[r] = tmp[r][j];
        bt_1d<A, V>(col, out);
#pragma unroll
        for (int i = 0; i < A; ++i) v[i][j] = out[i];
    }
}

// 1-D filter transform u = G g
template <int A>
__device__ __forceinline__ void g_1d(const float (&g)[3], float (&u)[A]);

template <>
__device__ __forceinline__ void g_1d<6>(const float (&g)[3], float (&u)[6]) {
    const float s = g[0] + g[2];
    u[0] = 0.25f * g[0];
    u[1] = (-1.f / 6.f) * (s + g[1]);
    u[2] = (-1.f / 6.f) * (s - g[1]);
    const float q = (1.f / 24.f) * g[0] + (1.f / 6.f) * g[2];
    u[3] = q + (1.f / 12.f) * g[1];
    u[4] = q - (1.f / 12.f) * g[1];
    u[5] = g[2];
}
template <>
__device__ __forceinline__ void g_1d<4>(const float (&g)[3], float (&u)[4]) {
    const float s = g[0] + g[2];
    u[0] = g[0];
    u[1] = 0.5f * (s + g[1]);
    u[2] = 0.5f * (s - g[1]);
    u[3] = g[2];
}

template <int A>
__device__ __forceinline__ void filter_tile_transform(const float (&g)[3][3], float (&u)[A][A]) {
    float tmp[3][A];  // tmp[r][j] = sum_s g[r][s] G[j][s]
#pragma unroll
    for (int r = 0; r < 3; ++r) g_1d<A>(g[r], tmp[r]);
#pragma unroll
    for (int j = 0; j < A; ++j) {
        float col[3], out[A];
#pragma unroll
        for (int r = 0; r < 3; ++r) col[r] = tmp[r][j];
        g_1d<A>(col, out);
#pragma unroll
        for (int i = 0; i < A; ++i) u[i][j] = out[i];
    }
}

// 1-D output transform y = A^T m (rows of A^T: comparison/wrapedConv_NCHW.cuh:1084-1101), 10 operations for F(4x4,3x3)
template <int A, typename V>
__device__ __forceinline__ void at_1d(const V (&m)[A], V (&y)[A - 2]) {
    if constexpr (A == 6) {
        const V s12 = vadd(m[1], m[2]), d12 = vsub(m[1], m[2]);
        const V s34 = vadd(m[3], m[4]), d34 = vsub(m[3], m[4]);
        y[0] = vadd(vadd(m[0], s12), s34);
        y[1] = vfma(2.f, d34, d12);
        y[2] = vfma(4.f, s34, s12);
        y[3] = vadd(vfma(8.f, d34, d12), m[5]);
    } else {
        y[0] = vadd(vadd(m[0], m[1]), m[2]);
        y[1] = vsub(vsub(m[1], m[2]), m[3]);
    }
}
// plain-float front end (tile GEMM epilogues)
template <int A>
__device__ __forceinline__ void at_1d(const float (&m)[A], float (&y)[A - 2]) {
    vf1 mm[A], yy[A - 2];
#pragma unroll
    for (int i = 0; i < A; ++i) mm[i].v = m[i];
    at_1d<A, vf1>(mm, yy);
#pragma unroll
    for (int i = 0; i < A - 2; ++i) y[i] = yy[i].v;
}

// Y = A^T M A for one A x A tile of products (row major mm[i][j]); result y[p][q]
template <int A, typename V>
__device__ __forceinline__ void output_tile_transform(const V (&mm)[A][A], V (&y)[A - 2][A - 2]) {
    V tmp[A][A - 2];  // tmp[i][q] = sum_j mm[i][j] A[j][q]
#pragma unroll
    for (int i = 0; i < A; ++i) at_1d<A, V>(mm[i], tmp[i]);
#pragma unroll
    for (int q = 0; q < A - 2; ++q) {
        V col[A], out[A - 2];
#pragma unroll
        for (int i = 0; i < A; ++i) col[i] = tmp[i][q];
        at_1d<A, V>(col, out);
#pragma unroll
        for (int p = 0; p < A - 2; ++p) y[p][q] = out[p];
    }
}

__device__ __forceinline__ vf1 vmax(vf1 a, vf1 b) { return {fmaxf(a.v, b.v)}; }
__device__ __forceinline__ vf2 vmax(vf2 a, vf2 b) { return {make_float2(fmaxf(a.v.x, b.v.x), fmaxf(a.v.y, b.v.y))}; }
__device__ __forceinline__ vf1 vzero(vf1) { return {0.f}; }
__device__ __forceinline__ vf2 vzero(vf2) { return {make_float2(0.f, 0.f)}; }

}  // namespace wino

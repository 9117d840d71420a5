// Filter transform U = G g G^T.
//
// Replaces wino_kernel_trans_{nchw,nhwc,chwn}_suitFor128 of the reference
// (comparison/wrapedConv_NCHW.cuh:861-900, wrapedConv_NHWC.cuh:333-372, wrapedConv_CHWN.cuh:279-319).
// One thread per (filter k, channel c); reads the nine taps through the filter layout's strides and
// writes U[xi][k][Cp] with c fastest across the warp, zero filling c in [C, Cp).  HBM bound and tiny
// (9 -> a*a values per (k, c)); meant to run once per weight tensor, not once per forward.
#include <type_traits>

#include "common.cuh"
#include "wino_math.cuh"

namespace wino {

template <int A, typename TIn, typename TOp>
__global__ void __launch_bounds__(256) filter_transform_kernel(const TIn* __restrict__ w, TOp* __restrict__ u, int K,
                                                               int C, int Cp, Strides sw) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)K * Cp) return;
    const int c = (int)(idx % Cp);
    const int k = (int)(idx / Cp);
    float g[3][3];
    if (c < C) {
        const TIn* p = w + k * sw.n + c * sw.c;
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int s = 0; s < 3; ++s) g[r][s] = to_float<TIn>(p[r * sw.h + s * sw.w]);
    } else {
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int s = 0; s < 3; ++s) g[r][s] = 0.f;
    }
    float t[A][A];
    filter_tile_transform<A>(g, t);
    if constexpr (std::is_same<TOp, tf32x2_t>::value) {
        // split operands: rows of 2*Cp floats, the TF32 heads in [0, Cp), the TF32 tails in [Cp, 2*Cp)
        float* uf = reinterpret_cast<float*>(u);
        const long long plane = (long long)K * 2 * Cp, at = (long long)k * 2 * Cp + c;
#pragma unroll
        for (int i = 0; i < A; ++i)
#pragma unroll
            for (int j = 0; j < A; ++j) {
                const tf32x2_t sp = split_tf32(t[i][j]);
                uf[(long long)(i * A + j) * plane + at] = sp.hi;
                uf[(long long)(i * A + j) * plane + at + Cp] = sp.lo;
            }
    } else {
        const long long plane = (long long)K * Cp;
#pragma unroll
        for (int i = 0; i < A; ++i)
#pragma unroll
            for (int j = 0; j < A; ++j) u[(long long)(i * A + j) * plane + idx] = from_float<TOp>(t[i][j]);
    }
}

template <int A, typename TIn, typename TOp>
static int run(const wino_conv_desc& d, const Geometry& g, const void* w, void* u, cudaStream_t st) {
    const long long total = (long long)d.k * g.cp;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    ProfScope prof(STAGE_FILTER, st);
    count_launch();
    filter_transform_kernel<A, TIn, TOp><<<(unsigned)blocks, threads, 0, st>>>(
        (const TIn*)w, (TOp*)u, d.k, d.c, g.cp, filter_strides(d.layout_in, d.k, d.c));
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

template <int A>
static int dispatch(const wino_conv_desc& d, const Geometry& g, const void* w, void* u, cudaStream_t st) {
    switch (g.operand) {
        case OP_F32: return run<A, float, float>(d, g, w, u, st);
        case OP_TF32: return run<A, float, tf32_t>(d, g, w, u, st);
        case OP_TF32X3: return run<A, float, tf32x2_t>(d, g, w, u, st);
        case OP_BF16: return run<A, __nv_bfloat16, __nv_bfloat16>(d, g, w, u, st);
        case OP_F16: return run<A, __nv_bfloat16, __half>(d, g, w, u, st);
    }
    return fail(WINO_E_BADARG, "filter transform: bad operand kind %d", g.operand);
}

int launch_filter_transform(const wino_conv_desc& d, const Geometry& g, const void* w, void* u, cudaStream_t st) {
    return g.a == 6 ? dispatch<6>(d, g, w, u, st) : dispatch<4>(d, g, w, u, st);
}

}  // namespace wino

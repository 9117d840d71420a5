// Output transform Y = A^T M A fused with bias, ReLU, optional 2x2 max-pool and the scatter into
// NCHW / NHWC / CHWN.
//
// Replaces wino_invers_nchw_suitFor128_3 / _nhwc_suitFor128 / _chwn_suitFor128_2
// (comparison/wrapedConv_NCHW.cuh:1034-1114, wrapedConv_NHWC.cuh:376-428, wrapedConv_CHWN.cuh:379-431)
// and the separate bias / ReLU / pool passes the reference runs afterwards
// (netTest/cudnn_test_0124/VGG_Batched/Network.h:456-519, CHWN_support.cuh:85-120, :198-270, :480-527).
//
// Every layout reads the same product buffer M[xi][tile][Kq] (filters contiguous, 128 B per warp load)
// with one thread per (tile, filter); the layouts differ in the scatter:
//   * NHWC: the filter index is the contiguous output dimension, so the thread stores directly;
//   * NCHW: TX adjacent tiles x 32 filters are staged in shared memory and written as row segments
//     contiguous along w;
//   * CHWN: one tile position x 8 images x 32 filters are staged and written contiguous along n.
// HBM bound: reads a*a*T*K floats, writes N*K*OH*OW elements (a quarter of that with the pool).
// The NHWC kernel also reads products stored in 3 bytes (a plane of 16-bit upper halves and a plane of third bytes,
// written by the CTA-pair tile GEMM): one 4-byte and one 2-byte load and two prmt per pair of products.
#include <type_traits>

#include "common.cuh"
#include "wino_math.cuh"

namespace wino {

struct OTArgs {
    const void* m;       // products M[a*a][tp][kq] (float) or row-transformed Z[a*m][tp][kq] (float / half)
    const void* m_lo;    // 3-byte products: plane of the third bytes (m is then the plane of the upper 16 bits)
    const float* bias;
    void* y;
    int K;
    int oh, ow;   // conv output size
    int ph, pw;   // stored output size
    int n0, ns;
    int bny, bnx;
    int kq;
    long long tp;
    int relu, pool;
    Strides sy;   // strides of y (dims N, K, ph, pw)
};

constexpr int OT_KB = 32;
constexpr int OT_TX = 8;
constexpr int OT_NB = 8;

// Finishes the output transform of one (tile, filter) - or, with V = vf2, of two adjacent filters at once through the
// packed FP32 instructions - from the products held in registers, then bias, ReLU and (POOL) the 2x2 max.
// ZF = false: `in` holds the a*a raw products M and both 1-D transforms run here.
// ZF = true: `in` holds Z = M A (a*m values, written by the row-fused tile GEMM) and only A^T along i is left.
// res[p][q] holds the MO x MO stored outputs of the tile, MO = M or M/2.
template <int A, bool POOL, bool ZF, typename V>
__device__ __forceinline__ void finish_tile_v(const V (&in)[ZF ? A * (A - 2) : A * A], V b, int relu,
                                              V (&res)[POOL ? (A - 2) / 2 : (A - 2)][POOL ? (A - 2) / 2 : (A - 2)]) {
    constexpr int M = A - 2;
    V y[M][M];
    if constexpr (ZF) {
#pragma unroll
        for (int q = 0; q < M; ++q) {
            V col[A], out[M];
#pragma unroll
            for (int i = 0; i < A; ++i) col[i] = in[i * M + q];
            at_1d<A, V>(col, out);
#pragma unroll
            for (int p = 0; p < M; ++p) y[p][q] = out[p];
        }
    } else {
        V mm[A][A];
#pragma unroll
        for (int i = 0; i < A; ++i)
#pragma unroll
            for (int j = 0; j < A; ++j) mm[i][j] = in[i * A + j];
        output_tile_transform<A, V>(mm, y);
    }
#pragma unroll
    for (int p = 0; p < M; ++p)
#pragma unroll
        for (int q = 0; q < M; ++q) {
            V v = vadd(y[p][q], b);
            if (relu) v = vmax(v, vzero(v));
            y[p][q] = v;
        }
    if constexpr (POOL) {
#pragma unroll
        for (int p = 0; p < M / 2; ++p)
#pragma unroll
            for (int q = 0; q < M / 2; ++q)
                res[p][q] = vmax(vmax(y[2 * p][2 * q], y[2 * p][2 * q + 1]), vmax(y[2 * p + 1][2 * q], y[2 * p + 1][2 * q + 1]));
    } else {
#pragma unroll
        for (int p = 0; p < M; ++p)
#pragma unroll
            for (int q = 0; q < M; ++q) res[p][q] = y[p][q];
    }
}

// one filter, plain floats
template <int A, bool POOL, bool ZF>
__device__ __forceinline__ void finish_tile(const float (&in)[ZF ? A * (A - 2) : A * A], float b, int relu,
                                            float (&res)[POOL ? (A - 2) / 2 : (A - 2)][POOL ? (A - 2) / 2 : (A - 2)]) {
    constexpr int MO = POOL ? (A - 2) / 2 : (A - 2);
    constexpr int P = ZF ? A * (A - 2) : A * A;
    vf1 vin[P], vres[MO][MO];
#pragma unroll
    for (int i = 0; i < P; ++i) vin[i].v = in[i];
    finish_tile_v<A, POOL, ZF, vf1>(vin, vf1{b}, relu, vres);
#pragma unroll
    for (int p = 0; p < MO; ++p)
#pragma unroll
        for (int q = 0; q < MO; ++q) res[p][q] = vres[p][q].v;
}

// two adjacent filters: in[i] = (filter k, filter k + 1)
template <int A, bool POOL, bool ZF>
__device__ __forceinline__ void finish_tile_pair(const float2 (&in)[ZF ? A * (A - 2) : A * A], float b0, float b1, int relu,
                                                 float (&r0)[POOL ? (A - 2) / 2 : (A - 2)][POOL ? (A - 2) / 2 : (A - 2)],
                                                 float (&r1)[POOL ? (A - 2) / 2 : (A - 2)][POOL ? (A - 2) / 2 : (A - 2)]) {
    constexpr int MO = POOL ? (A - 2) / 2 : (A - 2);
    constexpr int P = ZF ? A * (A - 2) : A * A;
    vf2 vin[P], vres[MO][MO];
#pragma unroll
    for (int i = 0; i < P; ++i) vin[i].v = in[i];
    finish_tile_v<A, POOL, ZF, vf2>(vin, vf2{make_float2(b0, b1)}, relu, vres);
#pragma unroll
    for (int p = 0; p < MO; ++p)
#pragma unroll
        for (int q = 0; q < MO; ++q) { r0[p][q] = vres[p][q].v.x; r1[p][q] = vres[p][q].v.y; }
}

// one (tile t, filter k): scalar loads, lanes along k
template <int A, bool POOL, bool ZF, typename TP>
__device__ __forceinline__ void tile_outputs(const OTArgs& a, long long t, int k,
                                             float (&res)[POOL ? (A - 2) / 2 : (A - 2)][POOL ? (A - 2) / 2 : (A - 2)]) {
    constexpr int P = ZF ? A * (A - 2) : A * A;
    float in[P];
    const long long plane = a.tp * a.kq;
    const TP* src = reinterpret_cast<const TP*>(a.m) + t * a.kq + k;
#pragma unroll
    for (int i = 0; i < P; ++i) in[i] = to_float<TP>(src[(long long)i * plane]);
    finish_tile<A, POOL, ZF>(in, a.bias ? __ldg(a.bias + k) : 0.f, a.relu, res);
}

template <typename TP>
__device__ __forceinline__ float2 load_pair(const TP* p);
template <>
__device__ __forceinline__ float2 load_pair<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <>
__device__ __forceinline__ float2 load_pair<__half>(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }

// Raw products stored in 3 bytes: the upper 24 bits of the float (sign, exponent, 15 mantissa bits; the tile GEMM rounds
// to nearest), as one plane of 16-bit upper halves and one plane of third bytes with the same [a*a][tp][kq] indexing.
struct m24_t { unsigned short hi; };
__device__ __forceinline__ float2 load_pair_m24(const unsigned short* hi, const unsigned char* lo) {
    const uint32_t h = *reinterpret_cast<const uint32_t*>(hi);
    const uint32_t l = *reinterpret_cast<const unsigned short*>(lo);
    // float 0: bytes (0, lo.b0, hi.b0, hi.b1); float 1: bytes (0, lo.b1, hi.b2, hi.b3); selector 4 picks l.b0, 5 l.b1
    // (selector 7 is the top byte of the zero-extended 16-bit load: the low byte of each float is 0)
    const uint32_t f0 = __byte_perm(h, l, 0x1047);
    const uint32_t f1 = __byte_perm(h, l, 0x3257);
    return make_float2(__uint_as_float(f0), __uint_as_float(f1));
}

template <typename T>
__device__ __forceinline__ void store_pair(T* p, float a, float b);
template <>
__device__ __forceinline__ void store_pair<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// NHWC destination, two adjacent filters per thread (K even): every warp-wide load covers a full 128-byte (half
// products) or 256-byte (float products) row segment and every store a full 128 / 256-byte segment of y.
template <int A, bool POOL, bool ZF, typename TP, typename TOut>
__global__ void __launch_bounds__(256) output_transform_direct_x2(OTArgs a, long long T) {
    constexpr int MO = POOL ? (A - 2) / 2 : (A - 2);
    constexpr int P = ZF ? A * (A - 2) : A * A;
    const int kpairs = (a.K + 1) / 2;
    const int kspan = (kpairs + 31) / 32 * 32;
    const long long item = (long long)blockIdx.x * 256 + threadIdx.x;
    const int k = (int)(item % kspan) * 2;
    const long long t = item / kspan;
    if (t >= T || k >= a.K) return;
    float2 in[P];
    const long long plane = a.tp * a.kq;
    if constexpr (std::is_same<TP, m24_t>::value) {
        // both planes are below 4 GiB (the launcher checks): 32-bit offsets from the two plane bases
        const unsigned char* __restrict__ hi = reinterpret_cast<const unsigned char*>(a.m);
        const unsigned char* __restrict__ lo = reinterpret_cast<const unsigned char*>(a.m_lo);
        const unsigned off0 = (unsigned)(t * a.kq + k), pl = (unsigned)plane;
#pragma unroll
        for (int i = 0; i < P; ++i)
            in[i] = load_pair_m24(reinterpret_cast<const unsigned short*>(hi + 2u * (off0 + (unsigned)i * pl)), lo + (off0 + (unsigned)i * pl));
    } else {
        const TP* src = reinterpret_cast<const TP*>(a.m) + t * a.kq + k;
#pragma unroll
        for (int i = 0; i < P; ++i) in[i] = load_pair<TP>(src + (long long)i * plane);
    }
    float r0[MO][MO], r1[MO][MO];
    float b0 = 0.f, b1 = 0.f;
    if (a.bias) { b0 = __ldg(a.bias + k); b1 = __ldg(a.bias + k + 1); }
    finish_tile_pair<A, POOL, ZF>(in, b0, b1, a.relu, r0, r1);
    const int tiles_img = a.bny * a.bnx;
    const int n = a.n0 + (int)(t / tiles_img);
    const int rem = (int)(t % tiles_img);
    const int by = rem / a.bnx, bx = rem % a.bnx;
    TOut* __restrict__ y = (TOut*)a.y + (long long)n * a.sy.n + k;
#pragma unroll
    for (int p = 0; p < MO; ++p) {
        const int oy = by * MO + p;
        if (oy >= a.ph) continue;
#pragma unroll
        for (int q = 0; q < MO; ++q) {
            const int ox = bx * MO + q;
            if (ox < a.pw) store_pair<TOut>(y + oy * a.sy.h + ox * a.sy.w, r0[p][q], r1[p][q]);
        }
    }
}

// NHWC destination: direct store, lanes along k
template <int A, bool POOL, bool ZF, typename TP, typename TOut>
__global__ void __launch_bounds__(256) output_transform_direct(OTArgs a, long long T) {
    constexpr int MO = POOL ? (A - 2) / 2 : (A - 2);
    const int kchunks = (a.K + OT_KB - 1) / OT_KB;
    const long long item = (long long)blockIdx.x * 256 + threadIdx.x;
    const int k = (int)(item % (kchunks * OT_KB));
    const long long t = item / (kchunks * OT_KB);
    if (t >= T || k >= a.K) return;
    float res[MO][MO];
    tile_outputs<A, POOL, ZF, TP>(a, t, k, res);
    const int tiles_img = a.bny * a.bnx;
    const int n = a.n0 + (int)(t / tiles_img);
    const int rem = (int)(t % tiles_img);
    const int by = rem / a.bnx, bx = rem % a.bnx;
    TOut* __restrict__ y = (TOut*)a.y + (long long)n * a.sy.n + (long long)k * a.sy.c;
#pragma unroll
    for (int p = 0; p < MO; ++p) {
        const int oy = by * MO + p;
        if (oy >= a.ph) continue;
#pragma unroll
        for (int q = 0; q < MO; ++q) {
            const int ox = bx * MO + q;
            if (ox < a.pw) y[oy * a.sy.h + ox * a.sy.w] = from_float<TOut>(res[p][q]);
        }
    }
}

// packs VE consecutive outputs into one 16-byte vector
template <typename TOut>
__device__ __forceinline__ uint4 pack16(const float* v);
template <>
__device__ __forceinline__ uint4 pack16<float>(const float* v) {
    return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
}
template <>
__device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
        w[e] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Transform step shared by the NCHW and CHWN kernels: the thread loads the products of two adjacent filters
// (k, k+1) of tile t — always inside the Kq-padded rows — and leaves the MO x MO outputs of both in the staging
// array at [pos(p, q)][k_l], [pos][k_l + 1].
template <int A, bool POOL, bool ZF, typename TP, typename PosFn>
__device__ __forceinline__ void stage_pair(const OTArgs& a, long long t, int k, int k_l, float* stage, int pitch, PosFn pos) {
    constexpr int MO = POOL ? (A - 2) / 2 : (A - 2);
    constexpr int P = ZF ? A * (A - 2) : A * A;
    float2 in[P];
    const long long plane = a.tp * a.kq;
    const TP* src = reinterpret_cast<const TP*>(a.m) + t * a.kq + k;
#pragma unroll
    for (int i = 0; i < P; ++i) in[i] = load_pair<TP>(src + (long long)i * plane);
    float r0[MO][MO], r1[MO][MO];
    float b0 = 0.f, b1 = 0.f;
    if (a.bias) {
        b0 = k < a.K ? __ldg(a.bias + k) : 0.f;
        b1 = k + 1 < a.K ? __ldg(a.bias + k + 1) : 0.f;
    }
    finish_tile_pair<A, POOL, ZF>(in, b0, b1, a.relu, r0, r1);
#pragma unroll
    for (int p = 0; p < MO; ++p)
#pragma unroll
        for (int q = 0; q < MO; ++q) {
            float* dst = stage + pos(p, q) * pitch + k_l;
            dst[0] = r0[p][q];
            dst[1] = r1[p][q];
        }
}

constexpr int OT_KB2 = 64;          // filters per CTA of the staged kernels
constexpr int OT_PITCH = OT_KB2 + 1;

// NCHW destination: 8 adjacent tiles x 64 filters are staged, then written as 16-byte vectors along w (consecutive
// lanes cover consecutive vectors of one output row, so a row segment of 8 tiles goes out as one contiguous run).
template <int A, bool POOL, bool ZF, typename TP, typename TOut>
__global__ void __launch_bounds__(256, 2) output_transform_strip(const OTArgs a) {
    constexpr int MO = POOL ? (A - 2) / 2 : (A - 2);
    constexpr int COLS = MO * OT_TX;
    constexpr int VE = 16 / (int)sizeof(TOut);
    constexpr int NVEC = COLS / VE;
    static_assert(COLS % VE == 0 || COLS < VE, "row segment must split into whole vectors");
    __shared__ float stage[MO * COLS * OT_PITCH];

    const int kchunks = (a.K + OT_KB2 - 1) / OT_KB2;
    const int k0 = (blockIdx.x % kchunks) * OT_KB2;
    const int bx0 = (blockIdx.x / kchunks) * OT_TX;
    const int by = blockIdx.y;
    const int n = a.n0 + blockIdx.z;
    {
        const int lane = threadIdx.x % 32, tl = threadIdx.x / 32;
        const int bx = bx0 + tl, k = k0 + 2 * lane;
        if (bx < a.bnx && k < a.K) {
            const long long t = ((long long)blockIdx.z * a.bny + by) * a.bnx + bx;
            stage_pair<A, POOL, ZF, TP>(a, t, k, 2 * lane, stage, OT_PITCH, [&](int p, int q) { return p * COLS + tl * MO + q; });
        }
    }
    __syncthreads();
    TOut* __restrict__ y = (TOut*)a.y + (long long)n * a.sy.n;
    const int ox0 = bx0 * MO;
    const bool vec_ok = NVEC > 0 && (a.pw % VE) == 0 && ((a.sy.n | a.sy.c) % VE) == 0 && (reinterpret_cast<uintptr_t>(a.y) & 15) == 0;
    if (vec_ok) {
        for (int idx = threadIdx.x; idx < MO * OT_KB2 * NVEC; idx += 256) {
            const int vec = idx % NVEC;
            const int rk = idx / NVEC;
            const int k_l = rk % OT_KB2, p = rk / OT_KB2;
            const int oy = by * MO + p, ox = ox0 + vec * VE, k = k0 + k_l;
            if (oy >= a.ph || k >= a.K || ox >= a.pw) continue;
            float v[VE];
#pragma unroll
            for (int e = 0; e < VE; ++e) v[e] = stage[(p * COLS + vec * VE + e) * OT_PITCH + k_l];
            TOut* dst = y + (long long)k * a.sy.c + oy * a.sy.h + ox;
            if (ox + VE <= a.pw) {
                *reinterpret_cast<uint4*>(dst) = pack16<TOut>(v);
            } else {
                for (int e = 0; e < VE && ox + e < a.pw; ++e) dst[e] = from_float<TOut>(v[e]);
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < MO * COLS * OT_KB2; idx += 256) {
            const int col = idx % COLS;
            const int rk = idx / COLS;
            const int k_l = rk % OT_KB2, p = rk / OT_KB2;
            const int oy = by * MO + p, ox = ox0 + col, k = k0 + k_l;
            if (oy < a.ph && ox < a.pw && k < a.K)
                y[(long long)k * a.sy.c + oy * a.sy.h + ox * a.sy.w] = from_float<TOut>(stage[(p * COLS + col) * OT_PITCH + k_l]);
        }
    }
}

// CHWN destination: one tile position x 8 images x 64 filters are staged, then written as 16-byte vectors along n
template <int A, bool POOL, bool ZF, typename TP, typename TOut>
__global__ void __launch_bounds__(256, 2) output_transform_batch(const OTArgs a) {
    constexpr int MO = POOL ? (A - 2) / 2 : (A - 2);
    constexpr int VE = 16 / (int)sizeof(TOut);       // images per vector: 8 (bf16) or 4 (float)
    constexpr int NVEC = OT_NB / VE;
    __shared__ float stage[MO * MO * OT_NB * OT_PITCH];

    const int kchunks = (a.K + OT_KB2 - 1) / OT_KB2;
    const int k0 = (blockIdx.x % kchunks) * OT_KB2;
    const int nb0 = (blockIdx.x / kchunks) * OT_NB;
    const int bx = blockIdx.y, by = blockIdx.z;
    {
        const int lane = threadIdx.x % 32, n_l = threadIdx.x / 32;
        const int k = k0 + 2 * lane;
        if (nb0 + n_l < a.ns && k < a.K) {
            const long long t = ((long long)(nb0 + n_l) * a.bny + by) * a.bnx + bx;
            stage_pair<A, POOL, ZF, TP>(a, t, k, 2 * lane, stage, OT_PITCH, [&](int p, int q) { return (p * MO + q) * OT_NB + n_l; });
        }
    }
    __syncthreads();
    TOut* __restrict__ y = (TOut*)a.y;
    const int nbase = a.n0 + nb0;
    const bool vec_ok = ((a.sy.c | a.sy.h | a.sy.w) % VE) == 0 && (nbase % VE) == 0 && (reinterpret_cast<uintptr_t>(a.y) & 15) == 0;
    // the NVEC vectors of one (filter, pixel) - 32 contiguous bytes for float output - go to adjacent lanes, so a warp
    // writes whole sectors
    for (int idx = threadIdx.x; idx < MO * MO * OT_KB2 * NVEC; idx += 256) {
        const int vec = idx % NVEC;
        const int rk = idx / NVEC;
        const int k_l = rk % OT_KB2, pq = rk / OT_KB2;
        const int oy = by * MO + pq / MO, ox = bx * MO + pq % MO, k = k0 + k_l;
        const int n_l0 = vec * VE;
        if (oy >= a.ph || ox >= a.pw || k >= a.K || nb0 + n_l0 >= a.ns) continue;
        float v[VE];
#pragma unroll
        for (int e = 0; e < VE; ++e) v[e] = stage[(pq * OT_NB + n_l0 + e) * OT_PITCH + k_l];
        TOut* dst = y + (long long)k * a.sy.c + oy * a.sy.h + ox * a.sy.w + (nbase + n_l0);
        if (vec_ok && nb0 + n_l0 + VE <= a.ns) {
            *reinterpret_cast<uint4*>(dst) = pack16<TOut>(v);
        } else {
            for (int e = 0; e < VE && nb0 + n_l0 + e < a.ns; ++e) dst[e] = from_float<TOut>(v[e]);
        }
    }
}

template <int A, bool POOL, bool ZF, typename TP, typename TOut>
static int run(const wino_conv_desc& d, const Geometry& g, const OTArgs& a, cudaStream_t st) {
    const int kchunks = (d.k + OT_KB - 1) / OT_KB, kchunks2 = (d.k + OT_KB2 - 1) / OT_KB2;
    ProfScope prof(STAGE_OUTPUT, st);
    count_launch();
    if (d.layout_out == WINO_NHWC && d.k % 2 == 0 && ((uintptr_t)a.m & 7) == 0 && ((uintptr_t)a.y & 7) == 0) {
        const long long T = (long long)a.ns * g.tiles_img;
        const long long items = T * (((d.k / 2) + 31) / 32 * 32);
        output_transform_direct_x2<A, POOL, ZF, TP, TOut><<<(unsigned)((items + 255) / 256), 256, 0, st>>>(a, T);
    } else if (d.layout_out == WINO_NHWC) {
        const long long T = (long long)a.ns * g.tiles_img;
        const long long items = T * kchunks * OT_KB;
        output_transform_direct<A, POOL, ZF, TP, TOut><<<(unsigned)((items + 255) / 256), 256, 0, st>>>(a, T);
    } else if (d.layout_out == WINO_NCHW) {
        dim3 grid((unsigned)(((g.bnx + OT_TX - 1) / OT_TX) * kchunks2), (unsigned)g.bny, (unsigned)a.ns);
        output_transform_strip<A, POOL, ZF, TP, TOut><<<grid, 256, 0, st>>>(a);
    } else {
        dim3 grid((unsigned)(((a.ns + OT_NB - 1) / OT_NB) * kchunks2), (unsigned)g.bnx, (unsigned)g.bny);
        output_transform_batch<A, POOL, ZF, TP, TOut><<<grid, 256, 0, st>>>(a);
    }
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

template <int A, bool ZF, typename TP>
static int dispatch(const wino_conv_desc& d, const Geometry& g, const OTArgs& a, cudaStream_t st) {
    const bool bf16 = g.out_bf16 != 0;
    if (d.pool2x2)
        return bf16 ? run<A, true, ZF, TP, __nv_bfloat16>(d, g, a, st) : run<A, true, ZF, TP, float>(d, g, a, st);
    return bf16 ? run<A, false, ZF, TP, __nv_bfloat16>(d, g, a, st) : run<A, false, ZF, TP, float>(d, g, a, st);
}

// 3-byte products exist for the NHWC two-filters-per-thread kernel only (the caller checks output_transform_m24_ok)
template <int A>
static int run_m24(const wino_conv_desc& d, const Geometry& g, const OTArgs& a, cudaStream_t st) {
    ProfScope prof(STAGE_OUTPUT, st);
    count_launch();
    const long long T = (long long)a.ns * g.tiles_img;
    const long long items = T * (((d.k / 2) + 31) / 32 * 32);
    const unsigned blocks = (unsigned)((items + 255) / 256);
    const bool bf16 = g.out_bf16 != 0;
    if (d.pool2x2) {
        if (bf16) output_transform_direct_x2<A, true, false, m24_t, __nv_bfloat16><<<blocks, 256, 0, st>>>(a, T);
        else output_transform_direct_x2<A, true, false, m24_t, float><<<blocks, 256, 0, st>>>(a, T);
    } else {
        if (bf16) output_transform_direct_x2<A, false, false, m24_t, __nv_bfloat16><<<blocks, 256, 0, st>>>(a, T);
        else output_transform_direct_x2<A, false, false, m24_t, float><<<blocks, 256, 0, st>>>(a, T);
    }
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

bool output_transform_m24_ok(const wino_conv_desc& d, const void* y) {
    return d.layout_out == WINO_NHWC && d.k % 2 == 0 && ((uintptr_t)y & 7) == 0;
}

// prod_kind: 0 = raw products M (float), 1 = row-transformed Z (float), 2 = row-transformed Z (half), 3 = raw products in 3 bytes (two planes)
int launch_output_transform(const wino_conv_desc& d, const Geometry& g, const void* m, int prod_kind, const float* bias,
                            void* y, int n0, int ns, long long tp, cudaStream_t st) {
    if (ns <= 0) return WINO_OK;
    if (ns > 65535 || g.bny > 65535 || g.bnx > 65535)
        return fail(WINO_E_UNSUPPORTED, "output transform: slab of %d images / %dx%d tiles exceeds the grid limits", ns,
                    g.bny, g.bnx);
    OTArgs a;
    a.m = m; a.m_lo = nullptr; a.bias = d.has_bias ? bias : nullptr; a.y = y; a.K = d.k;
    a.oh = g.oh; a.ow = g.ow; a.ph = g.ph; a.pw = g.pw;
    a.n0 = n0; a.ns = ns; a.bny = g.bny; a.bnx = g.bnx; a.kq = g.kq; a.tp = tp;
    a.relu = d.relu; a.pool = d.pool2x2;
    a.sy = act_strides(d.layout_out, d.n, d.k, g.ph, g.pw);
    if (prod_kind == 0) return g.a == 6 ? dispatch<6, false, float>(d, g, a, st) : dispatch<4, false, float>(d, g, a, st);
    if (prod_kind == 1) return g.a == 6 ? dispatch<6, true, float>(d, g, a, st) : dispatch<4, true, float>(d, g, a, st);
    if (prod_kind == 2) return g.a == 6 ? dispatch<6, true, __half>(d, g, a, st) : dispatch<4, true, __half>(d, g, a, st);
    if (prod_kind == 3) {
        if (!output_transform_m24_ok(d, y) || ((uintptr_t)m & 15))
            return fail(WINO_E_BADARG, "output transform: 3-byte products need an NHWC destination and an even filter count");
        if ((long long)g.a * g.a * tp * g.kq * 2 >= (1LL << 32))
            return fail(WINO_E_UNSUPPORTED, "output transform: 3-byte product planes are limited to 4 GiB per slab");
        a.m_lo = (const char*)m + (long long)g.a * g.a * tp * g.kq * 2;
        return g.a == 6 ? run_m24<6>(d, g, a, st) : run_m24<4>(d, g, a, st);
    }
    return fail(WINO_E_BADARG, "output transform: bad product kind %d", prod_kind);
}

}  // namespace wino

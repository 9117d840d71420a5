// Input transform V = B^T d B fused with the gather from NCHW / NHWC / CHWN.
//
// Replaces wino_input_trans_nchw_suitFor128_2 / _nhwc_suitFor128 / _chwn_suitFor128
// (comparison/wrapedConv_NCHW.cuh:760-856, wrapedConv_NHWC.cuh:266-329, wrapedConv_CHWN.cuh:225-275),
// which map one thread to one (tile, channel) and issue a*a scalar stores at plane stride.
//
// Design: every layout writes the same operand buffer V[xi][tile][Cp] (channels contiguous = the
// K-major operand the tile GEMM wants), so the layouts differ only in how a CTA stages its input
// patch in shared memory:
//   * NHWC, NCHW ("strip"): a CTA owns TX horizontally adjacent tiles x 32 channels of one image row
//     of tiles; it stages the a x (m*TX+2) x 32 halo patch once (the horizontal halo is read once, not
//     1.5x), with global loads coalesced along c (NHWC) or along w (NCHW); zero padding is the loader's
//     predicate.
//   * CHWN ("batch"): a CTA owns one tile position x 8 images x 32 channels, loads coalesced along n.
// Shared memory is [position][channel] with a row pitch chosen so that both the layout's load order
// and the transform's read order (lanes along c) are bank-conflict free.  Then each thread transforms
// one (tile, channel) patch in registers and the warp stores 32 consecutive channels per (xi, tile).
// HBM bound: reads N*C*H*W elements (x ~1.5 through L2 for the vertical halo), writes a*a*T*Cp.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "wino_math.cuh"

namespace wino {

// WINO_GENERIC_TRANSFORMS=1 routes every layout through the generic staged kernels (testing aid)
static bool force_generic() {
    static const bool v = [] { const char* e = getenv("WINO_GENERIC_TRANSFORMS"); return e && e[0] == '1'; }();
    return v;
}

struct ITArgs {
    const void* x;
    void* v;
    int C, H, W, pad;
    int n0, ns;
    int bny, bnx;
    int cp;
    long long tp;
    Strides sx;
};

constexpr int IT_CB = 32;   // channels per CTA
constexpr int IT_TX = 8;    // tiles per CTA along x (strip mode)
constexpr int IT_NB = 8;    // images per CTA (batch mode)

template <int A, typename TOp>
__device__ __forceinline__ void transform_and_store(const float* patch, int pos_stride_r, int pos_stride_s, int pitch,
                                                    int c_l, TOp* __restrict__ v, long long tp, int cp, long long t,
                                                    int c) {
    float d[A][A], o[A][A];
#pragma unroll
    for (int r = 0; r < A; ++r)
#pragma unroll
        for (int s = 0; s < A; ++s) d[r][s] = patch[(r * pos_stride_r + s * pos_stride_s) * pitch + c_l];
    input_tile_transform<A>(d, o);
    const long long plane = tp * cp;
    TOp* dst = v + t * cp + c;
#pragma unroll
    for (int i = 0; i < A; ++i)
#pragma unroll
        for (int j = 0; j < A; ++j) dst[(long long)(i * A + j) * plane] = from_float<TOp>(o[i][j]);
}

// strip mode: NHWC (W_FASTEST = false) and NCHW (W_FASTEST = true)
template <int A, bool W_FASTEST, typename TIn, typename TOp>
__global__ void __launch_bounds__(256) input_transform_strip(ITArgs a) {
    constexpr int M = A - 2;
    constexpr int COLS = M * IT_TX + 2;
    constexpr int PITCH = IT_CB + 1;
    __shared__ float patch[A * COLS * PITCH];

    const int cchunks = (a.cp + IT_CB - 1) / IT_CB;
    const int c0 = (blockIdx.x % cchunks) * IT_CB;
    const int bx0 = (blockIdx.x / cchunks) * IT_TX;
    const int by = blockIdx.y;
    const int n = a.n0 + blockIdx.z;
    const int gh0 = by * M - a.pad, gw0 = bx0 * M - a.pad;
    const TIn* __restrict__ x = (const TIn*)a.x + (long long)n * a.sx.n;

    for (int idx = threadIdx.x; idx < A * COLS * IT_CB; idx += 256) {
        int c_l, col, r;
        if (W_FASTEST) {
            col = idx % COLS;
            const int rc = idx / COLS;
            c_l = rc % IT_CB;
            r = rc / IT_CB;
        } else {
            c_l = idx % IT_CB;
            const int rc = idx / IT_CB;
            col = rc % COLS;
            r = rc / COLS;
        }
        const int gh = gh0 + r, gw = gw0 + col, c = c0 + c_l;
        float val = 0.f;
        if (gh >= 0 && gh < a.H && gw >= 0 && gw < a.W && c < a.C)
            val = to_float<TIn>(x[c * a.sx.c + gh * a.sx.h + gw * a.sx.w]);
        patch[(r * COLS + col) * PITCH + c_l] = val;
    }
    __syncthreads();

    const int item = threadIdx.x;  // IT_TX * IT_CB == 256
    const int c_l = item % IT_CB, tl = item / IT_CB;
    const int bx = bx0 + tl, c = c0 + c_l;
    if (bx < a.bnx && c < a.cp) {
        const long long t = ((long long)blockIdx.z * a.bny + by) * a.bnx + bx;
        transform_and_store<A, TOp>(patch + tl * M * PITCH, COLS, 1, PITCH, c_l, (TOp*)a.v, a.tp, a.cp, t, c);
    }
}

// batch mode: CHWN
template <int A, typename TIn, typename TOp>
__global__ void __launch_bounds__(256) input_transform_batch(ITArgs a) {
    constexpr int M = A - 2;
    constexpr int PITCH = IT_CB + 4;  // lanes (n_l, c_l) -> bank 4*n_l + c_l on store, c_l on load
    __shared__ float patch[A * A * IT_NB * PITCH];

    const int cchunks = (a.cp + IT_CB - 1) / IT_CB;
    const int c0 = (blockIdx.x % cchunks) * IT_CB;
    const int nb0 = (blockIdx.x / cchunks) * IT_NB;
    const int bx = blockIdx.y, by = blockIdx.z;
    const int gh0 = by * M - a.pad, gw0 = bx * M - a.pad;
    const TIn* __restrict__ x = (const TIn*)a.x;

    for (int idx = threadIdx.x; idx < A * A * IT_NB * IT_CB; idx += 256) {
        const int n_l = idx % IT_NB;
        const int rc = idx / IT_NB;
        const int c_l = rc % IT_CB;
        const int rs = rc / IT_CB;
        const int gh = gh0 + rs / A, gw = gw0 + rs % A, c = c0 + c_l;
        float val = 0.f;
        if (gh >= 0 && gh < a.H && gw >= 0 && gw < a.W && c < a.C && nb0 + n_l < a.ns)
            val = to_float<TIn>(x[(long long)(a.n0 + nb0 + n_l) * a.sx.n + c * a.sx.c + gh * a.sx.h + gw * a.sx.w]);
        patch[(rs * IT_NB + n_l) * PITCH + c_l] = val;
    }
    __syncthreads();

    const int item = threadIdx.x;  // IT_NB * IT_CB == 256
    const int c_l = item % IT_CB, n_l = item / IT_CB;
    const int c = c0 + c_l;
    if (nb0 + n_l < a.ns && c < a.cp) {
        const long long t = ((long long)(nb0 + n_l) * a.bny + by) * a.bnx + bx;
        transform_and_store<A, TOp>(patch + n_l * PITCH, A * IT_NB, IT_NB, PITCH, c_l, (TOp*)a.v, a.tp, a.cp, t, c);
    }
}

// ---- NHWC fast path: TMA-staged, persistent ---------------------------------------------------------
// Used when the pixel pitch C*sizeof(T) is a multiple of 16 bytes (TMA's stride rule).  A CTA walks work
// units (image, tile row, 8 adjacent tiles, 128 bytes of channels) round-robin; one elected thread brings
// each unit's a x (8m+2) x 128-byte halo patch into a 3-deep shared-memory ring with a single 4-D
// cp.async.bulk.tensor load whose out-of-range rows, columns and channels are zero filled by the TMA unit
// (= the convolution's zero padding and the Cp padding of V, with no predicates in the kernel).  Warp w owns
// tile w of the unit, lane l owns the l-th 4-byte word of the 128-byte channel chunk (two bf16 or one float
// channel): shared-memory reads are conflict free and every global store instruction writes one full 128-byte
// line of V.
constexpr int ITT_STAGES = 3;
constexpr int ITT_WAIT_CODE = 5;

template <typename TIn, typename TOp>
struct WordIO;
template <typename TOp>
struct WordIO<float, TOp> {          // one float channel per word
    static constexpr int VEC = 1;
    static __device__ __forceinline__ float get(uint32_t w, int) { return __uint_as_float(w); }
    static __device__ __forceinline__ uint32_t put(float a, float) {
        return __float_as_uint(to_float<TOp>(from_float<TOp>(a)));
    }
};
template <>
struct WordIO<__nv_bfloat16, __nv_bfloat16> {
    static constexpr int VEC = 2;
    static __device__ __forceinline__ float get(uint32_t w, int i) { return __uint_as_float(i ? (w & 0xffff0000u) : (w << 16)); }
    static __device__ __forceinline__ uint32_t put(float a, float b) {
        __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&p);
    }
};
template <>
struct WordIO<__nv_bfloat16, __half> {
    static constexpr int VEC = 2;
    static __device__ __forceinline__ float get(uint32_t w, int i) { return __uint_as_float(i ? (w & 0xffff0000u) : (w << 16)); }
    static __device__ __forceinline__ uint32_t put(float a, float b) {
        __half2 p = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&p);
    }
};

template <int A, typename TIn, typename TOp>
__global__ void __launch_bounds__(256, 2)
input_transform_nhwc_tma(const __grid_constant__ CUtensorMap tm_x, const ITArgs a, const int bxchunks, const int cchunks,
                         const long long units, int* status) {
    using IO = WordIO<TIn, TOp>;
    constexpr int M = A - 2;
    constexpr int COLS = M * IT_TX + 2;
    constexpr int VEC = IO::VEC;
    constexpr int CH = 32 * VEC;                       // channels per unit (128 bytes)
    constexpr int STAGE_BYTES = A * COLS * 128;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t ring = smem_u32(smem);
    const uint32_t bars = ring + ITT_STAGES * STAGE_BYTES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + ITT_STAGES * STAGE_BYTES + 8 * ITT_STAGES);

    const long long first = blockIdx.x;
    const long long n_my = first < units ? (units - first + gridDim.x - 1) / gridDim.x : 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < ITT_STAGES; ++s) mbar_init(bars + 8 * s, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    auto decode = [&](long long i, int& n_l, int& by, int& bx0, int& c0) {
        long long u = first + i * gridDim.x;
        c0 = (int)(u % cchunks) * CH; u /= cchunks;
        bx0 = (int)(u % bxchunks) * IT_TX; u /= bxchunks;
        by = (int)(u % a.bny);
        n_l = (int)(u / a.bny);
    };
    auto issue = [&](long long i) {
        int n_l, by, bx0, c0;
        decode(i, n_l, by, bx0, c0);
        const int s = (int)(i % ITT_STAGES);
        mbar_arrive_expect_tx(bars + 8 * s, STAGE_BYTES);
        tma_load_4d(ring + s * STAGE_BYTES, &tm_x, bars + 8 * s, c0, bx0 * M - a.pad, by * M - a.pad, a.n0 + n_l);
    };
    if (threadIdx.x == 0)
        for (long long i = 0; i < n_my && i < ITT_STAGES - 1; ++i) issue(i);

    const int tl = threadIdx.x / 32, lane = threadIdx.x % 32;
    const long long plane_words = a.tp * a.cp / VEC;
    uint32_t* __restrict__ vw = reinterpret_cast<uint32_t*>(a.v);
    bool aborted = false;
    for (long long i = 0; i < n_my; ++i) {
        if (threadIdx.x == 0 && i + ITT_STAGES - 1 < n_my) issue(i + ITT_STAGES - 1);
        const int s = (int)(i % ITT_STAGES);
        bool ok = mbar_wait_bounded(bars + 8 * s, (uint32_t)((i / ITT_STAGES) & 1), abort_flag, status, ITT_WAIT_CODE);
        if (!__syncthreads_and(ok)) { aborted = true; break; }
        int n_l, by, bx0, c0;
        decode(i, n_l, by, bx0, c0);
        const int bx = bx0 + tl, c = c0 + lane * VEC;
        if (bx < a.bnx && c < a.cp) {
            const uint32_t* src = reinterpret_cast<const uint32_t*>(smem + s * STAGE_BYTES) + (tl * M) * 32 + lane;
            uint32_t w[A][A];
#pragma unroll
            for (int r = 0; r < A; ++r)
#pragma unroll
                for (int q = 0; q < A; ++q) w[r][q] = src[(r * COLS + q) * 32];
            float d[A][A], lo[A][A], hi[A][A];
#pragma unroll
            for (int r = 0; r < A; ++r)
#pragma unroll
                for (int q = 0; q < A; ++q) d[r][q] = IO::get(w[r][q], 0);
            input_tile_transform<A>(d, lo);
            if (VEC == 2) {
#pragma unroll
                for (int r = 0; r < A; ++r)
#pragma unroll
                    for (int q = 0; q < A; ++q) d[r][q] = IO::get(w[r][q], 1);
                input_tile_transform<A>(d, hi);
            }
            const long long t = ((long long)n_l * a.bny + by) * a.bnx + bx;
            uint32_t* dst = vw + (t * a.cp + c) / VEC;
#pragma unroll
            for (int r = 0; r < A; ++r)
#pragma unroll
                for (int q = 0; q < A; ++q) dst[(long long)(r * A + q) * plane_words] = IO::put(lo[r][q], VEC == 2 ? hi[r][q] : 0.f);
        }
        __syncthreads();   // the slot is free for the load issued at the top of the next iteration
    }
    if (aborted && threadIdx.x == 0) drain_after_abort();
}

template <int A, typename TIn, typename TOp>
static int run_nhwc_tma(const wino_conv_desc& d, const Geometry& g, const ITArgs& a, cudaStream_t st) {
    constexpr int M = A - 2;
    constexpr int COLS = M * IT_TX + 2;
    constexpr int VEC = 4 / (int)sizeof(TIn);
    constexpr int CH = 32 * VEC;
    constexpr int SMEM = ITT_STAGES * A * COLS * 128 + 8 * ITT_STAGES + 16;
    CUtensorMap tm;
    const unsigned long long es = sizeof(TIn);
    const unsigned long long dims[4] = {(unsigned long long)d.c, (unsigned long long)d.w, (unsigned long long)d.h,
                                        (unsigned long long)d.n};
    const unsigned long long strides[3] = {d.c * es, (unsigned long long)d.w * d.c * es,
                                           (unsigned long long)d.h * d.w * d.c * es};
    const unsigned box[4] = {(unsigned)CH, (unsigned)COLS, (unsigned)A, 1u};
    int rc = encode_tensor_map(&tm, sizeof(TIn) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                               a.x, dims, strides, box, false);
    if (rc) return rc;
    int* status = nullptr;
    if ((rc = status_word(&status))) return rc;
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(input_transform_nhwc_tma<A, TIn, TOp>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    });
    WINO_CUDA_CHECK(attr_err);
    const int cchunks = (g.cp + CH - 1) / CH, bxchunks = (g.bnx + IT_TX - 1) / IT_TX;
    const long long units = (long long)a.ns * g.bny * bxchunks * cchunks;
    const long long max_ctas = 2LL * sm_count();
    ProfScope prof(STAGE_INPUT, st);
    count_launch();
    input_transform_nhwc_tma<A, TIn, TOp><<<(unsigned)(units < max_ctas ? units : max_ctas), 256, SMEM, st>>>(
        tm, a, bxchunks, cchunks, units, status);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

template <int A, typename TIn, typename TOp>
static int run(const wino_conv_desc& d, const Geometry& g, const ITArgs& a, cudaStream_t st) {
    static_assert(IT_TX * IT_CB == 256 && IT_NB * IT_CB == 256, "one work item per thread");
    if (d.layout_in == WINO_NHWC && (d.c * sizeof(TIn)) % 16 == 0 && ((uintptr_t)a.x & 15) == 0 && !force_generic())
        return run_nhwc_tma<A, TIn, TOp>(d, g, a, st);
    const int cchunks = (g.cp + IT_CB - 1) / IT_CB;
    ProfScope prof(STAGE_INPUT, st);
    count_launch();
    if (d.layout_in == WINO_CHWN) {
        dim3 grid((unsigned)(((a.ns + IT_NB - 1) / IT_NB) * cchunks), (unsigned)g.bnx, (unsigned)g.bny);
        input_transform_batch<A, TIn, TOp><<<grid, 256, 0, st>>>(a);
    } else {
        dim3 grid((unsigned)(((g.bnx + IT_TX - 1) / IT_TX) * cchunks), (unsigned)g.bny, (unsigned)a.ns);
        if (d.layout_in == WINO_NCHW)
            input_transform_strip<A, true, TIn, TOp><<<grid, 256, 0, st>>>(a);
        else
            input_transform_strip<A, false, TIn, TOp><<<grid, 256, 0, st>>>(a);
    }
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

template <int A>
static int dispatch(const wino_conv_desc& d, const Geometry& g, const ITArgs& a, cudaStream_t st) {
    switch (g.operand) {
        case OP_F32: return run<A, float, float>(d, g, a, st);
        case OP_TF32: return run<A, float, tf32_t>(d, g, a, st);
        case OP_BF16: return run<A, __nv_bfloat16, __nv_bfloat16>(d, g, a, st);
        case OP_F16: return run<A, __nv_bfloat16, __half>(d, g, a, st);
    }
    return fail(WINO_E_BADARG, "input transform: bad operand kind %d", g.operand);
}

int launch_input_transform(const wino_conv_desc& d, const Geometry& g, const void* x, int n0, int ns, void* v,
                           long long tp, cudaStream_t st) {
    if (ns <= 0) return WINO_OK;
    if (ns > 65535 || g.bny > 65535 || g.bnx > 65535)
        return fail(WINO_E_UNSUPPORTED, "input transform: slab of %d images / %dx%d tiles exceeds the grid limits", ns,
                    g.bny, g.bnx);
    ITArgs a;
    a.x = x; a.v = v; a.C = d.c; a.H = d.h; a.W = d.w; a.pad = d.pad;
    a.n0 = n0; a.ns = ns; a.bny = g.bny; a.bnx = g.bnx; a.cp = g.cp; a.tp = tp;
    a.sx = act_strides(d.layout_in, d.n, d.c, d.h, d.w);
    return g.a == 6 ? dispatch<6>(d, g, a, st) : dispatch<4>(d, g, a, st);
}

}  // namespace wino
